"""Paged KV pool and per-sequence page lists (mirror of tidal/utils/kv_cache.py:8-137).

One tensor [layers, capacity, 2, page_size, kv_heads, head_dim]; a layer's slice is
what the kernels call "the pool".  Unlike the reference, every logical layer has
its own buffer unless `layer_alias` > 1 asks for the reference's memory trick of
sharing one buffer among several layers (kv_cache.py:84,117 hard-wires 4).
Page ids are handed out lowest-first, so a sequence that is never interleaved
with another occupies consecutive pages; the device-side page table is kept in
step with the host list by copying only the entries that were added.
"""
from __future__ import annotations

import torch

from .utils import TensorLayout


class KvPool:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, capacity: int, block_len: int,
                 dtype: torch.dtype, device: torch.device):
        self._layout = TensorLayout.NHD
        self._buf = torch.empty((num_layers, capacity, 2, block_len, num_heads, head_dim), dtype=dtype, device=device)
        self._free = list(range(capacity - 1, -1, -1))    # pop() hands out the lowest id

    @property
    def layout(self):
        return self._layout

    @property
    def buf(self):
        return self._buf

    @property
    def num_layers(self):
        return self._buf.shape[0]

    @property
    def block_len(self):
        return self._buf.shape[3]

    @property
    def num_free_blocks(self):
        return len(self._free)

    @property
    def capacity(self):
        return self._buf.shape[1]

    def alloc_block(self) -> int:
        if not self._free:
            raise RuntimeError("KV pool exhausted: raise max_seq_len")
        return self._free.pop()

    def free_block(self, idx: int):
        self.free_blocks([idx])

    def free_blocks(self, ids):
        for idx in ids:
            assert 0 <= idx < self.capacity
        self._free.extend(ids)
        self._free.sort(reverse=True)


class KvCache:
    """Key-value cache of `batch_size` sequences that grow in lockstep."""

    def __init__(self, num_layers, num_heads, head_dim, max_seq_len: int, page_size, dtype: torch.dtype,
                 device: torch.device, layer_alias: int = 1, batch_size: int = 1):
        if max_seq_len <= 0:
            raise ValueError("max_seq_len must be positive")
        if layer_alias < 1:
            raise ValueError("layer_alias must be >= 1")
        self.batch_size = batch_size
        self._pages_per_seq = (max_seq_len + page_size - 1) // page_size
        self._pool = KvPool(num_layers=max(1, num_layers // layer_alias), num_heads=num_heads, head_dim=head_dim,
                            capacity=self._pages_per_seq * batch_size, block_len=page_size, dtype=dtype, device=device)
        self._indicies = [[] for _ in range(batch_size)]
        self._seqlen = 0
        self.device = device
        # device page table [batch, pages_per_seq] and its pinned staging row
        self.page_table = torch.zeros((batch_size, self._pages_per_seq), dtype=torch.int32, device=device)
        self._stage = torch.zeros((batch_size, self._pages_per_seq), dtype=torch.int32).pin_memory() \
            if torch.device(device).type == "cuda" else torch.zeros((batch_size, self._pages_per_seq), dtype=torch.int32)
        self._synced = 0          # pages per sequence already on the device

    @property
    def pool(self) -> KvPool:
        return self._pool

    @property
    def seqlen(self) -> int:
        return self._seqlen

    @property
    def last_page_len(self) -> int:
        return (self.seqlen - 1) % self._pool.block_len + 1

    @property
    def indicies(self):
        """Page ids in use by sequence 0 (the reference's only sequence)."""
        return self._indicies[0][: self.num_pages]

    @property
    def num_pages(self) -> int:
        """Pages in use by the current sequence length (reserved pages beyond it are not counted)."""
        return (self._seqlen + self._pool.block_len - 1) // self._pool.block_len

    def buf_layer(self, layer_idx: int):
        return self._pool.buf[layer_idx % self._pool.num_layers]

    def _ensure_pages(self, n_pages: int) -> int:
        """Allocate until every sequence owns n_pages pages; extends the device page table by the new entries."""
        added = 0
        while len(self._indicies[0]) < n_pages:
            for b in range(self.batch_size):
                self._indicies[b].append(self._pool.alloc_block())
            added += 1
        if added:
            n0, n1 = self._synced, len(self._indicies[0])
            for b in range(self.batch_size):
                self._stage[b, n0:n1] = torch.tensor(self._indicies[b][n0:n1], dtype=torch.int32)
            self.page_table[:, n0:n1].copy_(self._stage[:, n0:n1], non_blocking=True)
            self._synced = n1
        return added

    def reserve(self, total_tokens: int) -> None:
        """Own the pages for `total_tokens` tokens per sequence now, so that later appends touch neither the
        allocator nor the page table (a decode step replayed as a CUDA graph needs exactly that)."""
        self._ensure_pages((total_tokens + self._pool.block_len - 1) // self._pool.block_len)

    def append_seq(self, seq_len: int) -> int:
        """Make room for seq_len more tokens per sequence; returns pages added per sequence."""
        if seq_len <= 0:
            return 0
        self._seqlen += seq_len
        return self._ensure_pages(self.num_pages)

    def release(self):
        self._seqlen = 0
        for b in range(self.batch_size):
            self._pool.free_blocks(self._indicies[b])
            self._indicies[b].clear()
        self._synced = 0
