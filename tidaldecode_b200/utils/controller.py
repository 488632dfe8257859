"""Decode-step state (mirror of tidal/utils/controller.py:8-193).

Same constructor arguments, attributes and methods as the reference's
InferenceController, but everything is allocated once here: `begin_forward`
only moves scalars and re-slices views (the reference re-uploads the page list,
re-allocates and re-zeroes its score and top-k buffers and re-plans the KV split
on every call, four times per token: controller.py:93-177, llama.py:505-520).

Extensions, all optional: grouped-query heads (`num_kv_heads`), a batch of
sequences in lockstep (`batch_size`), how selection scores are reduced
(`head_reduce`: "none" keeps one top-k set per query head as both reference
paths do; "sum" adds the logits of all query heads and keeps one shared set),
whether the newest token is always kept (`force_last_token`, the kernel-path
rule: decode_page.cuh:326-341, controller.py:140-147), and `layer_alias` to
share one KV buffer among that many layers (the reference hard-wires 4:
kv_cache.py:84,117; here 1 = no sharing).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _kernels, ops
from .decode_wrapper import BatchDecodeWithPagedKVCacheWrapper
from .kv_cache import KvCache
from .utils import TensorLayout


class InferenceController:
    def __init__(self, num_layers, num_heads, head_dim, page_size, token_budget, max_seq_len, dtype, device,
                 num_kv_heads: Optional[int] = None, batch_size: int = 1, head_reduce: str = "none",
                 force_last_token: bool = True, layer_alias: int = 1, quest_metadata: bool = False,
                 metadata_page_size: int = 16):
        assert page_size == 1, "Only support page_size=1"
        if head_reduce not in ("none", "sum"):
            raise ValueError("head_reduce must be 'none' or 'sum'")
        num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.kv_cache = KvCache(num_layers=num_layers, num_heads=num_kv_heads, head_dim=head_dim, max_seq_len=max_seq_len,
                                page_size=page_size, dtype=dtype, device=device, layer_alias=layer_alias,
                                batch_size=batch_size)
        # The reference always allocates a second pool for Quest's per-page min/max of the keys
        # (controller.py:31-39); no TidalDecode layer reads it, so it exists only on request
        # (quest_metadata=True: append_kv keeps it up to date, decode_estimate reads it).  One entry per KV
        # page, metadata_page_size entries per metadata page, sequence b's pages at [b * per_seq, ...).
        self.metadata_cache = None
        if quest_metadata:
            kv_pages = (max_seq_len + page_size - 1) // page_size
            per_seq = (kv_pages + metadata_page_size - 1) // metadata_page_size
            self.metadata_cache = torch.zeros((max(1, num_layers // layer_alias), per_seq * batch_size, 2, metadata_page_size,
                                               num_kv_heads, head_dim), dtype=dtype, device=device)
        self.layout = TensorLayout.NHD
        self.device = device
        self.dtype = dtype

        self.num_layers = num_layers
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.page_size = page_size
        self.max_seq_len = max_seq_len
        self.batch_size = batch_size
        self.head_reduce = head_reduce
        self.force_last_token = force_last_token

        self._token_budget = token_budget
        self._decode_handler = BatchDecodeWithPagedKVCacheWrapper(kv_layout="NHD")

        rows_per_seq = 1 if head_reduce == "sum" else num_heads
        self.score_rows = rows_per_seq
        rows = batch_size * rows_per_seq
        self.workspace = ops.Workspace(batch_size, num_heads, head_dim, rows, max_seq_len, device=device)
        # the per-head page-list form of the attention call (BatchDecodeWithPagedKVCacheWrapper) shares it
        _kernels.adopt_workspace(self.workspace)
        shape = (batch_size, max_seq_len) if head_reduce == "sum" else (batch_size, num_heads, max_seq_len)
        # fp32 logits of the last selection layer; column = token position
        self.qk_product = torch.empty(shape, dtype=torch.float32, device=device)
        self._max_budget = min(int(token_budget), max_seq_len)
        idx_shape = (batch_size, self._max_budget) if head_reduce == "sum" else (batch_size, num_heads, self._max_budget)
        self._topk_indices_full = torch.zeros(idx_shape, dtype=torch.int32, device=device)
        self._topk_values_full = torch.zeros(idx_shape, dtype=torch.float32, device=device)
        # valid entries per selection list (= the step's budget for every list), refilled when the budget changes
        self._counts_full = torch.full((rows,), self._max_budget, dtype=torch.int32, device=device)
        self._counts_value = self._max_budget
        self.topk_buf = None                       # the reference's RAFT scratch; the workspace replaces it

        self.kv_indices_with_last = None
        self.kv_indices_with_last_decode = None
        self.kv_indices_without_last = None
        self.metadata_indices = None
        self.kv_last_page_idx = None
        self.metadata_last_page_idx = None
        self.kv_indptr_for_append = None
        self.metadata_indptr_for_append = None
        self.kv_indptr_for_approx_decode = None
        self.inference_token_budget = None
        self.topk_dout_buffer = None
        self.topk_dindices_buffer = None
        self._selection_valid = False

        self.prefill_latency = []
        self.decode_latency = []

    # Used for controlling the number of pages (reference: skips the first layers by raising it)
    def set_token_budget(self, token_budget: int):
        self._token_budget = token_budget

    def prepare_metadata(self, seq_len: int):
        """Reserve page slots for seq_len new tokens per sequence (controller.py:81-85)."""
        self.kv_cache.append_seq(seq_len)
        self._selection_valid = False            # a new token invalidates the previous step's set

    def begin_forward(self, seq_len: int, updateTensor: bool = True):
        """Refresh the per-step views (controller.py:93-177); allocates nothing."""
        cur_pages = self.kv_cache.num_pages
        table = self.kv_cache.page_table
        self.kv_last_page_idx = self.kv_cache.indicies[-1]
        self.kv_indices_with_last = table[0, :cur_pages]
        if seq_len > 1:
            return
        assert cur_pages > 1  # at least two pages for excluding last page
        self.kv_indices_with_last_decode = self.kv_indices_with_last
        self.kv_indices_without_last = table[0, : cur_pages - 1]
        self.inference_token_budget = min(self._token_budget, cur_pages, self._max_budget)
        b = self.inference_token_budget
        self.topk_dindices_buffer = self._topk_indices_full[..., :b]
        self.topk_dout_buffer = self._topk_values_full[..., :b]
        if b != self._counts_value:
            self._counts_full.fill_(b)
            self._counts_value = b
        # as the reference does every step (controller.py:170-177); the scratch is in place already unless
        # another controller's smaller workspace was adopted on this device since
        self._decode_handler.begin_forward(None, self.num_heads, self.num_kv_heads, self.head_dim, self.page_size, self.dtype,
                                           max_pages=0, device=self.device)

    def end_forward(self):
        self._decode_handler.end_forward()

    def need_estimate(self) -> bool:
        if self.inference_token_budget is None:
            return False
        return self.kv_cache.seqlen > self.inference_token_budget

    def clean_states(self):
        self.kv_cache.release()
        self._selection_valid = False
