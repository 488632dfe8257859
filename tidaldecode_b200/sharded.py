"""Sequence-sharded decode attention: the KV cache of every layer is split by
position across the ranks of one process group; each rank runs the kernels on
its shard and one packed all-gather per layer makes the result exact.

    selection layer   local attention -> (m, l, o) partials + local top-k
                      candidates (score, global position); all-gather; every rank
                      merges the partials and picks the global top-k from the
                      g*k candidates, keeping the positions it owns;
    sparse layer      local attention over the owned selected positions ->
                      partials; all-gather; merge.

The reference has no multi-GPU path; the merge is the one it uses across KV
chunks inside one GPU (kernels/include/decode/decode_attn.cuh:213-232,
VariableLengthMergeStates :1012-1020), applied across ranks.  Exactness: the
selection score is the raw logit, so the global top-k is contained in the union
of the shard-local top-k sets; softmax partials merge associatively.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    """Contiguous position ranges: rank r owns [bounds[r], bounds[r+1])."""
    world: int
    seq_len: int
    bounds: Tuple[int, ...]

    @staticmethod
    def contiguous(seq_len: int, world: int) -> "ShardPlan":
        base, rem = divmod(seq_len, world)
        b = [0]
        for r in range(world):
            b.append(b[-1] + base + (1 if r < rem else 0))
        return ShardPlan(world, seq_len, tuple(b))

    def range_of(self, rank: int) -> Tuple[int, int]:
        return self.bounds[rank], self.bounds[rank + 1]

    def owner_of(self, pos: int) -> int:
        for r in range(self.world):
            if self.bounds[r] <= pos < self.bounds[r + 1]:
                return r
        raise ValueError(f"position {pos} outside [0, {self.seq_len})")


def packed_floats(batch: int, hq: int, d: int, rows: int, k: int) -> int:
    """fp32 words one rank contributes per layer: m, l, o, candidate scores, candidate
    positions (int32 bit patterns) — one buffer, one collective."""
    return batch * hq * (d + 2) + 2 * rows * k


def pack_layout(batch: int, hq: int, d: int, rows: int, k: int):
    """Offsets (in fp32 words) of the regions inside one rank's packed buffer."""
    o_m = 0
    o_l = o_m + batch * hq
    o_o = o_l + batch * hq
    o_cs = o_o + batch * hq * d
    o_ci = o_cs + rows * k
    return dict(m=o_m, l=o_l, o=o_o, cs=o_cs, ci=o_ci, total=o_ci + rows * k)


class ShardedDecodeAttention:
    """Per-rank driver of the kernels for one (batch, heads, context) geometry."""

    def __init__(self, batch: int, hq: int, hkv: int, d: int, dtype: torch.dtype, plan: ShardPlan, rank: int,
                 top_k: int, head_reduce: str = "sum", group: Optional[dist.ProcessGroup] = None, device="cuda",
                 ops=None):
        if ops is None:
            from . import ops  # the CUDA library; raises if it is missing (tests of the exchange logic inject a stand-in)

        self.ops = ops
        self.B, self.Hq, self.Hkv, self.D, self.dtype = batch, hq, hkv, d, dtype
        self.plan, self.rank, self.k, self.group = plan, rank, top_k, group
        self.world = plan.world
        self.lo, self.hi = plan.range_of(rank)
        self.local_len = self.hi - self.lo
        if head_reduce not in ("sum", "none"):
            raise ValueError(head_reduce)
        self.rows_per_seq = 1 if head_reduce == "sum" else hq
        self.rows = batch * self.rows_per_seq
        self.k_local = min(top_k, max(self.local_len, 1))
        self.k_global = min(top_k, plan.seq_len)
        L = pack_layout(batch, hq, d, self.rows, top_k)
        self.layout = L
        self.ws = ops.Workspace(batch, hq, d, self.rows, max(self.local_len, self.world * top_k, 1), device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.send = torch.zeros(L["total"], **f32)
        self.recv = torch.zeros(self.world, L["total"], **f32)
        self.scores = torch.empty((batch, max(self.local_len, 1)) if head_reduce == "sum"
                                  else (batch, hq, max(self.local_len, 1)), **f32)
        self.gm = torch.empty(self.world, batch, hq, **f32)
        self.gl = torch.empty(self.world, batch, hq, **f32)
        self.go = torch.empty(self.world, batch, hq, d, **f32)
        self.cand_s = torch.empty(self.rows, self.world * top_k, **f32)
        self.cand_i = torch.empty(self.rows, self.world * top_k, dtype=torch.int32, device=device)
        self.sel_local = torch.zeros(self.rows, top_k, dtype=torch.int32, device=device)
        self.sel_count = torch.zeros(self.rows, dtype=torch.int32, device=device)
        self.sel_global = torch.zeros(self.rows, top_k, dtype=torch.int32, device=device)
        self.out = torch.empty(batch, hq, d, dtype=dtype, device=device)

    # views into the send buffer
    def _send_views(self):
        L, B, Hq, D, R, k = self.layout, self.B, self.Hq, self.D, self.rows, self.k
        s = self.send
        return (s[L["m"]:L["l"]].view(B, Hq), s[L["l"]:L["o"]].view(B, Hq), s[L["o"]:L["cs"]].view(B, Hq, D),
                s[L["cs"]:L["ci"]].view(R, k), s[L["ci"]:L["total"]].view(torch.int32).view(R, k))

    def _all_gather(self):
        if self.world == 1:
            self.recv[0].copy_(self.send)
        else:
            dist.all_gather_into_tensor(self.recv.view(-1), self.send, group=self.group)

    def _unpack_partials(self):
        L, B, Hq, D = self.layout, self.B, self.Hq, self.D
        r = self.recv
        self.gm.copy_(r[:, L["m"]:L["l"]].reshape(self.world, B, Hq))
        self.gl.copy_(r[:, L["l"]:L["o"]].reshape(self.world, B, Hq))
        self.go.copy_(r[:, L["o"]:L["cs"]].reshape(self.world, B, Hq, D))

    def selection_layer(self, q: torch.Tensor, kv_local: torch.Tensor, pages_per_seq: Optional[int] = None,
                        page_table: Optional[torch.Tensor] = None, want_global: bool = False) -> torch.Tensor:
        """q [B,Hq,D]; kv_local: this rank's pool holding positions [lo, hi) of every sequence."""
        ops, k = self.ops, self.k
        m, l, o, cs, ci = self._send_views()
        cs.fill_(-float("inf"))
        ci.zero_()
        if self.local_len > 0:
            ops.decode_attention(q, kv_local, self.local_len, self.ws, page_table=page_table, pages_per_seq=pages_per_seq,
                                 scores=self.scores, hist=self.ws.hist[: self.rows], partials=(m, l, o), want_out=False)
            ops.topk(self.scores, k, self.ws, n=self.local_len, out_idx=ci, out_val=cs, idx_offset=self.lo,
                     hist=self.ws.hist[: self.rows])
        else:
            m.fill_(-float("inf"))
            l.zero_()
            o.zero_()
        self._all_gather()
        self._unpack_partials()
        ops.merge_partials(self.gm, self.gl, self.go, self.dtype, out=self.out)
        L, R = self.layout, self.rows
        # [world][rows][k] -> [rows][world*k]
        self.cand_s.view(R, self.world, k).copy_(self.recv[:, L["cs"]:L["ci"]].reshape(self.world, R, k).permute(1, 0, 2))
        self.cand_i.view(R, self.world, k).copy_(
            self.recv[:, L["ci"]:L["total"]].view(torch.int32).reshape(self.world, R, k).permute(1, 0, 2))
        # global set (for callers that want it) and the part of it this rank owns
        if want_global:
            ops.topk(self.cand_s, self.k_global, self.ws, in_idx=self.cand_i, out_idx=self.sel_global)
        ops.topk(self.cand_s, self.k_global, self.ws, in_idx=self.cand_i, out_idx=self.sel_local,
                 own_range=(self.lo, max(self.hi, self.lo + 1)) if self.local_len > 0 else (self.lo, self.lo + 1),
                 out_count=self.sel_count)
        if self.local_len == 0:
            self.sel_count.zero_()
        return self.out

    def sparse_layer(self, q: torch.Tensor, kv_local: torch.Tensor, pages_per_seq: Optional[int] = None,
                     page_table: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops = self.ops
        m, l, o, _, _ = self._send_views()
        sel = self.sel_local.view(self.B, self.k) if self.rows_per_seq == 1 else self.sel_local.view(self.B, self.Hq, self.k)
        cnt = self.sel_count.view(self.B) if self.rows_per_seq == 1 else self.sel_count.view(self.B, self.Hq)
        ops.decode_attention(q, kv_local, max(self.local_len, 1), self.ws, page_table=page_table, pages_per_seq=pages_per_seq,
                             sel_idx=sel, sel_counts=cnt, partials=(m, l, o), want_out=False)
        self._all_gather()
        self._unpack_partials()
        return ops.merge_partials(self.gm, self.gl, self.go, self.dtype, out=self.out)

    def selected_global(self) -> torch.Tensor:
        """[B, k] or [B, Hq, k] global positions chosen by the last selection layer."""
        s = self.sel_global[:, : self.k_global]
        return s.view(self.B, -1) if self.rows_per_seq == 1 else s.view(self.B, self.Hq, -1)
