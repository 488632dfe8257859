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


class RankLost(RuntimeError):
    """A rank of the sharded group announced that it is leaving; its shard of the KV is gone."""


class GroupHealth:
    """Host-side liveness of a sharded group over the process group's key-value store.

    A rank leaves only between steps, with none of its kernels or collectives in flight: it calls
    `leave()`; the others call `check()` before they launch their next step and get `RankLost`
    instead of a collective that can never complete.  (A rank that dies without saying so is caught
    by the next collective's timeout: the process-group timeout for NCCL/gloo, the bounded device-side
    wait — TIDAL_DEV_WAIT_TIMEOUT — for the peer-store exchange.)"""

    def __init__(self, store, rank: int, world: int, prefix: str = "tidal/health"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/left/{r}"

    def leave(self) -> None:
        self.store.set(self._key(self.rank), b"1")

    def check(self) -> None:
        for r in range(self.world):
            if r != self.rank and self.store.check([self._key(r)]):
                raise RankLost(f"rank {r} has left the group")


# largest group the peer-store exchange has run on; larger groups get NCCL unless exchange="peer" is asked for
kPeerValidatedWorld = 8


class ShardedDecodeAttention:
    """Per-rank driver of the kernels for one (batch, heads, context) geometry."""

    def __init__(self, batch: int, hq: int, hkv: int, d: int, dtype: torch.dtype, plan: ShardPlan, rank: int,
                 top_k: int, head_reduce: str = "sum", group: Optional[dist.ProcessGroup] = None, device="cuda",
                 ops=None, exchange: str = "auto", health: Optional[GroupHealth] = None):
        """exchange: "peer" = tidal_peer_all_gather (NVLink peer stores from this library's own kernel),
        "nccl" = one all_gather_into_tensor per layer, "auto" = peer for groups of up to kPeerValidatedWorld
        CUDA ranks where symmetric memory can be set up, else nccl."""
        if ops is None:
            from . import ops  # the CUDA library; raises if it is missing (tests of the exchange logic inject a stand-in)

        self.ops = ops
        self.health = health           # checked on the host before every layer's launches, if given
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
        L["total"] = (L["total"] + 3) // 4 * 4             # blocks start on 16-byte boundaries in the receive buffer
        self.layout = L
        self.ws = ops.Workspace(batch, hq, d, self.rows, max(self.local_len, self.world * top_k, 1), device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.send = torch.zeros(L["total"], **f32)
        self.recv = torch.zeros(self.world, L["total"], **f32)
        self.scores = torch.empty((batch, max(self.local_len, 1)) if head_reduce == "sum"
                                  else (batch, hq, max(self.local_len, 1)), **f32)
        self.sel_local = torch.zeros(self.rows, top_k, dtype=torch.int32, device=device)
        self.sel_count = torch.zeros(self.rows, dtype=torch.int32, device=device)
        self.sel_global = torch.zeros(self.rows, top_k, dtype=torch.int32, device=device)
        self.out = torch.empty(batch, hq, d, dtype=dtype, device=device)
        # views of rank 0's block inside the receive buffer: the merge and the candidate top-k read
        # all ranks' blocks in place, L["total"] words apart
        flat = self.recv.view(-1)
        self._rm, self._rl, self._ro = flat[L["m"]:], flat[L["l"]:], flat[L["o"]:]
        self._rcs, self._rci = flat[L["cs"]:], flat.view(torch.int32)[L["ci"]:]
        self._partial_geom = (self.world, batch, hq, d, L["total"])
        # one rank: its block is the whole row, plain addressing (and k == n selects everything)
        self._cand_segments = (self.rows, top_k, L["total"], top_k) if self.world > 1 else None
        if self.world == 1:
            self._rcs = self._rcs[: self.rows * top_k].view(self.rows, top_k)
            self._rci = self._rci[: self.rows * top_k].view(self.rows, top_k)
        self.peer = None
        # "auto" takes the peer exchange up to the world size it has been validated on (kPeerValidatedWorld)
        use_peer = exchange == "peer" or (exchange == "auto" and self.world <= kPeerValidatedWorld)
        if self.world > 1 and use_peer and hasattr(ops, "PeerExchange") and torch.device(device).type == "cuda":
            try:
                self.peer = ops.PeerExchange(L["total"] * 4, group if group is not None else dist.group.WORLD, torch.device(device))
                self._xstatus = torch.zeros(1, dtype=torch.int32, device=device)
            except Exception:
                if exchange == "peer":
                    raise
                self.peer = None
        if self.local_len < top_k:
            # fewer local tokens than candidates: the unused slots stay at -inf / 0 for good
            _, _, _, cs, ci = self._send_views()
            cs.fill_(-float("inf"))
            ci.zero_()

    # views into the send buffer
    def _send_views(self):
        L, B, Hq, D, R, k = self.layout, self.B, self.Hq, self.D, self.rows, self.k
        s = self.send
        return (s[L["m"]:L["l"]].view(B, Hq), s[L["l"]:L["o"]].view(B, Hq), s[L["o"]:L["cs"]].view(B, Hq, D),
                s[L["cs"]:L["ci"]].view(R, k), s[L["ci"]:L["total"]].view(torch.int32).view(R, k))

    def _all_gather(self, words: Optional[int] = None, rank_candidates: bool = False, want_recv: bool = True) -> bool:
        """Every rank's packed block into recv; `words`: only the leading fp32 words are needed (sparse layers
        exchange the partials, not the candidate lists, and need no receive buffer).  True if the exchange also
        merged the partials into self.out and — with rank_candidates — ranked the candidates into
        sel_local / sel_count (the peer-store kernel does both in its one launch)."""
        if self.world == 1:
            self.recv[0].copy_(self.send)
        elif self.peer is not None:
            L = self.layout
            n = L["total"] if words is None else (words + 3) // 4 * 4
            cand = None
            if rank_candidates:
                cand = dict(rows=self.rows, k=self.k, select=self.k_global, score_off=L["cs"], idx_off=L["ci"],
                            own=(self.lo, max(self.hi, self.lo + 1)), out=self.sel_local, count=self.sel_count)
            self.peer.all_gather(self.send, self.recv if (words is None and want_recv) else None, nbytes=n * 4,
                                 status=self._xstatus, merge=(self.out.view(-1, self.D), L["m"], L["l"], L["o"]),
                                 candidates=cand)
            return True
        else:
            dist.all_gather_into_tensor(self.recv.view(-1), self.send, group=self.group)
        return False

    @property
    def _fused_ranking(self) -> bool:
        """The peer-store kernel ranks the candidates itself when they fit its shared-memory form."""
        return self.peer is not None and self.k_global <= 2048 and self.world * self.k <= 65536 and self.k_global < self.world * self.k

    def exchange_status(self) -> int:
        """Fault bits of the peer exchange (0 when the library all-gather is in use)."""
        return int(self._xstatus.item()) if self.peer is not None else 0

    def selection_layer(self, q: torch.Tensor, kv_local: torch.Tensor, pages_per_seq: Optional[int] = None,
                        page_table: Optional[torch.Tensor] = None, want_global: bool = False,
                        timing: Optional[list] = None) -> torch.Tensor:
        """q [B,Hq,D]; kv_local: this rank's pool holding positions [lo, hi) of every sequence.
        timing: a list that receives a (start, end) CUDA-event pair around the local attention."""
        ops, k = self.ops, self.k
        if self.health is not None:
            self.health.check()
        m, l, o, cs, ci = self._send_views()
        if self.local_len > 0:
            if timing is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            ops.decode_attention(q, kv_local, self.local_len, self.ws, page_table=page_table, pages_per_seq=pages_per_seq,
                                 scores=self.scores, hist=self.ws.hist[: self.rows], partials=(m, l, o), want_out=False)
            if timing is not None:
                e1.record()
                timing.append((e0, e1))
            ops.topk(self.scores, k, self.ws, n=self.local_len, out_idx=ci, out_val=cs, idx_offset=self.lo,
                     hist=self.ws.hist[: self.rows])
        else:
            m.fill_(-float("inf"))
            l.zero_()
            o.zero_()
        fused = self._fused_ranking
        if not self._all_gather(rank_candidates=fused, want_recv=want_global or not fused):
            ops.merge_partials(self._rm, self._rl, self._ro, self.dtype, out=self.out, geometry=self._partial_geom)
        # global top-k of the world*k candidates, read in place; keep the positions this rank owns
        n_cand = self.world * k
        if want_global:          # the whole global set, for callers that inspect it (the layers only need the owned part)
            ops.topk(self._rcs, self.k_global, self.ws, n=n_cand, in_idx=self._rci, out_idx=self.sel_global,
                     segments=self._cand_segments)
        if not fused:
            ops.topk(self._rcs, self.k_global, self.ws, n=n_cand, in_idx=self._rci, out_idx=self.sel_local,
                     own_range=(self.lo, max(self.hi, self.lo + 1)), out_count=self.sel_count, segments=self._cand_segments)
        if self.local_len == 0:
            self.sel_count.zero_()
        return self.out

    def sparse_layer(self, q: torch.Tensor, kv_local: torch.Tensor, pages_per_seq: Optional[int] = None,
                     page_table: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops = self.ops
        if self.health is not None:
            self.health.check()
        m, l, o, _, _ = self._send_views()
        sel = self.sel_local.view(self.B, self.k) if self.rows_per_seq == 1 else self.sel_local.view(self.B, self.Hq, self.k)
        cnt = self.sel_count.view(self.B) if self.rows_per_seq == 1 else self.sel_count.view(self.B, self.Hq)
        ops.decode_attention(q, kv_local, max(self.local_len, 1), self.ws, page_table=page_table, pages_per_seq=pages_per_seq,
                             sel_idx=sel, sel_counts=cnt, partials=(m, l, o), want_out=False)
        if not self._all_gather(words=self.layout["cs"]):
            ops.merge_partials(self._rm, self._rl, self._ro, self.dtype, out=self.out, geometry=self._partial_geom)
        return self.out

    def selected_global(self) -> torch.Tensor:
        """[B, k] or [B, Hq, k] global positions chosen by the last selection layer."""
        s = self.sel_global[:, : self.k_global]
        return s.view(self.B, -1) if self.rows_per_seq == 1 else s.view(self.B, self.Hq, -1)
