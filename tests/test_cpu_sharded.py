"""CPU tier for the sequence-sharded path: shard planning, the packed-buffer layout and the
exchange/merge orchestration of ShardedDecodeAttention, run as two gloo ranks with the oracle
standing in for the CUDA operators (so only host logic and the collective are under test)."""
from __future__ import annotations

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_plan():
    from tidaldecode_b200.sharded import ShardPlan, pack_layout, packed_floats

    p = ShardPlan.contiguous(10, 4)
    assert p.bounds == (0, 3, 6, 8, 10)
    assert [p.owner_of(i) for i in range(10)] == [0, 0, 0, 1, 1, 1, 2, 2, 3, 3]
    assert ShardPlan.contiguous(3, 8).bounds == (0, 1, 2, 3, 3, 3, 3, 3, 3)       # more ranks than tokens: empty shards
    with pytest.raises(ValueError):
        p.owner_of(10)
    L = pack_layout(4, 32, 128, 4, 128)
    assert L["total"] == packed_floats(4, 32, 128, 4, 128) == 4 * 32 * 130 + 2 * 4 * 128
    assert L["m"] == 0 and L["l"] == 128 and L["o"] == 256 and L["cs"] == 256 + 4 * 32 * 128


class _OracleOps:
    """The operator surface ShardedDecodeAttention uses, computed by the CPU oracle."""

    class Workspace:
        def __init__(self, *a, device="cpu"):
            self.hist = torch.zeros(a[3], 4096, dtype=torch.int32)

        def status(self):
            return 0

    @staticmethod
    def _dense(kv, n, B):
        # pool [B*n_alloc, 2, 1, Hkv, D] with identity page mapping -> K,V [B,Hkv,n,D]
        per = kv.shape[0] // B
        K = kv[:, 0, 0].view(B, per, *kv.shape[3:])[:, :n].permute(0, 2, 1, 3)
        V = kv[:, 1, 0].view(B, per, *kv.shape[3:])[:, :n].permute(0, 2, 1, 3)
        return K, V

    @classmethod
    def decode_attention(cls, q, kv, seq_len, ws, *, page_table=None, pages_per_seq=None, scores=None, hist=None,
                         partials=None, want_out=True, sel_idx=None, sel_counts=None, **kw):
        from oracle import tidal_oracle as O
        B = q.shape[0]
        K, V = cls._dense(kv, seq_len, B)
        qq = q[:, :, None, :]
        m, l, o = partials
        if sel_idx is None:
            if scores is not None:
                s = O.scores_fp32(qq, K, "sum" if scores.dim() == 2 else "none")
                scores[..., :seq_len] = s
            pm, pl, po = O.partial_attention(qq, K, V)
            m.copy_(pm * 1.4426950408889634); l.copy_(pl); o.copy_(po)
        else:
            for b in range(B):
                c = int(sel_counts[b])
                idx = sel_idx[b, :c].long()
                pm, pl, po = O.partial_attention(qq[b:b + 1], K[b:b + 1, :, idx], V[b:b + 1, :, idx])
                m[b] = pm[0] * 1.4426950408889634; l[b] = pl[0]; o[b] = po[0]
        return None

    @staticmethod
    def topk(scores, k, ws, *, n=None, in_idx=None, out_idx=None, out_val=None, idx_offset=0, own_range=None,
             out_count=None, hist=None, segments=None, **kw):
        if segments is not None:
            # element j of row r lives at (j // seg_len) * seg_stride + r * row_stride + j % seg_len
            nrows, seg_len, seg_stride, row_stride = segments
            j = torch.arange(n)
            off = (j // seg_len) * seg_stride + (j % seg_len)
            at = off[None, :] + torch.arange(nrows)[:, None] * row_stride
            scores = scores.reshape(-1)[at]
            in_idx = in_idx.reshape(-1)[at]
        rows = scores.reshape(-1, scores.shape[-1])
        n = rows.shape[1] if n is None else n
        kk = min(k, n)
        vals, pos = torch.topk(rows[:, :n], kk, dim=-1)
        pos, order = torch.sort(pos, dim=-1)
        vals = torch.gather(vals, 1, order)
        emit = torch.gather(in_idx.reshape(rows.shape[0], -1), 1, pos).to(torch.int32) if in_idx is not None \
            else (pos + idx_offset).to(torch.int32)
        oi = out_idx.reshape(rows.shape[0], -1)
        for r in range(rows.shape[0]):
            e = emit[r]
            if own_range is not None:
                keep = (e >= own_range[0]) & (e < own_range[1])
                e = e[keep] - own_range[0]
                if out_count is not None:
                    out_count.reshape(-1)[r] = e.numel()
            oi[r, : e.numel()] = e
            if out_val is not None:
                out_val.reshape(rows.shape[0], -1)[r, :kk] = vals[r]
        return out_idx

    @staticmethod
    def merge_partials(m, l, o, dtype, out=None, geometry=None):
        if geometry is not None:
            shards, B, Hq, D, stride = geometry
            pick = lambda t, cnt, shape: torch.stack([t.reshape(-1)[s * stride: s * stride + cnt].view(shape)
                                                      for s in range(shards)])
            m, l, o = pick(m, B * Hq, (B, Hq)), pick(l, B * Hq, (B, Hq)), pick(o, B * Hq * D, (B, Hq, D))
        M = m.max(dim=0).values
        w = torch.where(torch.isfinite(m), torch.exp2(m - M), torch.zeros_like(m))
        num = (w[..., None] * o).sum(0)
        den = (w * l).sum(0)
        res = (num / den[..., None]).to(dtype)
        out.copy_(res)
        return out


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import tidal_oracle as O
        from tidaldecode_b200.sharded import ShardedDecodeAttention, ShardPlan
        from tests.helpers import make_qkv

        B, Hq, Hkv, D, N, k = 2, 8, 2, 64, 301, 24
        q, K, V = make_qkv(7, B, Hq, Hkv, D, N, torch.float32, planted=6)
        plan = ShardPlan.contiguous(N, world)
        lo, hi = plan.range_of(rank)
        n = hi - lo
        pool = torch.zeros(B * n, 2, 1, Hkv, D)
        pool[:, 0, 0] = K[:, :, lo:hi].permute(0, 2, 1, 3).reshape(B * n, Hkv, D)
        pool[:, 1, 0] = V[:, :, lo:hi].permute(0, 2, 1, 3).reshape(B * n, Hkv, D)
        sh = ShardedDecodeAttention(B, Hq, Hkv, D, torch.float32, plan, rank, k, "sum", device="cpu", ops=_OracleOps)
        qd = q[:, :, 0].contiguous()
        o_sel = sh.selection_layer(qd, pool, pages_per_seq=n, want_global=True).clone()
        sel = sh.selected_global().clone()
        o_sp = sh.sparse_layer(qd, pool, pages_per_seq=n).clone()
        allidx = torch.arange(N, dtype=torch.int32)[None].expand(B, N)
        want_sel = O.gathered_attention(q, K, V, allidx)[:, :, 0]
        ok, why = O.topk_sets_match(O.scores_fp32(q, K, "sum"), sel, k, tie_band=1e-6)
        want_sp = O.gathered_attention(q, K, V, sel)[:, :, 0]
        res = dict(sel_ok=torch.allclose(o_sel, want_sel, rtol=1e-4, atol=1e-5), topk_ok=ok, why=why,
                   sp_ok=torch.allclose(o_sp, want_sp, rtol=1e-4, atol=1e-5), sel=sel,
                   owned=int(sh.sel_count.sum()))
        torch.save(res, os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_sharded_exchange_two_gloo_ranks(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    for r in res:
        assert r["sel_ok"], "merged selection-layer output differs from the unsharded oracle"
        assert r["topk_ok"], r["why"]
        assert r["sp_ok"], "merged sparse-layer output differs from the unsharded oracle"
    assert torch.equal(res[0]["sel"], res[1]["sel"]), "ranks disagree on the selected set"
    assert res[0]["owned"] + res[1]["owned"] == 2 * 24, "every selected position has exactly one owner"


def _leaving_worker(rank, world, port, result_dir):
    """Rank 1 leaves between steps; rank 0 learns of it on the host before its next launch, and — when it
    skips that check — its next collective ends with an error instead of hanging."""
    import datetime
    import time

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from tidaldecode_b200.sharded import GroupHealth, RankLost, ShardedDecodeAttention, ShardPlan
    from tests.helpers import make_qkv

    store = dist.distributed_c10d._get_default_store()
    health = GroupHealth(store, rank, world)
    B, Hq, Hkv, D, N, k = 1, 4, 2, 64, 90, 8
    q, K, V = make_qkv(3, B, Hq, Hkv, D, N, torch.float32)
    plan = ShardPlan.contiguous(N, world)
    lo, hi = plan.range_of(rank)
    n = hi - lo
    pool = torch.zeros(B * n, 2, 1, Hkv, D)
    pool[:, 0, 0] = K[:, :, lo:hi].permute(0, 2, 1, 3).reshape(B * n, Hkv, D)
    pool[:, 1, 0] = V[:, :, lo:hi].permute(0, 2, 1, 3).reshape(B * n, Hkv, D)
    sh = ShardedDecodeAttention(B, Hq, Hkv, D, torch.float32, plan, rank, k, "sum", device="cpu", ops=_OracleOps, health=health)
    qd = q[:, :, 0].contiguous()
    sh.selection_layer(qd, pool, pages_per_seq=n)              # step 0: everybody is there
    sh.sparse_layer(qd, pool, pages_per_seq=n)
    if rank == 1:
        health.leave()                                         # between steps, nothing in flight
        dist.destroy_process_group()
        return
    res = dict(noticed=False, collective_failed=False, seconds=None)
    deadline = time.time() + 20
    while time.time() < deadline:
        try:
            health.check()
            time.sleep(0.05)
        except RankLost:
            res["noticed"] = True
            break
    try:
        sh.selection_layer(qd, pool, pages_per_seq=n)          # with the check in place the launch never happens
    except RankLost:
        res["raised_before_launch"] = True
    sh.health = None                                           # a caller without the check: the collective must fail, not hang
    t0 = time.time()
    try:
        sh.selection_layer(qd, pool, pages_per_seq=n)
    except RankLost:
        raise
    except Exception as e:                                     # gloo: peer closed the connection, or the group timeout
        res["collective_failed"] = True
        res["error"] = type(e).__name__
    res["seconds"] = time.time() - t0
    torch.save(res, os.path.join(result_dir, "r0.pt"))
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_rank_leaving_between_steps_is_noticed_on_the_host(tmp_path):
    world = 2
    port = 29300 + (os.getpid() % 2000)
    mp.spawn(_leaving_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = torch.load(tmp_path / "r0.pt")
    assert res["noticed"] and res.get("raised_before_launch"), res
    assert res["collective_failed"], res
    assert res["seconds"] < 30, res


def test_peer_exchange_flags_are_independent_of_payload():
    """Every CTA of a rank publishes the NUMBER of the exchange in its own flag word, and a call waits for as many
    flags per rank as it has CTAs itself (all ranks launch the same grid for the same call).  So exchanges of
    different payloads and grids (selection layers send partials and candidates and rank them, sparse layers only
    partials) can follow each other in any order on one set of buffers: a model of the flag words over
    sel, sparse, sparse, sel, ... in which a flag left by an earlier, larger grid never satisfies a later wait."""
    from tidaldecode_b200 import _lib as L

    world, max_ctas = 4, L.XCHG_MAX_CTAS
    grids = {"sel": 25, "sparse": 9}                             # CTAs of the two kinds of call differ
    flags = [[[0] * max_ctas for _ in range(world)] for _ in range(2)]      # one rank's flag words [parity][source][CTA]
    epoch = 0
    for payload in ("sel", "sparse", "sparse", "sel", "sparse", "sel", "sel", "sparse", "sparse", "sparse"):
        e = epoch + 1
        par = e & 1
        g = grids[payload]
        assert g <= max_ctas
        # before anyone has published, no source rank's first g flags all show e (stale flags hold older numbers)
        assert not any(all(flags[par][r][c] - e >= 0 for c in range(g)) for r in range(world))
        for r in range(world):
            for c in range(g):
                flags[par][r][c] = e
        assert all(flags[par][r][c] - e >= 0 for r in range(world) for c in range(g))
        epoch = e
