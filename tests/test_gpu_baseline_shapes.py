"""GPU parity at the exact sizes of the benchmark configurations, through the C ABI, against
the CPU oracle: the kernels take other planner branches here than in the small cases of
test_gpu_kernels.py (a KV split over all SMs with a merge launch, whole stages in one bulk
copy, K|V of a token in one copy, the histogram hand-off to the top-k at 32 K - 1 M scores).

Inputs are the benchmark's own (tidaldecode_b200.workloads), generated on the device and read
back, so the oracle sees the bits the kernels read.  The reference-parity mode of configuration 2
(per-head sets) is covered against a fixture of the reference itself by
test_gpu_kernels.py::test_golden_reference_outputs[cfg2_f16_mha_32k].
"""
from __future__ import annotations

import os
import sys

import pytest
import torch

from oracle import tidal_oracle as O
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOG2E = 1.4426950408889634


def _inputs(name, lo, hi, device, context=None, seed=1000):
    """(w, q [B,Hq,D] on the host, pool on the device) for positions [lo,hi) of the workload's context."""
    from tidaldecode_b200 import workloads as WL

    w = dict(WL.WORKLOADS[name])
    if context is not None:
        w["planted"] = max(1, w["planted"] * context // w["N"])
        w["N"] = context
    dtype = getattr(torch, w["dtype"])
    q = WL.synth_queries(w, 1, seed=3)[0]
    pool = WL.synth_shard(w, lo, hi, seed, dtype, device)
    WL.plant(w, pool, q, lo, hi, seed=7)
    return w, q, pool


def _check_selection_and_sparse(T, w, q, pool, n, lo=0):
    """One selection pass + top-k + one sparse pass on the device; every sequence against the oracle."""
    from tidaldecode_b200 import workloads as WL

    B, Hq, D, k = w["B"], w["Hq"], w["D"], w["k"]
    dtype = pool.dtype
    ws = T.Workspace(B, Hq, D, B, n)
    qd = q.cuda()
    scores = torch.full((B, n), float("nan"), dtype=torch.float32, device="cuda")
    o_sel = T.decode_attention(qd, pool, n, ws, pages_per_seq=n, scores=scores, hist=ws.hist)
    idx = T.topk(scores, k, ws, hist=ws.hist, idx_offset=lo)
    local = (idx - lo).contiguous()
    o_sp = T.decode_attention(qd, pool, n, ws, pages_per_seq=n, sel_idx=local)
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert int(ws.hist.abs().sum()) == 0, "histogram must be left zeroed"
    for b in range(B):
        K, V = WL.dense_of_sequence(w, pool, b, n)
        qb = q[b:b + 1, :, None, :]
        want_o, want_s = O.attention_chunked(qb, K, V, "sum")
        assert_close(o_sel[b:b + 1], want_o, dtype, f"selection layer, sequence {b}")
        got_s = scores[b:b + 1].cpu()
        assert torch.allclose(got_s, want_s, rtol=1e-4, atol=2e-4 * Hq), (got_s - want_s).abs().max()
        ok, why = O.topk_sets_match(want_s, local[b:b + 1].cpu(), k, tie_band=1e-4)
        assert ok, f"sequence {b}: {why}"
        assert_close(o_sp[b:b + 1], O.gathered_attention_gqa(qb, K, V, local[b:b + 1].cpu()), dtype, f"sparse layer, sequence {b}")
    assert int(idx.min()) >= lo and int(idx.max()) < lo + n


@pytest.fixture(scope="module")
def T():
    import tidaldecode_b200.ops as ops
    return ops


def test_cfg2_verbatim_head_summed(T):
    """B=1, 32 x 128 MHA, fp16, context 32768, 64 planted keys, top_k 256, scores summed over heads."""
    w, q, pool = _inputs("cfg2", 0, 32768, "cuda")
    _check_selection_and_sparse(T, w, q, pool, 32768)


def test_cfg4_verbatim(T):
    """B=4, 32 q / 8 kv heads x 128, bf16, context 131072, top_k 128 (tensor-core kernel, K|V in one copy)."""
    w, q, pool = _inputs("cfg4", 0, 131072, "cuda")
    _check_selection_and_sparse(T, w, q, pool, 131072)


def test_cfg5_shard_of_eight(T):
    """What one of eight ranks holds of the 1 M-context workload: B=8, 64 q / 8 kv heads x 128, bf16,
    131072 positions [lo,hi) of every sequence, top_k 1024 with global positions."""
    lo = 3 * 131072
    w, q, pool = _inputs("cfg5", lo, lo + 131072, "cuda")
    _check_selection_and_sparse(T, w, q, pool, 131072, lo=lo)


# ------------------------------------------------------------------ the same through the sharded driver, 2 GPUs
def _sharded_worker(rank, world, port, result_dir, name, context):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from tidaldecode_b200 import workloads as WL
        from tidaldecode_b200.sharded import ShardedDecodeAttention, ShardPlan

        dev = torch.device("cuda", rank)
        plan = ShardPlan.contiguous(context, world)
        lo, hi = plan.range_of(rank)
        n = hi - lo
        w, q, pool = _inputs(name, lo, hi, dev, context=context, seed=1000 + rank)
        B, Hq, Hkv, D, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["k"]
        sh = ShardedDecodeAttention(B, Hq, Hkv, D, pool.dtype, plan, rank, k, "sum", device=dev, exchange="peer")
        qd = q.to(dev)
        for _ in range(2):                          # twice: buffers and counters are reused
            o_sel = sh.selection_layer(qd, pool, pages_per_seq=n).float().cpu()
            o_sp = sh.sparse_layer(qd, pool, pages_per_seq=n).float().cpu()
            o_sp2 = sh.sparse_layer(qd, pool, pages_per_seq=n).float().cpu()      # exchanges of different sizes in a row
        torch.cuda.synchronize()
        cnt = sh.sel_count.cpu()
        mine = [sh.sel_local[b, : int(cnt[b])].cpu().long() for b in range(B)]
        # oracle partials of this shard, all sequences
        sel_parts, sp_parts, sc = [], [], []
        for b in range(B):
            K, V = WL.dense_of_sequence(w, pool, b, n)
            qb = q[b:b + 1, :, None, :]
            part, s = O.attention_chunked(qb, K, V, "sum", return_partials=True)
            sc.append(s)
            sel_parts.append(part)
            sp_parts.append(O.partial_attention(qb, K[:, :, mine[b]], V[:, :, mine[b]]))
        torch.save(dict(o_sel=o_sel, o_sp=o_sp, o_sp2=o_sp2, mine=[m_ + lo for m_ in mine], scores=torch.cat(sc),
                        sel_parts=sel_parts, sp_parts=sp_parts, status=sh.ws.status() | sh.exchange_status()),
                   os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,context", [("cfg2", 32768), ("cfg4", 131072), ("cfg5", 262144)],
                         ids=["cfg2", "cfg4", "cfg5-shard-shape"])
def test_sharded_driver_at_benchmark_shapes(tmp_path, name, context):
    """ShardedDecodeAttention on two GPUs at the benchmark shapes (the third: the 1 M workload's heads, batch
    and top_k on a context whose per-rank share equals one of eight ranks' share of 1 M), peer-store exchange;
    the merged outputs and the union of the ranks' selected positions against the oracle's exact merge."""
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tidaldecode_b200 import workloads as WL

    world = 2
    port = 29900 + (os.getpid() % 2000)
    mp.spawn(_sharded_worker, args=(world, port, str(tmp_path), name, context), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    w = WL.WORKLOADS[name]
    B, k = w["B"], w["k"]
    dtype = getattr(torch, w["dtype"])
    scores = torch.cat([r["scores"] for r in res], dim=-1)              # [B, context]
    for b in range(B):
        want_sel = O.merge_partials([r["sel_parts"][b] for r in res])
        want_sp = O.merge_partials([r["sp_parts"][b] for r in res])
        chosen = torch.cat([r["mine"][b] for r in res])[None]
        ok, why = O.topk_sets_match(scores[b:b + 1], chosen, k, tie_band=1e-4)
        assert ok, f"sequence {b}: {why}"
        for r in res:
            assert r["status"] == 0
            assert_close(r["o_sel"][b:b + 1], want_sel, dtype, f"merged selection layer, sequence {b}")
            assert_close(r["o_sp"][b:b + 1], want_sp, dtype, f"merged sparse layer, sequence {b}")
            assert torch.equal(r["o_sp"], r["o_sp2"]), "a repeated sparse layer must reproduce its result"
