"""Sequence-sharded KV on real GPUs: one process per GPU, NCCL all-gather, CUDA kernels.
Needs at least two GPUs (skipped otherwise; the single-GPU emulation of the same protocol
is tests/test_gpu_kernels.py::test_sharded_partials_merge)."""
from __future__ import annotations

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_dir, reduce, exchange):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import tidal_oracle as O
        from tidaldecode_b200.sharded import ShardedDecodeAttention, ShardPlan
        from tests.helpers import make_qkv

        B, Hq, Hkv, D, N, k = 2, 32, 8, 128, 5001, 128
        dtype = torch.bfloat16
        q, K, V = make_qkv(11, B, Hq, Hkv, D, N, dtype, planted=32)
        plan = ShardPlan.contiguous(N, world)
        lo, hi = plan.range_of(rank)
        n = hi - lo
        pool = torch.zeros(B * n, 2, 1, Hkv, D, dtype=dtype)
        pool[:, 0, 0] = K[:, :, lo:hi].permute(0, 2, 1, 3).reshape(B * n, Hkv, D)
        pool[:, 1, 0] = V[:, :, lo:hi].permute(0, 2, 1, 3).reshape(B * n, Hkv, D)
        pool = pool.cuda()
        sh = ShardedDecodeAttention(B, Hq, Hkv, D, dtype, plan, rank, k, reduce, device=torch.device("cuda", rank),
                                    exchange=exchange)
        assert (sh.peer is not None) == (exchange == "peer")
        qd = q[:, :, 0].contiguous().cuda()
        res = {}
        for rep in range(3):                       # several times: buffers and counters must be reusable
            o_sel = sh.selection_layer(qd, pool, pages_per_seq=n, want_global=True).float().cpu()
            sel = sh.selected_global().cpu()
            o_sp = sh.sparse_layer(qd, pool, pages_per_seq=n).float().cpu()
        torch.cuda.synchronize()
        allidx = torch.arange(N, dtype=torch.int32)[None].expand(B, N)
        want_sel = O.gathered_attention(q, K, V, allidx)[:, :, 0]
        rows = B if reduce == "sum" else B * Hq
        ok, why = O.topk_sets_match(O.scores_fp32(q, K, reduce).reshape(rows, N), sel.reshape(rows, -1), k, tie_band=1e-4)
        want_sp = O.gathered_attention(q, K, V, sel)[:, :, 0]
        res = dict(sel_err=float((o_sel - want_sel).abs().max()), topk_ok=ok, why=why,
                   sp_err=float((o_sp - want_sp).abs().max()), sel=sel, status=sh.ws.status() | sh.exchange_status())
        torch.save(res, os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,exchange", [(2, "nccl"), (2, "peer"), (4, "peer"), (4, "nccl"), (8, "peer")],
                         ids=["2-nccl", "2-peer", "4-peer", "4-nccl", "8-peer"])
@pytest.mark.parametrize("reduce", ["sum", "none"])
def test_sharded_ranks(tmp_path, reduce, world, exchange):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path), reduce, exchange), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    for r in res:
        assert r["status"] == 0
        assert r["sel_err"] < 1e-2, r["sel_err"]
        assert r["topk_ok"], r["why"]
        assert r["sp_err"] < 1e-2, r["sp_err"]
        assert torch.equal(r["sel"], res[0]["sel"]), "ranks disagree on the selected set"
