"""Per-kernel breakdown of ONE rank's part of a sequence-sharded decode step, on one GPU.

    python -m tidaldecode_b200.bench_rank_step <cfg2|cfg4|cfg5> <world>

Times, each alone (back-to-back launches on distinct layer pools replayed as a CUDA graph), the kernels that
`ShardedDecodeAttention` issues on a rank that holds 1/world of the workload's context: the rank-local selection
attention, the rank-local top-k, the sparse attention over the owned selected positions, RoPE + append, and the
exchange launch in its two forms (selection layer: all-gather + merge + candidate ranking; sparse layer:
all-gather + merge).  The exchange runs on buffers looped back onto this GPU with the other ranks' flags preset,
so that no wait blocks and nothing crosses NVLink: what is timed is the kernel's own cost.  Prints one JSON line.
"""
from __future__ import annotations

import json
import sys

import torch


def main(name: str, world: int) -> dict:
    from . import ops as T
    from . import workloads as WL
    from .sharded import pack_layout

    w = WL.WORKLOADS[name]
    dtype = getattr(torch, w["dtype"])
    B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
    n = N // world
    dev = torch.device("cuda", torch.cuda.current_device())
    npool = max(2, min(8, int(3e8 // (2 * B * n * Hkv * D * 2)) + 2))       # enough pools that L2 cannot serve repeats
    pools = [WL.synth_shard(w, 0, n, 10 + i, dtype, dev) for i in range(npool)]
    q = torch.randn(B, Hq, D, device=dev).to(dtype)
    ws = T.Workspace(B, Hq, D, B, max(n, world * k), device=dev)
    L = pack_layout(B, Hq, D, B, k)
    tot = (L["total"] + 3) // 4 * 4
    send = torch.zeros(tot, device=dev)
    m, l, o = send[L["m"]:L["l"]].view(B, Hq), send[L["l"]:L["o"]].view(B, Hq), send[L["o"]:L["cs"]].view(B, Hq, D)
    cs, ci = send[L["cs"]:L["ci"]].view(B, k), send[L["ci"]:L["ci"] + B * k].view(torch.int32).view(B, k)
    scores = torch.empty(B, n, device=dev)
    kn, vn = torch.randn(B, Hkv, D, device=dev).to(dtype), torch.randn(B, Hkv, D, device=dev).to(dtype)
    qrot = torch.empty_like(q)
    own_idx = (torch.arange(B * k, device=dev, dtype=torch.int32).view(B, k) * 7) % n
    own_cnt = torch.full((B,), max(1, k // world), dtype=torch.int32, device=dev)

    def t_us(fn, reps=None, iters=10):
        reps = reps or npool
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps):
                fn(i % npool)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return round(a.elapsed_time(b) * 1e3 / (reps * iters), 2)

    def attn_topk(i):
        T.decode_attention(q, pools[i], n, ws, pages_per_seq=n, scores=scores, hist=ws.hist[:B], partials=(m, l, o), want_out=False)
        T.topk(scores, k, ws, n=n, out_idx=ci, out_val=cs, idx_offset=0, hist=ws.hist[:B])

    def attn(i):
        T.decode_attention(q, pools[i], n, ws, pages_per_seq=n, partials=(m, l, o), want_out=False)

    def sparse(i):
        T.decode_attention(q, pools[i], n, ws, pages_per_seq=n, sel_idx=own_idx, sel_counts=own_cnt, partials=(m, l, o), want_out=False)

    def rope(i):
        T.rope_append(qrot, kn, vn, pools[i], batch=B, pos0=n - 1, pages_per_seq=n, rope_mode=2, rotate_k_in_place=False, q_src=q)

    res = dict(workload=name, world=world, tokens_per_rank=n,
               selection_attention_plus_topk=t_us(attn_topk), full_attention=t_us(attn),
               sparse_attention_partials=t_us(sparse, reps=8), rope_append=t_us(rope, reps=8),
               attention_at_copy_rate_us=round(2 * B * n * Hkv * D * 2 / 6539.2e3, 2))
    if world >= 2:
        px = T.PeerExchange.loopback(tot * 4, world, dev)
        px.flags.fill_(1 << 30)                                   # every other rank "has arrived" at any exchange
        blocks = torch.randn(world, tot, device=dev)
        for r in range(world):
            pos = torch.stack([torch.sort(torch.randperm(n)[:k]).values for _ in range(B)]) + r * n
            blocks[r, L["ci"]:L["ci"] + B * k] = pos.to(torch.int32).view(torch.float32).reshape(-1).to(dev)
            px.stage[0, r].copy_(blocks[r].view(torch.uint8))
            px.stage[1, r].copy_(blocks[r].view(torch.uint8))
        snd = blocks[0].contiguous()
        out = torch.empty(B * Hq, D, dtype=dtype, device=dev)
        sel, cnt = torch.zeros(B, k, dtype=torch.int32, device=dev), torch.zeros(B, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        merge = (out, L["m"], L["l"], L["o"])
        cand = dict(rows=B, k=k, select=min(k, N), score_off=L["cs"], idx_off=L["ci"], own=(0, n), out=sel, count=cnt)
        res["exchange_selection_layer"] = t_us(lambda i: px.all_gather(snd, None, status=status, merge=merge, candidates=cand), reps=20)
        res["exchange_sparse_layer"] = t_us(lambda i: px.all_gather(snd, None, nbytes=(L["cs"] + 3) // 4 * 16, status=status, merge=merge), reps=20)
        res["exchange_bytes_per_rank"] = tot * 4
        res["exchange_status"] = int(status.item())
    res["status"] = ws.status()
    return res


if __name__ == "__main__":
    print(json.dumps(main(sys.argv[1], int(sys.argv[2]))))
