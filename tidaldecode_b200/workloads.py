"""Seeded synthetic inputs of the benchmark configurations (shapes, sizes and value
distributions of the decode-attention workloads; no dataset, no checkpoint).

    cfg2  one Llama-2-7B attention layer: B=1, 32 heads x 128 MHA, fp16, context 32768,
          K,V ~ N(0,1) plus 64 planted keys 3*q/|q| + N(0,0.1), top_k 256
    cfg4  Llama-3-8B attention shape: B=4, 32 q / 8 kv heads x 128, bf16, context 131072, top_k 128
    cfg5  long-context stress: B=8, 64 q / 8 kv heads x 128, bf16, context 1048576,
          1 % planted keys, top_k 1024

The KV of a rank is written straight into a paged pool [B*n, 2, 1, Hkv, D] on the device
(page_size 1, sequence b at pages [b*n, (b+1)*n)), n = the positions the rank holds.  The
benchmark and the parity tests at these sizes build their inputs here, so that what is timed
is what is checked.
"""
from __future__ import annotations

import torch

WORKLOADS = {
    "cfg2": dict(B=1, Hq=32, Hkv=32, D=128, dtype="float16", N=32768, k=256, planted=64, layer_pairs=4),
    "cfg4": dict(B=4, Hq=32, Hkv=8, D=128, dtype="bfloat16", N=131072, k=128, planted=64, layer_pairs=2),
    "cfg5": dict(B=8, Hq=64, Hkv=8, D=128, dtype="bfloat16", N=1048576, k=1024, planted=10486, layer_pairs=1),
}


def describe(name: str) -> str:
    w = WORKLOADS[name]
    return (f"{name}: selection layer + sparse layer, B={w['B']}, {w['Hq']}q/{w['Hkv']}kv heads x {w['D']}, "
            f"context {w['N']}, top_k {w['k']}, head-summed scores")


def synth_queries(w: dict, layers: int, seed: int = 1) -> torch.Tensor:
    """q ~ N(0,1) for `layers` layers: [layers, B, Hq, D] in the workload's dtype, on the host."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(layers, w["B"], w["Hq"], w["D"], generator=g).to(getattr(torch, w["dtype"]))


def synth_shard(w: dict, lo: int, hi: int, seed: int, dtype: torch.dtype, device) -> torch.Tensor:
    """K,V ~ N(0,1) for positions [lo,hi) of every sequence, written straight into a pool
    [B*(hi-lo), 2, 1, Hkv, D] on the device; planted keys are added by `plant`."""
    B, Hkv, D = w["B"], w["Hkv"], w["D"]
    n = hi - lo
    g = torch.Generator(device=device).manual_seed(seed)
    pool = torch.empty(B * max(n, 1), 2, 1, Hkv, D, dtype=dtype, device=device)
    step = 1 << 16
    flat = pool.view(B * max(n, 1), -1)
    for s in range(0, flat.shape[0], step):
        e = min(flat.shape[0], s + step)
        flat[s:e] = torch.randn(e - s, flat.shape[1], generator=g, device=device, dtype=torch.float32).to(dtype)
    return pool


def plant(w: dict, pool: torch.Tensor, q: torch.Tensor, lo: int, hi: int, seed: int) -> None:
    """Planted positions: K[p,h,:] = 3*q_h/|q_h| + N(0,0.1), positions from a seeded randperm
    over the whole context; only those inside [lo,hi) are written (q [B,Hq,D])."""
    B, Hq, Hkv, N = w["B"], w["Hq"], w["Hkv"], w["N"]
    G = Hq // Hkv
    g = torch.Generator().manual_seed(seed)
    for b in range(B):
        pos = torch.randperm(N, generator=g)[: w["planted"]]
        noise = 0.1 * torch.randn(w["planted"], Hkv, w["D"], generator=g)
        mine = (pos >= lo) & (pos < hi)
        if not bool(mine.any()):
            continue
        qh = q[b, ::G].float().cpu()                                    # first q head of each KV head
        rows = 3.0 * qh / qh.norm(dim=-1, keepdim=True)                 # [Hkv, D]
        vals = (rows[None] + noise[mine]).to(pool.dtype).to(pool.device)
        idx = (b * (hi - lo) + (pos[mine] - lo)).to(pool.device)
        pool[idx, 0, 0] = vals


def dense_of_sequence(w: dict, pool: torch.Tensor, b: int, n: int):
    """K,V [1,Hkv,n,D] of sequence b of a pool built by `synth_shard`, on the host (the bits the
    kernels read, for a checker)."""
    rows = pool[b * n:(b + 1) * n, :, 0]                                 # [n, 2, Hkv, D]
    K = rows[:, 0].permute(1, 0, 2)[None].contiguous().cpu()
    V = rows[:, 1].permute(1, 0, 2)[None].contiguous().cpu()
    return K, V
