"""Times tidal_prefill on one causal prompt of synthetic values (the measurement that
kernels/src/bench/bench_batch_prefill.cu makes for the reference's kernel): CUDA events around
`--iters` launches after `--warmup`, one JSON line with ms per launch and TFLOP/s counted on the
causal half (2 * n * n * Hq * D flop).  `--sdpa` also times torch's fused attention on the same
tensors gathered into a dense layout, as the library figure to compare with.

    python -m tidaldecode_b200.bench_prefill --n 8192 --heads 32 --kv_heads 8 --dtype bf16
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=8192, help="prompt length (queries = cached tokens)")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv_heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=128)
    ap.add_argument("--page_size", type=int, default=1)
    ap.add_argument("--dtype", default="bf16", choices=["f16", "bf16"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--sdpa", action="store_true")
    a = ap.parse_args()
    dtype = torch.float16 if a.dtype == "f16" else torch.bfloat16
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    n_pages = (a.n + a.page_size - 1) // a.page_size
    pool = torch.randn(n_pages, 2, a.page_size, a.kv_heads, a.head_dim, device=dev, generator=g).to(dtype)
    table = torch.randperm(n_pages, device=dev, generator=g).to(torch.int32)      # pages in shuffled order
    q = torch.randn(a.n, a.heads, a.head_dim, device=dev, generator=g).to(dtype)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters

    ms = timed(lambda: ops.prefill(q, pool, table, a.n, out=out, status=status))
    flop = 2.0 * a.n * a.n * a.heads * a.head_dim
    line = {"op": "tidal_prefill", "n": a.n, "heads": a.heads, "kv_heads": a.kv_heads, "head_dim": a.head_dim,
            "page_size": a.page_size, "dtype": a.dtype, "ms": round(ms, 4), "tflops_causal": round(flop / ms / 1e9, 1),
            "status": int(status.item())}
    if a.sdpa:
        sel = pool[table.long()]
        K = sel[:, 0].reshape(-1, a.kv_heads, a.head_dim)[:a.n].transpose(0, 1)[None].contiguous()
        V = sel[:, 1].reshape(-1, a.kv_heads, a.head_dim)[:a.n].transpose(0, 1)[None].contiguous()
        qq = q.transpose(0, 1)[None]
        f = lambda: torch.nn.functional.scaled_dot_product_attention(qq, K, V, is_causal=True, enable_gqa=a.heads != a.kv_heads)
        ms2 = timed(f)
        ref = f()[0].transpose(0, 1)
        line.update({"sdpa_ms": round(ms2, 4), "sdpa_tflops_causal": round(flop / ms2 / 1e9, 1),
                     "max_abs_diff_vs_sdpa": float((out.float() - ref.float()).abs().max())})
    print(json.dumps(line))


if __name__ == "__main__":
    main()
