"""Times tidal_topk alone on rows shaped like the long-context workloads' logits (a sum over heads of N(0,1) scores,
optionally with 1 % planted keys far above the rest), no histogram handed in, and checks the set against torch.topk.

    python -m tidaldecode_b200.bench_topk [--rows 8] [--k 1024]

CUDA events around graph replays of 8 back-to-back calls; one JSON line with µs per call for rows of 1 M, 512 K and
128 K scores.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops as T


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--k", type=int, default=1024)
    a = ap.parse_args()
    rows, k = a.rows, a.k
    res = {}
    for n in (1 << 20, 1 << 19, 1 << 17):
        g = torch.Generator(device="cuda").manual_seed(1)
        s = torch.randn(rows, n, device="cuda", generator=g) * 8
        planted = torch.rand(rows, n, device="cuda", generator=g) < 0.01
        s = torch.where(planted, 24 + torch.randn(rows, n, device="cuda", generator=g), s)
        ws = T.Workspace(rows, 1, 64, rows, n)
        idx = torch.zeros(rows, k, dtype=torch.int32, device="cuda")

        def t_us(fn, reps=8, iters=10):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(reps):
                    fn()
            gr.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            return round(e0.elapsed_time(e1) * 1e3 / (reps * iters), 2)

        with_planted = t_us(lambda: T.topk(s, k, ws, out_idx=idx))
        want = torch.topk(s, k, dim=-1).indices.sort(dim=-1).values.int()
        exact = bool(torch.equal(idx.sort(dim=-1).values, want))
        rnd = torch.randn(rows, n, device="cuda") * 8
        random_only = t_us(lambda: T.topk(rnd, k, ws, out_idx=idx))
        res[n] = dict(planted_us=with_planted, random_us=random_only, exact=exact, status=ws.status())
    print(json.dumps({"op": "tidal_topk", "rows": rows, "k": k, "by_row_length": res}))


if __name__ == "__main__":
    main()
