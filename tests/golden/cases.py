"""Seeded inputs of the golden attention cases.

The fixtures hold the reference's OUTPUTS plus a digest of the inputs; the inputs
themselves are regenerated from the seed by `make_case` (torch's CPU generator),
and a test that finds a different digest fails instead of comparing.
"""
from __future__ import annotations

import hashlib

import torch


def input_digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        h.update(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.float32 else t.numpy().tobytes())
    return h.hexdigest()


def make_case(seed, B, Hq, Hkv, D, N, k, dtype, planted=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, 1, D, generator=g)
    K = torch.randn(B, Hkv, N, D, generator=g)
    V = torch.randn(B, Hkv, N, D, generator=g)
    if planted:
        G = Hq // Hkv
        for b in range(B):
            pos = torch.randperm(N, generator=g)[:planted]
            for h in range(Hkv):
                qh = q[b, h * G, 0]
                K[b, h, pos] = 3.0 * qh / qh.norm() + 0.1 * torch.randn(planted, D, generator=g)
    return q.to(dtype), K.to(dtype), V.to(dtype)


ATTN_CASES = [
    # name, seed, B, Hq, Hkv, D, N, k, dtype, planted
    ("f32_mha_d64", 11, 1, 4, 4, 64, 300, 16, torch.float32, 0),
    ("f32_mha_d128", 12, 2, 4, 4, 128, 257, 32, torch.float32, 8),
    ("f16_mha_d128", 13, 1, 8, 8, 128, 1111, 64, torch.float16, 16),
    ("bf16_gqa4_d128", 14, 2, 8, 2, 128, 600, 32, torch.bfloat16, 8),
    ("f16_gqa8_d128", 15, 1, 16, 2, 128, 515, 128, torch.float16, 8),
    ("f32_k_ge_n", 16, 1, 4, 4, 64, 20, 128, torch.float32, 0),
    ("f16_mha_d64", 17, 1, 4, 4, 64, 777, 48, torch.float16, 4),
    # the single-layer benchmark configuration verbatim: Llama-2-7B attention shape, context 32768,
    # 64 planted keys 3*q/|q| + N(0,0.1), top_k 256 (per-q-head sets, as the reference selects)
    ("cfg2_f16_mha_32k", 2, 1, 32, 32, 128, 32768, 256, torch.float16, 64),
]
