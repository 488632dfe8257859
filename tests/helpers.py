"""Shared helpers of the GPU parity tests."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# BASELINE tolerance for attention outputs in fp16/bf16; fp32 is held tighter.
TOL = {torch.float16: dict(rtol=2e-3, atol=1e-2), torch.bfloat16: dict(rtol=2e-3, atol=1e-2),
       torch.float32: dict(rtol=1e-4, atol=1e-5)}


def make_qkv(seed, B, Hq, Hkv, D, N, dtype, planted=0):
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


def build_pool(K, V, page_size, shuffle_seed=None, spare_pages=3):
    """Dense K,V [B,Hkv,N,D] -> (pool [pages,2,page,Hkv,D], page_table int32 [B,ppb] or None).
    With shuffle_seed the pages are scattered over the pool; without, sequence b
    occupies pages [b*ppb, (b+1)*ppb)."""
    B, Hkv, N, D = K.shape
    ppb = (N + page_size - 1) // page_size
    total = B * ppb + (spare_pages if shuffle_seed is not None else 0)
    pool = torch.zeros(total, 2, page_size, Hkv, D, dtype=K.dtype)
    if shuffle_seed is not None:
        g = torch.Generator().manual_seed(shuffle_seed)
        perm = torch.randperm(total, generator=g)[: B * ppb].view(B, ppb)
    else:
        perm = torch.arange(B * ppb).view(B, ppb)
    Kp = torch.zeros(B, ppb * page_size, Hkv, D, dtype=K.dtype)
    Vp = torch.zeros_like(Kp)
    Kp[:, :N] = K.permute(0, 2, 1, 3)
    Vp[:, :N] = V.permute(0, 2, 1, 3)
    pool[perm.reshape(-1), 0] = Kp.view(B * ppb, page_size, Hkv, D)
    pool[perm.reshape(-1), 1] = Vp.view(B * ppb, page_size, Hkv, D)
    table = perm.to(torch.int32) if shuffle_seed is not None else None
    return pool, table, ppb


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name))
    return {k: z[k] for k in z.files}


def from_np(a, dtype):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype == torch.float32:
        return t
    return t.view(dtype)


def assert_close(got, want, dtype, what=""):
    tol = TOL[dtype]
    got, want = got.float().cpu(), want.float().cpu()
    ok = torch.allclose(got, want, **tol)
    if not ok:
        err = (got - want).abs()
        raise AssertionError(f"{what}: max abs err {err.max().item():.3e} "
                             f"(tol rtol={tol['rtol']} atol={tol['atol']}), at {int(err.argmax())}")
