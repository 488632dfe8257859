"""GPU parity: the sm_100a kernels, called through the C ABI, against the CPU
oracle and against the fixtures the reference produced (tests/golden)."""
from __future__ import annotations

import pytest
import torch

from oracle import tidal_oracle as O
from tests.golden.cases import ATTN_CASES, input_digest, make_case
from tests.helpers import assert_close, build_pool, from_np, load_golden, make_qkv

pytestmark = pytest.mark.gpu

DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


@pytest.fixture(scope="module")
def T():
    import tidaldecode_b200.ops as ops
    return ops


def _ws(T, B, Hq, D, rows, n):
    return T.Workspace(B, Hq, D, rows, n)


def _run_full(T, q, K, V, page_size, shuffle, **kw):
    B, Hq, _, D = q.shape
    N = K.shape[2]
    pool, table, ppb = build_pool(K, V, page_size, shuffle_seed=7 if shuffle else None)
    ws = _ws(T, B, Hq, D, B * Hq, N)
    o = T.decode_attention(q[:, :, 0].contiguous().cuda(), pool.cuda(), N, ws,
                           page_table=None if table is None else table.cuda(), pages_per_seq=ppb, **kw)
    torch.cuda.synchronize()
    assert ws.status() == 0
    return o, ws


FULL_CASES = [
    # dtype, B, Hq, Hkv, D, N, page_size, shuffle, chunks
    ("f16", 1, 32, 32, 128, 4099, 1, False, 0),
    ("f16", 1, 32, 32, 128, 63, 1, True, 0),
    ("f16", 1, 32, 32, 128, 1, 1, False, 0),
    ("f16", 1, 8, 8, 128, 2000, 16, True, 0),
    ("f16", 2, 8, 8, 64, 1110, 7, True, 3),
    ("bf16", 4, 32, 8, 128, 1500, 1, False, 0),
    ("bf16", 2, 16, 2, 128, 777, 3, True, 5),
    ("bf16", 1, 64, 8, 128, 3000, 1, False, 0),
    ("f16", 1, 16, 8, 128, 513, 1, False, 2),
    ("f32", 1, 4, 4, 64, 2055, 1, False, 0),
    ("f32", 2, 4, 4, 128, 300, 1, True, 0),
    ("f16", 1, 64, 64, 128, 600, 1, False, 0),
    ("f16", 1, 4, 1, 128, 127, 1, False, 0),
]


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,N,page,shuffle,chunks", FULL_CASES)
def test_full_attention(T, dt, B, Hq, Hkv, D, N, page, shuffle, chunks):
    dtype = DT[dt]
    q, K, V = make_qkv(100 + N, B, Hq, Hkv, D, N, dtype)
    o, _ = _run_full(T, q, K, V, page, shuffle, num_chunks=chunks)
    want = O.gathered_attention(q, K, V, torch.arange(N, dtype=torch.int32)[None].expand(B, N))
    assert_close(o, want[:, :, 0], dtype, "full attention")


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,N,page", [
    ("f16", 1, 32, 32, 128, 4099, 1), ("bf16", 2, 32, 8, 128, 1029, 1), ("f32", 1, 4, 4, 64, 700, 1),
    ("f16", 2, 8, 8, 64, 333, 4), ("bf16", 1, 64, 8, 128, 2048, 1),
])
@pytest.mark.parametrize("reduce", ["sum", "none"])
def test_selection_scores(T, dt, B, Hq, Hkv, D, N, page, reduce):
    """Logits written by the selection layer equal q.k/sqrt(D) of the stored inputs."""
    dtype = DT[dt]
    q, K, V = make_qkv(200 + N, B, Hq, Hkv, D, N, dtype, planted=8)
    shape = (B, N) if reduce == "sum" else (B, Hq, N)
    scores = torch.full(shape, float("nan"), dtype=torch.float32, device="cuda")
    o, _ = _run_full(T, q, K, V, page, True, scores=scores)
    want = O.scores_fp32(q, K, reduce)
    tol = 2e-4 * (Hq if reduce == "sum" else 1)
    assert torch.allclose(scores.cpu(), want, rtol=1e-4, atol=tol), (scores.cpu() - want).abs().max()
    full = O.gathered_attention(q, K, V, torch.arange(N, dtype=torch.int32)[None].expand(B, N))
    assert_close(o, full[:, :, 0], dtype, "selection layer output")


PATH_CASES = [
    # dtype, B, Hq, Hkv, D, N, page
    ("f16", 1, 32, 32, 128, 1500, 1),     # MHA forced onto tensor cores (4 head slices)
    ("bf16", 2, 32, 8, 128, 2049, 1),
    ("f16", 1, 64, 8, 128, 1000, 1),
    ("bf16", 1, 16, 2, 64, 777, 3),
    ("f16", 2, 16, 1, 128, 300, 1),       # MQA, 16 query heads on one KV head
    ("bf16", 1, 8, 4, 128, 17, 1),
    ("f16", 1, 24, 12, 64, 500, 2),       # 12 KV heads: slices of 4
]


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,N,page", PATH_CASES)
@pytest.mark.parametrize("tc", [1, -1])
def test_tensor_core_and_cuda_core_paths(T, dt, B, Hq, Hkv, D, N, page, tc):
    """Both kernels, forced, on full / selection (per-head logits) / sparse layers."""
    if tc < 0 and Hq // Hkv > 8:
        pytest.skip("the CUDA-core kernel is built for up to 8 query heads per KV head")
    dtype = DT[dt]
    q, K, V = make_qkv(400 + N, B, Hq, Hkv, D, N, dtype, planted=4)
    pool, table, ppb = build_pool(K, V, page, shuffle_seed=5)
    ws = _ws(T, B, Hq, D, B * Hq, N)
    qd, pd, td = q[:, :, 0].contiguous().cuda(), pool.cuda(), table.cuda()
    scores = torch.full((B, Hq, N), float("nan"), dtype=torch.float32, device="cuda")
    o = T.decode_attention(qd, pd, N, ws, page_table=td, scores=scores, use_tensor_cores=tc)
    allidx = torch.arange(N, dtype=torch.int32)[None].expand(B, N)
    assert_close(o, O.gathered_attention(q, K, V, allidx)[:, :, 0], dtype, "full")
    want = O.scores_fp32(q, K, "none")
    assert torch.allclose(scores.cpu(), want, rtol=1e-4, atol=2e-4), (scores.cpu() - want).abs().max()
    if Hkv in (1, 2, 4, 8, 16, 32):
        ssum = torch.full((B, N), float("nan"), dtype=torch.float32, device="cuda")
        T.decode_attention(qd, pd, N, ws, page_table=td, scores=ssum, use_tensor_cores=tc if Hkv <= 8 else -1)
        assert torch.allclose(ssum.cpu(), want.sum(1), rtol=1e-4, atol=2e-4 * Hq)
    g = torch.Generator().manual_seed(N)
    k = min(48, N)
    shared = torch.stack([torch.randperm(N, generator=g)[:k] for _ in range(B)]).to(torch.int32)
    o = T.decode_attention(qd, pd, N, ws, page_table=td, sel_idx=shared.cuda(), use_tensor_cores=tc)
    assert_close(o, O.gathered_attention(q, K, V, shared)[:, :, 0], dtype, "shared list")
    per_head = torch.stack([torch.stack([torch.randperm(N, generator=g)[:k] for _ in range(Hq)]) for _ in range(B)]).to(torch.int32)
    o = T.decode_attention(qd, pd, N, ws, page_table=td, sel_idx=per_head.cuda(), use_tensor_cores=tc)
    assert_close(o, O.gathered_attention(q, K, V, per_head)[:, :, 0], dtype, "per-head lists")
    torch.cuda.synchronize()
    assert ws.status() == 0


def test_tensor_core_request_is_refused_where_it_cannot_run(T):
    q, K, V = make_qkv(1, 1, 4, 4, 64, 50, torch.float32)
    pool, _, ppb = build_pool(K, V, 1)
    ws = _ws(T, 1, 4, 64, 4, 50)
    with pytest.raises(RuntimeError):
        T.decode_attention(q[:, :, 0].contiguous().cuda(), pool.cuda(), 50, ws, pages_per_seq=ppb, use_tensor_cores=1)


TOPK_CASES = [
    # rows, n, k
    (1, 32768, 256), (32, 4099, 256), (4, 131072, 128), (2, 1000, 1), (3, 1000, 999), (3, 1000, 1000),
    (3, 1000, 5000), (1, 63, 16), (8, 50000, 1024), (2, 17, 16), (1, 300000, 4096), (1, 20000, 8192),
]


@pytest.mark.parametrize("rows,n,k", TOPK_CASES)
def test_topk_random(T, rows, n, k):
    g = torch.Generator().manual_seed(n + k)
    s = torch.randn(rows, n, generator=g)
    ws = _ws(T, 1, 1, 64, rows, n)
    idx = T.topk(s.cuda(), k, ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    ok, why = O.topk_sets_match(s, idx.cpu(), k, tie_band=0.0)
    assert ok, why
    if min(k, n) <= 4096:
        assert bool((idx[:, 1:] > idx[:, :-1]).all()), "indices must ascend"
    # the counters are zero at rest: a second call on the same workspace agrees
    idx2 = T.topk(s.cuda(), k, ws)
    assert torch.equal(torch.sort(idx, -1).values, torch.sort(idx2, -1).values)


@pytest.mark.parametrize("rows,n,k", [(2, 200000, 1000), (1, 1 << 20, 1024), (3, 70000, 2048)])
def test_topk_crowded_threshold_bin(T, rows, n, k):
    """Thousands of keys share the threshold bin (quantised scores, and a planted 1 % of
    near-equal high scores as in the long-context configuration): more candidates than fit
    in shared memory."""
    g = torch.Generator().manual_seed(n)
    s = torch.round(torch.randn(rows, n, generator=g) * 2) / 2
    hot = torch.randperm(n, generator=g)[: n // 100]
    s[:, hot] = 40.0 + 0.001 * torch.randn(rows, hot.numel(), generator=g)
    ws = _ws(T, 1, 1, 64, rows, n)
    idx = T.topk(s.cuda(), k, ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    ok, why = O.topk_sets_match(s, idx.cpu(), k, tie_band=0.0)
    assert ok, why
    # ties resolve towards the lower position: the result is exactly torch's stable descending sort prefix
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(torch.sort(idx.cpu().long(), -1).values, torch.sort(order, -1).values)


def test_topk_ties_and_values(T):
    """All-equal rows and heavy ties resolve towards the lower index; values are returned."""
    n, k = 5000, 100
    ws = _ws(T, 1, 1, 64, 4, n)
    s = torch.zeros(4, n)
    s[1] = torch.randint(0, 3, (n,)).float()           # three distinct values
    s[2, 1234] = 5.0
    s[3] = -torch.arange(n).float()
    val = torch.empty(4, k, device="cuda")
    idx = T.topk(s.cuda(), k, ws, out_val=val).cpu()
    assert ws.status() == 0
    assert torch.equal(idx[0], torch.arange(k, dtype=torch.int32))
    twos = torch.nonzero(s[1] == 2).flatten()[:k].to(torch.int32)
    assert torch.equal(idx[1], twos)
    assert 1234 in idx[2].tolist() and set(idx[2].tolist()) == set(range(k - 1)) | {1234}
    assert torch.equal(idx[3], torch.arange(k, dtype=torch.int32))
    assert torch.equal(val.cpu(), torch.gather(s, 1, idx.long()))


def test_topk_special_values(T):
    n, k = 3000, 10
    ws = _ws(T, 1, 1, 64, 1, n)
    s = torch.randn(1, n)
    s[0, 5] = float("inf")
    s[0, 6] = -float("inf")
    s[0, 7] = -0.0
    s[0, 8] = 1e-42          # denormal
    idx = T.topk(s.cuda(), k, ws).cpu()
    assert ws.status() == 0
    ok, why = O.topk_sets_match(s, idx, k, tie_band=0.0)
    assert ok, why
    assert 5 in idx[0].tolist() and 6 not in idx[0].tolist()


def test_topk_force_last_offset_in_idx_own(T):
    n, k = 2000, 64
    g = torch.Generator().manual_seed(5)
    s = torch.randn(2, n, generator=g)
    ws = _ws(T, 1, 1, 64, 2, n)
    idx = T.topk(s.cuda(), k, ws, force_last=True).cpu()
    ok, why = O.topk_sets_match(s, idx, k, tie_band=0.0, force_last=True)
    assert ok, why
    base = torch.sort(T.topk(s.cuda(), k, ws).cpu(), -1).values
    off = torch.sort(T.topk(s.cuda(), k, ws, idx_offset=1000).cpu(), -1).values
    assert torch.equal(off, base + 1000)
    remap = torch.randperm(n, generator=g).to(torch.int32)[None].expand(2, n).contiguous()
    got = T.topk(s.cuda(), k, ws, in_idx=remap.cuda()).cpu()
    assert torch.equal(torch.sort(got, -1).values, torch.sort(torch.gather(remap, 1, base.long()), -1).values)
    cnt = torch.zeros(2, dtype=torch.int32, device="cuda")
    own = T.topk(s.cuda(), k, ws, own_range=(500, 1500), out_count=cnt).cpu()
    for r in range(2):
        want = base[r][(base[r] >= 500) & (base[r] < 1500)] - 500
        assert int(cnt[r]) == want.numel()
        assert torch.equal(own[r, : want.numel()], want)
    assert ws.status() == 0


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,N,k,page", [
    ("f16", 1, 32, 32, 128, 4099, 256, 1), ("bf16", 2, 32, 8, 128, 3000, 128, 1), ("f32", 1, 4, 4, 64, 2055, 128, 1),
    ("f16", 1, 8, 8, 128, 500, 16, 16), ("bf16", 1, 64, 8, 128, 5000, 1024, 1), ("f16", 2, 8, 2, 64, 900, 33, 5),
])
@pytest.mark.parametrize("reduce", ["sum", "none"])
def test_select_then_sparse(T, dt, B, Hq, Hkv, D, N, k, page, reduce):
    """Selection layer (+ fused first-digit histogram) -> top-k -> sparse layer."""
    dtype = DT[dt]
    q, K, V = make_qkv(300 + N, B, Hq, Hkv, D, N, dtype, planted=min(64, k // 2))
    pool, table, ppb = build_pool(K, V, page, shuffle_seed=3)
    rows = B if reduce == "sum" else B * Hq
    ws = _ws(T, B, Hq, D, rows, N)
    shape = (B, N) if reduce == "sum" else (B, Hq, N)
    scores = torch.empty(shape, dtype=torch.float32, device="cuda")
    qd, pd, td = q[:, :, 0].contiguous().cuda(), pool.cuda(), table.cuda()
    T.decode_attention(qd, pd, N, ws, page_table=td, scores=scores, hist=ws.hist)
    idx = T.topk(scores, k, ws, hist=ws.hist)
    assert int(ws.hist.abs().sum()) == 0, "histogram must be left zeroed"
    want_scores = O.scores_fp32(q, K, reduce)
    ok, why = O.topk_sets_match(want_scores.reshape(rows, N), idx.reshape(rows, -1).cpu(), k, tie_band=1e-4)
    assert ok, why
    # without the fused histogram the same set comes out
    idx_b = T.topk(scores, k, ws)
    assert torch.equal(idx, idx_b)
    o = T.decode_attention(qd, pd, N, ws, page_table=td, sel_idx=idx)
    torch.cuda.synchronize()
    assert ws.status() == 0
    want = O.gathered_attention(q, K, V, idx.cpu())
    assert_close(o, want[:, :, 0], dtype, "sparse layer")
    # and equals the reference's dense-masked formulation within tolerance
    mask = torch.zeros(B, rows // B, 1, N).scatter_(-1, idx.cpu().long().view(B, rows // B, 1, -1), 1.0)
    dense = O.sparse_layer(q, K, V, mask)
    assert_close(o, dense[:, :, 0], dtype, "sparse layer vs masked dense")


@pytest.mark.parametrize("case", ATTN_CASES, ids=[c[0] for c in ATTN_CASES])
def test_golden_reference_outputs(T, case):
    """Outputs of the reference's llama_tidal_attention_forward (fixtures) vs the kernels
    in reference-parity mode: per-q-head sets, newest token not forced."""
    name, seed, B, Hq, Hkv, D, N, k, dtype, planted = case
    z = load_golden(f"attn_{name}.npz")
    q, K, V = make_case(seed, B, Hq, Hkv, D, N, k, dtype, planted)
    assert input_digest(q, K, V) == str(z["input_sha256"]), "seeded inputs differ from the ones the fixture was made from"
    pool, table, ppb = build_pool(K, V, 1)
    ws = _ws(T, B, Hq, D, B * Hq, N)
    scores = torch.empty(B, Hq, N, dtype=torch.float32, device="cuda")
    qd, pd = q[:, :, 0].contiguous().cuda(), pool.cuda()
    o_sel = T.decode_attention(qd, pd, N, ws, pages_per_seq=ppb, scores=scores, hist=ws.hist)
    idx = T.topk(scores, k, ws, hist=ws.hist)
    assert_close(o_sel, from_np(z["o_select"], dtype)[:, :, 0], dtype, "selection layer vs reference")
    ref_sets = torch.from_numpy(z["sel_idx"])
    kk = min(N, k)
    if dtype == torch.float32:
        assert torch.equal(torch.sort(idx.cpu(), -1).values, torch.sort(ref_sets, -1).values)
    else:
        # the reference ranks logits rounded to 16 bits; compare through the tie rule on fp32 logits,
        # with a band of one 16-bit ulp at the k-th logit
        s32 = O.scores_fp32(q, K, "none").reshape(B * Hq, N)
        ok, why = O.topk_sets_match(s32, idx.reshape(B * Hq, kk).cpu(), k, tie_band=1e-4)
        assert ok, why
        kth = torch.topk(s32, kk).values[:, -1].abs().max().item()
        band = kth * (2 ** -7 if dtype == torch.bfloat16 else 2 ** -10) * 2 + 1e-4
        ok, why = O.topk_sets_match(s32, ref_sets.reshape(B * Hq, kk), k, tie_band=band)
        assert ok, "fixture itself outside the rounding band: " + why
    # sparse layer on the REFERENCE's sets must reproduce the reference's output
    o_sp = T.decode_attention(qd, pd, N, ws, pages_per_seq=ppb, sel_idx=ref_sets.cuda())
    assert_close(o_sp, from_np(z["o_sparse"], dtype)[:, :, 0], dtype, "sparse layer vs reference")
    assert ws.status() == 0


def test_physical_lists_and_extra_page(T):
    """Reference-shaped call: per-head lists of pool pages plus the newest token's page
    (tidal/utils/__init__.py:275-286, decode_attn.cuh:726-730)."""
    B, H, D, N, k = 1, 32, 128, 900, 64
    q, K, V = make_qkv(9, B, H, H, D, N, torch.float16)
    pool, table, _ = build_pool(K, V, 1, shuffle_seed=11)
    g = torch.Generator().manual_seed(1)
    logical = torch.stack([torch.randperm(N - 1, generator=g)[: k - 1] for _ in range(H)])[None]   # history only
    phys = table[0][logical.long()].to(torch.int32)
    ws = _ws(T, B, H, D, H, N)
    o = T.decode_attention(q[:, :, 0].contiguous().cuda(), pool.cuda(), N, ws, sel_idx=phys.cuda(), sel_physical=True,
                           extra_page=int(table[0, N - 1]))
    full = torch.cat((logical, torch.full((1, H, 1), N - 1)), dim=-1).to(torch.int32)
    want = O.gathered_attention(q, K, V, full)
    assert_close(o, want[:, :, 0], torch.float16, "physical lists + newest token")
    assert ws.status() == 0


def test_variable_lengths_and_counts(T):
    B, Hq, Hkv, D, N = 3, 8, 2, 128, 640
    q, K, V = make_qkv(17, B, Hq, Hkv, D, N, torch.bfloat16)
    pool, table, ppb = build_pool(K, V, 1)
    lens = torch.tensor([640, 1, 333], dtype=torch.int32)
    ws = _ws(T, B, Hq, D, B, N)
    qd, pd = q[:, :, 0].contiguous().cuda(), pool.cuda()
    o = T.decode_attention(qd, pd, N, ws, pages_per_seq=ppb, seq_lens=lens.cuda())
    for b in range(B):
        n = int(lens[b])
        want = O.gathered_attention(q[b:b + 1], K[b:b + 1, :, :n], V[b:b + 1, :, :n], torch.arange(n, dtype=torch.int32)[None])
        assert_close(o[b], want[0, :, 0], torch.bfloat16, f"sequence {b}")
    # shared lists with per-sequence valid counts (an empty list gives zeros)
    sel = torch.stack([torch.randperm(300)[:40] for _ in range(B)]).to(torch.int32)
    cnt = torch.tensor([40, 0, 7], dtype=torch.int32)
    o = T.decode_attention(qd, pd, N, ws, pages_per_seq=ppb, sel_idx=sel.cuda(), sel_counts=cnt.cuda())
    for b in range(B):
        c = int(cnt[b])
        if c == 0:
            assert float(o[b].float().abs().max()) == 0.0
            continue
        want = O.gathered_attention(q[b:b + 1], K[b:b + 1], V[b:b + 1], sel[b:b + 1, :c])
        assert_close(o[b], want[0, :, 0], torch.bfloat16, f"list {b}")
    assert ws.status() == 0


LONG_LIST_CASES = [
    # dtype, B, Hq, Hkv, D, N, k, page_size, shuffle, kwargs  — lists long enough (two chunks) that every CTA looks
    # up several blocks of pool rows, on every producer layout (1, 2 and 4 producer warps, stages of 16 and 32 tokens)
    ("bf16", 2, 32, 8, 128, 6000, 3000, 1, False, dict(use_tensor_cores=-1, heads_per_cta=2)),   # 4 producers, 16-token stages
    ("bf16", 2, 32, 8, 128, 6000, 3000, 1, False, dict(use_tensor_cores=-1, heads_per_cta=1)),   # 4 producers, 32-token stages
    ("bf16", 2, 32, 8, 128, 6000, 3000, 1, False, dict(heads_per_cta=2)),                        # tensor cores, 2 producers
    ("bf16", 2, 32, 8, 128, 6000, 3000, 1, False, dict()),                                       # tensor cores, K|V in one copy
    ("bf16", 1, 32, 8, 128, 6000, 3000, 4, True, dict()),                                        # paged: 2 producers, 16-token stages
    ("f16", 1, 32, 32, 128, 5000, 2500, 1, False, dict()),                                       # CUDA cores, whole rows
    ("f16", 1, 32, 32, 128, 5000, 2500, 1, True, dict(heads_per_cta=1)),                          # 256-byte rows, page table
    ("f16", 2, 8, 8, 64, 4000, 1999, 3, True, dict(heads_per_cta=2)),
]


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,N,k,page,shuffle,kw", LONG_LIST_CASES)
def test_long_selection_lists(T, dt, B, Hq, Hkv, D, N, k, page, shuffle, kw):
    dtype = DT[dt]
    q, K, V = make_qkv(23, B, Hq, Hkv, D, N, dtype)
    pool, table, ppb = build_pool(K, V, page, shuffle_seed=5 if shuffle else None)
    g = torch.Generator().manual_seed(3)
    sel = torch.stack([torch.randperm(N, generator=g)[:k] for _ in range(B)]).to(torch.int32)
    ws = _ws(T, B, Hq, D, B, N)
    o = T.decode_attention(q[:, :, 0].contiguous().cuda(), pool.cuda(), N, ws, pages_per_seq=ppb,
                           page_table=None if table is None else table.cuda(), sel_idx=sel.cuda(), num_chunks=2, **kw)
    torch.cuda.synchronize()
    assert ws.status() == 0
    for b in range(B):
        want = O.gathered_attention(q[b:b + 1], K[b:b + 1], V[b:b + 1], sel[b:b + 1])
        assert_close(o[b], want[0, :, 0], dtype, f"sequence {b}")
    # the same list in a full layer's clothes: long paged sequences take the same lookups
    if table is not None:
        o_full = T.decode_attention(q[:, :, 0].contiguous().cuda(), pool.cuda(), N, ws, pages_per_seq=ppb, page_table=table.cuda(),
                                    num_chunks=3, **kw)
        want = O.gathered_attention(q, K, V, torch.arange(N, dtype=torch.int32)[None].expand(B, N))
        assert_close(o_full, want[:, :, 0], dtype, "full layer through the page table")
        assert ws.status() == 0


@pytest.mark.parametrize("B,Hq,Hkv,k", [(8, 64, 8, 1024), (4, 32, 8, 2048), (3, 64, 8, 1500)])
def test_sparse_lists_long_enough_for_several_clusters(T, B, Hq, Hkv, k):
    """Lists of a thousand and more tokens with all KV heads in one CTA (bf16, page_size 1): the planner puts two
    clusters of 8 (or four of 4) on each list; every cluster leaves its share in the workspace and the last to
    arrive finishes.  Checked against the gathered oracle, three calls in a row (the arrival counters must be
    back at zero each time), normalised output and un-normalised partials."""
    D, N, dtype = 128, 5000, torch.bfloat16
    q, K, V = make_qkv(29, B, Hq, Hkv, D, N, dtype)
    pool, _, ppb = build_pool(K, V, 1)
    g = torch.Generator().manual_seed(k)
    sel = torch.stack([torch.sort(torch.randperm(N, generator=g)[:k]).values for _ in range(B)]).to(torch.int32)
    ws = _ws(T, B, Hq, D, B, N)
    qd, pd, sd = q[:, :, 0].contiguous().cuda(), pool.cuda(), sel.cuda()
    want = torch.cat([O.gathered_attention(q[b:b + 1], K[b:b + 1], V[b:b + 1], sel[b:b + 1])[:, :, 0] for b in range(B)])
    for rep in range(3):
        o = T.decode_attention(qd, pd, N, ws, pages_per_seq=ppb, sel_idx=sd)
        torch.cuda.synchronize()
        assert ws.status() == 0
        assert_close(o, want, dtype, f"call {rep}")
    m = torch.empty(B, Hq, device="cuda")
    l = torch.empty(B, Hq, device="cuda")
    acc = torch.empty(B, Hq, D, device="cuda")
    T.decode_attention(qd, pd, N, ws, pages_per_seq=ppb, sel_idx=sd, partials=(m, l, acc), want_out=False)
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert_close((acc / l[..., None]).to(dtype), want, dtype, "partials")


def test_bad_index_is_flagged_not_followed(T):
    B, H, D, N = 1, 8, 128, 100
    q, K, V = make_qkv(1, B, H, H, D, N, torch.float16)
    pool, _, ppb = build_pool(K, V, 1)
    ws = _ws(T, B, H, D, B, N)
    sel = torch.tensor([[3, 5, 100000, -4]], dtype=torch.int32)
    T.decode_attention(q[:, :, 0].contiguous().cuda(), pool.cuda(), N, ws, pages_per_seq=ppb, sel_idx=sel.cuda())
    torch.cuda.synchronize()
    assert ws.status() & 2
    ws.reset()
    assert ws.status() == 0


def test_sharded_partials_merge(T):
    """Sequence-sharded KV emulated on one GPU: per-shard partials + candidates, merged."""
    B, Hq, Hkv, D, N, k, g = 2, 32, 8, 128, 4000, 128, 4
    dtype = torch.bfloat16
    q, K, V = make_qkv(23, B, Hq, Hkv, D, N, dtype, planted=32)
    bounds = [0, 1000, 1001, 2500, N]       # uneven shards, one of a single token
    qd = q[:, :, 0].contiguous().cuda()
    ws = _ws(T, B, Hq, D, B, N)
    m = torch.empty(g, B, Hq, device="cuda")
    l = torch.empty(g, B, Hq, device="cuda")
    o = torch.empty(g, B, Hq, D, device="cuda")
    cs = torch.full((B, g, k), -float("inf"), device="cuda")
    ci = torch.zeros((B, g, k), dtype=torch.int32, device="cuda")
    pools = []
    for r in range(g):
        lo, hi = bounds[r], bounds[r + 1]
        pool, _, ppb = build_pool(K[:, :, lo:hi].contiguous(), V[:, :, lo:hi].contiguous(), 1)
        pools.append((pool.cuda(), ppb))
        sc = torch.empty(B, hi - lo, device="cuda")
        T.decode_attention(qd, pools[r][0], hi - lo, ws, pages_per_seq=ppb, scores=sc, hist=ws.hist,
                           partials=(m[r], l[r], o[r]), want_out=False)
        kk = min(k, hi - lo)
        idx = torch.zeros(B, k, dtype=torch.int32, device="cuda")
        val = torch.full((B, k), -float("inf"), device="cuda")
        T.topk(sc, k, ws, out_idx=idx, out_val=val, idx_offset=lo, hist=ws.hist)
        cs[:, r], ci[:, r] = val, idx
        if kk < k:
            cs[:, r, kk:] = -float("inf")
    out = T.merge_partials(m, l, o, dtype)
    want = O.gathered_attention(q, K, V, torch.arange(N, dtype=torch.int32)[None].expand(B, N))
    assert_close(out, want[:, :, 0], dtype, "merged shards")
    gidx = T.topk(cs.view(B, g * k), k, ws, in_idx=ci.view(B, g * k))
    ok, why = O.topk_sets_match(O.scores_fp32(q, K, "sum"), gidx.cpu(), k, tie_band=1e-4)
    assert ok, why
    # sparse layer: every shard attends to the selected tokens it owns
    for r in range(g):
        lo, hi = bounds[r], bounds[r + 1]
        cnt = torch.zeros(B, dtype=torch.int32, device="cuda")
        loc = torch.zeros(B, k, dtype=torch.int32, device="cuda")
        T.topk(cs.view(B, g * k), k, ws, in_idx=ci.view(B, g * k), out_idx=loc, own_range=(lo, hi), out_count=cnt)
        T.decode_attention(qd, pools[r][0], hi - lo, ws, pages_per_seq=pools[r][1], sel_idx=loc, sel_counts=cnt,
                           partials=(m[r], l[r], o[r]), want_out=False)
    out = T.merge_partials(m, l, o, dtype)
    want = O.gathered_attention(q, K, V, gidx.cpu())
    assert_close(out, want[:, :, 0], dtype, "sharded sparse layer")
    assert ws.status() == 0


@pytest.mark.parametrize("name,dtype,D", [("f32_d64", torch.float32, 64), ("f16_d128", torch.float16, 128),
                                          ("bf16_d128", torch.bfloat16, 128)])
def test_rope_golden(T, name, dtype, D):
    """apply_rotary_pos_emb of the reference model (fixture) vs the fused kernel, per position."""
    z = load_golden("rope.npz")
    q, k = from_np(z[f"{name}_q"], dtype), from_np(z[f"{name}_k"], dtype)        # [1,H,n,D]
    qe, ke = from_np(z[f"{name}_qe"], dtype), from_np(z[f"{name}_ke"], dtype)
    theta = float(z[f"{name}_theta"])
    inv = O.rope_inv_freq(D, theta).cuda()
    for j, pos in enumerate(z[f"{name}_pos"][0].tolist()):
        qd, kd = q[0, :, j][None].contiguous().cuda(), k[0, :, j][None].contiguous().cuda()
        T.rope_append(qd, kd, None, None, pos0=pos, rope_theta=theta, rope_mode=1, inv_freq=inv)
        tol = dict(rtol=0, atol=2e-6) if dtype == torch.float32 else dict(rtol=0, atol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -9)
        # large angles lose fp32 precision in the sincos argument itself; one storage ulp of slack
        assert torch.allclose(qd.cpu().float()[0], qe[0, :, j].float(), **tol), (name, pos)
        assert torch.allclose(kd.cpu().float()[0], ke[0, :, j].float(), **tol), (name, pos)
        if dtype != torch.float32:
            # after rounding to 16 bits the last-ulp differences of cosf/sinf between host and device vanish
            exact = (qd.cpu()[0] == qe[0, :, j]).float().mean().item()
            assert exact > 0.97, f"{name} pos {pos}: only {exact:.3f} of elements bit-equal"


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,page,tps", [("f16", 1, 32, 32, 128, 1, 1), ("bf16", 4, 32, 8, 128, 1, 1),
                                                     ("f32", 1, 4, 4, 64, 1, 1), ("f16", 2, 8, 8, 128, 16, 37),
                                                     ("bf16", 1, 64, 8, 128, 3, 5)])
def test_rope_append(T, dt, B, Hq, Hkv, D, page, tps):
    """q/k rotated, k/v land in the right pool slots (cpu_reference.h:294-327), nothing else is touched."""
    dtype = DT[dt]
    g = torch.Generator().manual_seed(77)
    n = B * tps
    q = torch.randn(n, Hq, D, generator=g).to(dtype)
    k = torch.randn(n, Hkv, D, generator=g).to(dtype)
    v = torch.randn(n, Hkv, D, generator=g).to(dtype)
    past = torch.tensor([5, 1000, 31, 64][:B], dtype=torch.int32)
    ppb = (int(past.max()) + tps + page - 1) // page + 1
    total = B * ppb + 2
    table = torch.randperm(total, generator=g)[: B * ppb].view(B, ppb).to(torch.int32)
    pool0 = torch.randn(total, 2, page, Hkv, D, generator=g).to(dtype)
    pool = pool0.clone().cuda()
    qd, kd = q.clone().cuda(), k.clone().cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    T.rope_append(qd, kd, v.cuda(), pool, batch=B, pos0_dev=past.cuda(), page_table=table.cuda(), rope_theta=1e4,
                  rope_mode=2, status=status)
    pos = (past[:, None] + torch.arange(tps)[None]).reshape(-1)
    q_want, k_want = O.apply_rope_fp32(q, pos, 1e4), O.apply_rope_fp32(k, pos, 1e4)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=0, atol=2 ** -6 if dtype == torch.bfloat16 else 2 ** -8)
    assert torch.allclose(qd.cpu().float(), q_want.float(), **tol)
    assert torch.allclose(kd.cpu().float(), k_want.float(), **tol)
    want_pool = pool0.clone()
    for b in range(B):
        seq_len = int(past[b]) + tps
        O.append_paged_kv(want_pool, table[b].tolist(), seq_len, kd.cpu()[b * tps:(b + 1) * tps], v[b * tps:(b + 1) * tps])
    assert torch.equal(pool.cpu(), want_pool), "pool contents differ from the CPU append"
    assert int(status) == 0


LINEAR_CASES = [
    # dtype, M, N, K, norm, residual, silu_mul
    ("f16", 1, 4096, 4096, False, False, False),
    ("f16", 1, 22016, 4096, True, False, True),          # gate|up of a 7B layer behind its RMSNorm
    ("f16", 1, 4096, 11008, False, True, False),         # down projection into the residual stream
    ("bf16", 4, 6144, 4096, True, False, False),         # q|k|v of an 8B layer, four sequences
    ("bf16", 8, 512, 1024, False, True, False),
    ("bf16", 4, 28672, 4096, True, False, True),         # gate|up of an 8B layer, four sequences (tensor-core kernel, tile pairs)
    ("bf16", 4, 4096, 14336, False, True, False),        # activations too large to keep resident: they travel with the weights
    ("f16", 8, 1024, 8192, False, False, False),
    ("f16", 2, 1000, 4096, False, True, False),          # N not a multiple of the 16-row tile
    ("bf16", 1, 688, 352, False, False, True),           # F = 344 is not a multiple of 16: CUDA-core kernel
    ("f16", 3, 1001, 512, True, True, False),            # odd N: the last row has no partner
    ("f32", 1, 1024, 256, True, False, False),           # config 1: lm_head behind the final norm
    ("f32", 2, 1376, 256, True, False, True),            # config 1: gate|up, F = 688
    ("f32", 1, 256, 688, False, True, False),            # K not a multiple of a warp's stride
]


@pytest.mark.parametrize("dt,M,N,K,norm,res,silu", LINEAR_CASES)
def test_decode_linear(T, dt, M, N, K, norm, res, silu):
    """tidal_decode_linear against the same ops done one by one in torch (tidal/models/llama.py:160-208):
    rms_norm -> linear -> (+ residual | silu(gate) * up), every intermediate rounded to the storage type."""
    dtype = DT[dt]
    g = torch.Generator().manual_seed(11)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype)
    nw = (1.0 + 0.1 * torch.randn(K, generator=g)).to(dtype) if norm else None
    r = torch.randn(M, N // 2 if silu else N, generator=g).to(dtype) if res else None
    xin = O.rms_norm(x, nw, 1e-6) if norm else x
    y = (xin.double() @ w.double().t()).to(dtype)                      # fp32-or-better accumulation, one rounding
    if silu:
        F = N // 2
        want = (torch.nn.functional.silu(y[:, :F].float()).to(dtype).float() * y[:, F:].float()).to(dtype)
    elif res:
        want = (y.float() + r.float()).to(dtype)
    else:
        want = y
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = T.linear(x.cuda(), w.cuda(), residual=None if r is None else r.cuda(), norm_weight=None if nw is None else nw.cuda(),
                   eps=1e-6, silu_mul=silu, status=status)
    assert got.shape == want.shape
    assert_close(got, want, dtype, "decode linear")
    torch.cuda.synchronize()
    again = T.linear(x.cuda(), w.cuda(), residual=None if r is None else r.cuda(), norm_weight=None if nw is None else nw.cuda(),
                     eps=1e-6, silu_mul=silu, status=status, static_weights=True)       # weights fetched ahead of stream order
    assert torch.equal(again, got) and int(status.item()) == 0
    if res:   # in place: the residual stream is the output
        buf = r.cuda().clone()
        T.linear(x.cuda(), w.cuda(), out=buf, residual=buf, norm_weight=None if nw is None else nw.cuda(), eps=1e-6)
        assert torch.equal(buf, got)


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,K,page,mode", [
    ("f16", 1, 32, 32, 128, 4096, 1, 1), ("bf16", 4, 32, 8, 128, 4096, 1, 2), ("bf16", 2, 8, 2, 64, 512, 4, 1),
    ("f16", 3, 4, 4, 64, 256, 1, 0),
])
def test_fused_qkv_projection_rope_append(T, dt, B, Hq, Hkv, D, K, page, mode):
    """tidal_decode_qkv = RMSNorm + q|k|v projection + RoPE + KV append in one launch, against the same
    steps as separate calls (tidal_decode_linear, tidal_rope_append), which have their own parity tests."""
    dtype = DT[dt]
    g = torch.Generator().manual_seed(5)
    N = (Hq + 2 * Hkv) * D
    x = torch.randn(B, K, generator=g).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype).cuda()
    nw = (1.0 + 0.1 * torch.randn(K, generator=g)).to(dtype).cuda()
    ppb = 6
    pages = B * ppb + 3
    table = torch.randperm(pages, generator=g)[:B * ppb].view(B, ppb).to(torch.int32).cuda()    # distinct pages per sequence
    pos = torch.tensor([(7 * b + 5) % (ppb * page) for b in range(B)], dtype=torch.int32).cuda()
    inv = (1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))).cuda()
    rope = dict(pos0_dev=pos, page_table=table, rope_theta=1e4, rope_scale=1.0, rope_mode=mode, inv_freq=inv)
    # separate calls
    pool_a = torch.zeros(pages, 2, page, Hkv, D, dtype=dtype, device="cuda")
    qkv = T.linear(x, w, norm_weight=nw, eps=1e-6)
    q_a = qkv[:, :Hq * D].contiguous().view(B, Hq, D)
    k_a = qkv[:, Hq * D:(Hq + Hkv) * D].contiguous().view(B, Hkv, D)
    v_a = qkv[:, (Hq + Hkv) * D:].contiguous().view(B, Hkv, D)
    T.rope_append(q_a, k_a, v_a, pool_a, batch=B, **rope)
    # one call
    pool_b = torch.zeros_like(pool_a)
    q_b = torch.empty(B, Hq, D, dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    T.qkv_rope_append(x, w, q_b, pool_b, num_kv_heads=Hkv, norm_weight=nw, eps=1e-6, status=status, **rope)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    tol = dict(rtol=0, atol=0) if mode != 2 else dict(rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -10, atol=1e-6)
    assert torch.allclose(q_b.float(), q_a.float(), **tol)
    assert torch.allclose(pool_b.float(), pool_a.float(), **tol)
    assert float(pool_b.float().abs().sum()) > 0


PREFILL_CASES = [
    # dtype, n_q, kv_len, Hq, Hkv, D, page_size, causal
    ("f16", 128, 128, 1, 1, 128, 1, True),
    ("bf16", 300, 300, 8, 2, 128, 16, True),          # GQA, ragged last tile, pages of 16 in shuffled order
    ("f16", 63, 2047, 4, 4, 128, 1, True),            # a later chunk of a prompt (kernels/src/test/test_prefill.cu:305)
    ("bf16", 513, 513, 4, 1, 64, 3, True),            # head_dim 64, page size that divides nothing
    ("f16", 200, 200, 2, 2, 64, 1, False),            # non-causal
    ("f16", 2048, 2048, 4, 2, 128, 1, True),
    ("bf16", 1, 65, 2, 1, 128, 1, True),              # a single row
    ("f16", 17, 17, 32, 8, 128, 31, True),            # shortest length of the reference's sweep, one partial page
    ("f32", 2048, 2048, 4, 4, 64, 1, True),           # configuration 1's prompt: fp32 storage, the CUDA-core kernel
    ("f32", 130, 333, 8, 2, 128, 5, True),            # fp32 GQA, a later chunk, ragged pages
    ("f32", 65, 65, 2, 2, 64, 16, False),
    ("bf16", 1000, 5000, 8, 2, 128, 4, True),         # two row blocks, 40 tiles: the ring of five wraps many times, ragged on both ends
    ("f16", 100, 3001, 4, 4, 128, 1, True),           # one row block, 24 tiles, odd length
    ("bf16", 700, 700, 4, 4, 64, 2, False),           # head_dim 64 with two row blocks, non-causal
]


@pytest.mark.parametrize("dt,n_q,kv_len,Hq,Hkv,D,page,causal", PREFILL_CASES)
def test_prefill(T, dt, n_q, kv_len, Hq, Hkv, D, page, causal):
    """tidal_prefill (tcgen05 kernel) against the oracle's causal attention over the same stored values;
    shapes follow kernels/src/test/test_prefill.cu:408-491 (GQA 4/8/32 kv heads, ragged lengths)."""
    dtype = DT[dt]
    g = torch.Generator().manual_seed(n_q * 7 + kv_len)
    n_pages = (kv_len + page - 1) // page
    pool = torch.randn(n_pages + 5, 2, page, Hkv, D, generator=g).to(dtype)
    table = torch.randperm(n_pages + 5, generator=g)[:n_pages].to(torch.int32)
    q = torch.randn(n_q, Hq, D, generator=g).to(dtype)
    sel = pool[table.long()]
    K = sel[:, 0].reshape(-1, Hkv, D)[:kv_len]
    V = sel[:, 1].reshape(-1, Hkv, D)[:kv_len]
    want = O.causal_prefill(q, K, V, causal)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = T.prefill(q.cuda(), pool.cuda(), table.cuda(), kv_len, causal=causal, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_close(got, want, dtype, "prefill")
    # the last row is what a decode step over the same cache computes
    if causal:
        ws = T.Workspace(1, Hq, D, Hq, kv_len)
        dec = T.decode_attention(q[-1:].cuda().contiguous(), pool.cuda(), kv_len, ws, page_table=table.cuda().view(1, -1))
        assert_close(got[-1:], dec, dtype, "prefill last row vs decode")


def test_prefill_rejects_what_it_does_not_compute(T):
    q = torch.zeros(4, 2, 128, device="cuda")
    pool = torch.zeros(4, 2, 1, 2, 128, device="cuda")
    table = torch.arange(4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="head_dim"):
        T.prefill(torch.zeros(4, 2, 32, device="cuda").half(), torch.zeros(4, 2, 1, 2, 32, device="cuda").half(), table, 4)
    with pytest.raises(RuntimeError, match="kv_len"):
        T.prefill(q.half(), pool.half(), table, 3)


def test_prefill_bad_page_entry_is_flagged_not_followed(T):
    """A page-table entry outside the pool reads as zeros and sets TIDAL_DEV_BAD_INDEX; nothing is fetched
    through it (the decode kernels treat their lists the same way)."""
    from tidaldecode_b200 import _lib as L

    g = torch.Generator().manual_seed(3)
    n, Hq, Hkv, D = 200, 4, 2, 128
    pool = torch.randn(n, 2, 1, Hkv, D, generator=g).half()
    q = torch.randn(n, Hq, D, generator=g).half()
    table = torch.arange(n, dtype=torch.int32)
    bad = table.clone()
    bad[57] = n + 1000
    bad[58] = -4
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = T.prefill(q.cuda(), pool.cuda(), bad.cuda(), n, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == L.DEV_BAD_INDEX
    # tokens 57 and 58 read as zero rows: logit 0 and value 0 for the rows that see them
    K = pool[:, 0, 0].clone()
    V = pool[:, 1, 0].clone()
    K[57:59] = 0
    V[57:59] = 0
    assert_close(got, O.causal_prefill(q, K, V, True), torch.float16, "prefill with two unreadable pages")


def test_rope_append_out_of_place_queries(T):
    """q_src: the queries are read from one buffer and written, rotated, to another; the source survives."""
    g = torch.Generator().manual_seed(8)
    B, Hq, Hkv, D = 3, 8, 2, 128
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    pool_a = torch.zeros(B * 8, 2, 1, Hkv, D, dtype=torch.bfloat16, device="cuda")
    pool_b = torch.zeros_like(pool_a)
    q_in_place, k_in_place = q.clone(), k.clone()
    T.rope_append(q_in_place, k_in_place, v, pool_a, batch=B, pos0=5, rope_theta=5e5, rope_mode=2)
    q_out, q_keep, k_keep = torch.zeros_like(q), q.clone(), k.clone()
    T.rope_append(q_out, k_keep, v, pool_b, batch=B, pos0=5, rope_theta=5e5, rope_mode=2, q_src=q_keep, rotate_k_in_place=False)
    torch.cuda.synchronize()
    assert torch.equal(q_out, q_in_place) and torch.equal(pool_a, pool_b)
    assert torch.equal(q_keep, q) and torch.equal(k_keep, k), "sources must be left as they were"


def test_peer_exchange_wait_runs_out_and_reset_recovers(T):
    """Rank 0 of a two-rank exchange whose peer never calls: the bounded wait runs out, the status word says
    so and the kernel returns (the context stays usable).  After tidal_peer_exchange_reset the same buffers
    carry a complete exchange again — the missing rank's block and arrivals are written by the host before
    the launch, so no kernel ever waits on another one."""
    from tidaldecode_b200 import _lib as L

    dev = torch.device("cuda", 0)
    words = 4 * 8 * (64 + 2)                                     # m, l, o of 4 x 8 heads x 64
    px = T.PeerExchange.loopback(words * 4, 2, dev, wait_limit=2000)
    send = torch.arange(words, dtype=torch.float32, device=dev)
    recv = torch.zeros(2, words, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    px.all_gather(send, recv, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == L.DEV_WAIT_TIMEOUT
    assert torch.equal(recv[0], send), "its own block still arrives"
    px.reset()
    status.zero_()
    torch.cuda.synchronize()
    assert int(px.flags.abs().sum()) == 0 and int(px.state.abs().sum()) == 0
    # the peer's part of exchange 1 (parity 1), as its kernel would have left it: block in slot [1][1], every CTA's flag = 1
    other = torch.full((words,), 7.0, dtype=torch.float32, device=dev)
    px.stage[1, 1].copy_(other.view(torch.uint8))
    px.flags[1, 1] = 1
    px.all_gather(send, recv, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(recv[0], send) and torch.equal(recv[1], other)
    # and exchange 2 (parity 0) with another payload size on the same buffers
    half = words // 2 // 4 * 4
    px.stage[0, 1, : half * 4].copy_(other[:half].view(torch.uint8))
    px.flags[0, 1] = 2
    recv.zero_()
    px.all_gather(send, recv, nbytes=half * 4, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(recv[0, :half], send[:half]) and torch.equal(recv[1, :half], other[:half])


@pytest.mark.parametrize("world,B,Hq,D,k,rows_per_seq,dt", [
    (2, 2, 8, 64, 24, 1, "f32"), (4, 4, 32, 128, 128, 1, "bf16"), (8, 8, 64, 128, 1024, 1, "bf16"),
    (4, 1, 32, 128, 256, 1, "f16"), (2, 2, 8, 128, 48, 8, "bf16"),
])
def test_peer_exchange_merges_and_ranks_in_one_launch(T, world, B, Hq, D, k, rows_per_seq, dt):
    """The exchange kernel's own merge of the ranks' partials and its ranking of their candidates against
    tidal_merge_partials and tidal_topk on the gathered blocks.  One GPU stands for all ranks: rank 0's
    kernel runs, the other ranks' blocks and arrivals are placed by the host beforehand (nothing waits on
    another kernel).  Twice, so that both parities of the double buffer are used."""
    from tidaldecode_b200.sharded import pack_layout

    dev = torch.device("cuda", 0)
    dtype = DT[dt]
    rows = B * rows_per_seq
    L = pack_layout(B, Hq, D, rows, k)
    tot = (L["total"] + 3) // 4 * 4
    px = T.PeerExchange.loopback(tot * 4, world, dev, wait_limit=100000)
    g = torch.Generator().manual_seed(world * 100 + k)
    n_loc = 5 * k                                                   # positions per rank
    ws = T.Workspace(B, Hq, D, rows, world * k)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for exchange in range(1, 4):
        blocks = torch.zeros(world, tot)
        for r in range(world):
            blocks[r, L["m"]:L["l"]] = torch.randn(B * Hq, generator=g) * 3
            blocks[r, L["l"]:L["o"]] = torch.rand(B * Hq, generator=g) + 0.5
            blocks[r, L["o"]:L["cs"]] = torch.randn(B * Hq * D, generator=g)
            sc = torch.round(torch.randn(rows, k, generator=g) * 8) / 8         # ties across ranks
            pos = torch.stack([torch.sort(torch.randperm(n_loc, generator=g)[:k]).values for _ in range(rows)]) + r * n_loc
            blocks[r, L["cs"]:L["ci"]] = sc.reshape(-1)
            blocks[r, L["ci"]:L["ci"] + rows * k] = pos.to(torch.int32).view(torch.float32).reshape(-1)
        if exchange == 2:
            blocks[1, L["m"]:L["l"]] = -float("inf")                 # a rank that attended nothing
        blocks = blocks.to(dev)
        par = exchange & 1
        for r in range(1, world):
            px.stage[par, r].copy_(blocks[r].view(torch.uint8))
            px.flags[par, r] = exchange
        own = (2 * n_loc, 3 * n_loc) if world > 2 else (0, n_loc)
        out = torch.full((B * Hq, D), float("nan"), dtype=dtype, device=dev)
        sel = torch.full((rows, k), -1, dtype=torch.int32, device=dev)
        cnt = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        recv = torch.zeros(world, tot, device=dev)
        px.all_gather(blocks[0].contiguous(), recv, status=status, merge=(out, L["m"], L["l"], L["o"]),
                      candidates=dict(rows=rows, k=k, select=k, score_off=L["cs"], idx_off=L["ci"], own=own, out=sel, count=cnt))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(recv, blocks)
        flat = recv.view(-1)
        want = T.merge_partials(flat[L["m"]:], flat[L["l"]:], flat[L["o"]:], dtype, geometry=(world, B, Hq, D, tot))
        assert torch.equal(out.view(B, Hq, D), want)
        want_sel = torch.full((rows, k), -1, dtype=torch.int32, device=dev)
        want_cnt = torch.zeros(rows, dtype=torch.int32, device=dev)
        T.topk(flat[L["cs"]:], k, ws, n=world * k, in_idx=flat.view(torch.int32)[L["ci"]:], out_idx=want_sel, own_range=own,
               out_count=want_cnt, segments=(rows, k, tot, k))
        torch.cuda.synchronize()
        assert torch.equal(cnt, want_cnt)
        for r in range(rows):
            c = int(cnt[r])
            assert torch.equal(sel[r, :c], want_sel[r, :c])
    assert ws.status() == 0


@pytest.mark.parametrize("dt,B,Hq,Hkv,D,N,page,mpage", [
    ("f16", 1, 32, 32, 128, 1000, 16, 16),      # the reference's shape: MHA, pages of 16 (test_max_possible.cu)
    ("bf16", 2, 8, 2, 128, 333, 16, 4), ("f32", 1, 4, 4, 64, 77, 8, 3), ("f16", 1, 8, 8, 64, 40, 1, 16),
])
def test_quest_page_metadata_and_estimate(T, dt, B, Hq, Hkv, D, N, page, mpage):
    """Per-page key bounds rebuilt from the pool (after a prompt, then after single-token appends) are exactly the
    oracle's, and the estimate equals sum_d max(q_d max_d, q_d min_d) within the reference's 1e-3 / 1e-3
    (kernels/src/test/test_max_possible.cu:29-154)."""
    dtype = DT[dt]
    q, K, V = make_qkv(600 + N, B, Hq, Hkv, D, N, dtype)
    pool, table, ppb = build_pool(K, V, page, shuffle_seed=4)
    g = torch.Generator().manual_seed(N)
    mper = (ppb + mpage - 1) // mpage
    mtable = torch.randperm(B * mper + 2, generator=g)[: B * mper].view(B, mper).to(torch.int32)
    meta = torch.full((B * mper + 2, 2, mpage, Hkv, D), float("nan")).to(dtype).cuda()
    pd, td, mtd = pool.cuda(), table.cuda(), mtable.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    n0 = N - 3
    T.update_page_meta(pd, meta, n0, 0, batch=B, page_table=td, meta_table=mtd, status=status)        # the prompt
    for n in range(n0 + 1, N + 1):                                                                        # then token by token
        T.update_page_meta(pd, meta, n, n - 1, batch=B, page_table=td, meta_table=mtd, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    out = T.estimate(q[:, :, 0].contiguous().cuda(), meta, ppb - 1, meta_table=mtd, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    mh = meta.cpu()
    for b in range(B):
        want_max, want_min = O.page_key_bounds(K[b].permute(1, 0, 2), page)            # [P,Hkv,D]
        for e in range(ppb):
            slot = mh[int(mtable[b, e // mpage]), :, e % mpage]
            assert torch.equal(slot[0], want_max[e]) and torch.equal(slot[1], want_min[e]), (b, e)
        want = O.estimate_scores(q[b, :, 0], want_max, want_min)[:, : ppb - 1]
        assert torch.allclose(out[b, :, : ppb - 1].float().cpu(), want, rtol=1e-3 if dt == "f32" else 4e-3, atol=1e-3 if dt == "f32" else 3e-2)


def test_estimate_through_the_reference_operator_names(T):
    """append_kv_cache_prefill / _decode maintain the metadata pool they are given and estimate_attn_score reads it,
    with the reference's argument lists (tidal/ops/csrc/bsk_ops.h:20-76)."""
    import tidaldecode_b200._kernels as Kn

    H, D, N, page = 8, 128, 100, 16
    q, K, V = make_qkv(77, 1, H, H, D, N, torch.float16)
    n_pages = (N + page - 1) // page
    pool = torch.zeros(n_pages + 1, 2, page, H, D, dtype=torch.float16, device="cuda")
    meta = torch.zeros(2, 2, page, H, D, dtype=torch.float16, device="cuda")
    kv_idx = torch.arange(n_pages, dtype=torch.int32, device="cuda")
    meta_idx = torch.tensor([1], dtype=torch.int32, device="cuda")
    indptr = torch.tensor([0, n_pages], dtype=torch.int32, device="cuda")
    mindptr = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    Kt, Vt = K[0].permute(1, 0, 2).contiguous().cuda(), V[0].permute(1, 0, 2).contiguous().cuda()      # [N,H,D]
    n0 = N - 1
    p0 = (n0 + page - 1) // page
    Kn.append_kv_cache_prefill(Kt[:n0].contiguous(), Vt[:n0].contiguous(), pool, kv_idx[:p0].contiguous(), indptr, (n0 - 1) % page + 1,
                               int(kv_idx[p0 - 1]), meta, meta_idx, mindptr, p0, 1, 0)
    Kn.append_kv_cache_decode(Kt[n0:N].contiguous(), Vt[n0:N].contiguous(), pool, kv_idx, indptr, (N - 1) % page + 1, int(kv_idx[-1]),
                              meta, meta_idx, mindptr, n_pages, 1, 0)
    o = torch.zeros(H, n_pages - 1, dtype=torch.float16, device="cuda")
    Kn.estimate_attn_score(q[:, :, 0].contiguous().cuda(), o, meta, meta_idx, mindptr, n_pages, 1, 0)
    torch.cuda.synchronize()
    mx, mn = O.page_key_bounds(K[0].permute(1, 0, 2), page)
    want = O.estimate_scores(q[0, :, 0], mx, mn)[:, : n_pages - 1]
    assert torch.allclose(o.float().cpu(), want, rtol=4e-3, atol=3e-2)
