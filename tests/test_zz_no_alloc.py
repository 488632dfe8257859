"""tidal_topk_static: the top-k entry point for callers that cannot allocate — a plugin
whose host runtime owns every byte of device memory, or a serving loop that forbids
allocator calls once it is warm because cudaMalloc/cudaFree can stall all streams.
It keeps its scratch in a fixed array inside the library instead of a workspace.

Checked here, through the C ABI: its output equals the workspace-based tidal_topk's,
bit for bit (both emit position-ordered sets), and is a valid top-k of the scores by the
CPU oracle's rule, on two calls in a row with different inputs (the second must not see
anything the first left in the shared array); the call leaves the device's free memory
as it found it; sizes and argument forms beyond its stated limits are refused; the fault
word it keeps for callers without a status word can be read and cleared.  This file
sorts last so that a failure here cannot hide any other test from a run that stops at
the first failure.
"""
from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_topk(L, scores, k, out_idx, out_val=None, status=None, **kw):
    a = L.TopkArgs()
    rows, n = scores.shape
    a.d_scores, a.rows, a.n, a.row_stride, a.k = scores.data_ptr(), rows, n, n, k
    a.d_out_idx, a.out_stride = out_idx.data_ptr(), out_idx.shape[-1]
    a.d_out_val = out_val.data_ptr() if out_val is not None else None
    for key, v in kw.items():
        setattr(a, key, v)
    stream = torch.cuda.current_stream().cuda_stream
    return L.lib.tidal_topk_static(C.byref(a), status.data_ptr() if status is not None else None, stream)


def test_static_topk_matches_workspace_topk_twice():
    import tidaldecode_b200.ops as T
    from tidaldecode_b200 import _lib as L

    torch.cuda.set_device(0)
    before = torch.cuda.memory_allocated()
    g = torch.Generator().manual_seed(99)
    cases = [(4, 32768, 256, False), (8, 5000, 1000, True)]        # second call: other shape, heavy ties, forced last
    inputs = []
    for rows, n, k, ties in cases:
        s = torch.randn(rows, n, generator=g)
        if ties:
            s = torch.round(s * 4) / 4
        inputs.append((s.cuda(), k, ties))
    ws = T.Workspace(1, 1, 64, 8, 32768)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    from oracle import tidal_oracle as O
    # one untimed call first: the library looks up its array's address on the first use on a device
    warm = torch.zeros(1, 8, dtype=torch.int32, device="cuda")
    assert _static_topk(L, inputs[0][0][:1, :64].contiguous(), 8, warm) == 0
    torch.cuda.synchronize()
    for s, k, force in inputs:
        rows, n = s.shape
        want_idx = torch.full((rows, k), -1, dtype=torch.int32, device="cuda")
        want_val = torch.zeros(rows, k, device="cuda")
        T.topk(s, k, ws, out_idx=want_idx, out_val=want_val, force_last=force)
        got_idx = torch.full((rows, k), -1, dtype=torch.int32, device="cuda")
        got_val = torch.zeros(rows, k, device="cuda")
        torch.cuda.synchronize()
        held, free = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = _static_topk(L, s, k, got_idx, got_val, status, force_last=1 if force else 0)
        assert rc == 0, L.last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == held, "the call must not allocate through torch"
        assert torch.cuda.mem_get_info()[0] == free, "the call must not allocate from the driver either"
        assert torch.equal(got_idx, want_idx)
        assert torch.equal(got_val, want_val)
        ok, why = O.topk_sets_match(s.cpu(), got_idx.cpu(), k, tie_band=0.0, force_last=force)
        assert ok, why
    assert int(status) == 0 and ws.status() == 0
    # k >= n selects everything, in order
    s = inputs[1][0][:2, :100].contiguous()
    out = torch.full((2, 100), -1, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s, 500, out) == 0
    assert torch.equal(out.cpu(), torch.arange(100, dtype=torch.int32)[None].expand(2, 100))
    del ws
    assert torch.cuda.memory_allocated() <= before + 64 * 1024 * 1024


def test_static_topk_refuses_sizes_beyond_its_limits():
    from tidaldecode_b200 import _lib as L

    torch.cuda.set_device(0)
    s = torch.zeros(9, 64, device="cuda")
    out = torch.zeros(9, 8, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s, 8, out) == L.ERR_ARG and "at most 8 rows" in L.last_error()
    a = L.TopkArgs()
    a.d_scores, a.d_out_idx, a.rows, a.n, a.row_stride, a.k, a.out_stride = s.data_ptr(), out.data_ptr(), 1, 1 << 19, 1 << 19, 8, 8
    assert L.lib.tidal_topk_static(C.byref(a), None, None) == L.ERR_ARG and "at most 262144" in L.last_error()
    a.n, a.row_stride, a.k, a.out_stride = 1 << 18, 1 << 18, 20000, 20000
    assert L.lib.tidal_topk_static(C.byref(a), None, None) == L.ERR_ARG and "at most 16384" in L.last_error()
    hist = torch.zeros(4096, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s[:1], 8, out[:1], d_hist=hist.data_ptr()) == L.ERR_ARG
    # argument forms of tidal_topk that this entry point does not implement are refused, not ignored
    assert _static_topk(L, s[:1], 8, out[:1], seg_len=16, seg_stride=64) == L.ERR_ARG and "seg_len" in L.last_error()
    lens = torch.full((1,), 32, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s[:1], 8, out[:1], d_row_len=lens.data_ptr()) == L.ERR_ARG and "d_row_len" in L.last_error()


def test_static_topk_large_k_and_crowded_threshold_bin():
    """k above the position-ordered limit (sets compared), and more equal scores in the threshold
    bin than the array has candidate slots for (the kernel rescans the row instead)."""
    import tidaldecode_b200.ops as T
    from tidaldecode_b200 import _lib as L

    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(5)
    ws = T.Workspace(1, 1, 64, 2, 1 << 18)
    s = torch.randn(2, 100000, generator=g).cuda()
    got = torch.full((2, 8192), -1, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s, 8192, got) == 0, L.last_error()
    want = T.topk(s, 8192, ws)
    assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)
    s = torch.randn(1, 1 << 18, generator=g)
    s[0, torch.randperm(1 << 18, generator=g)[:40000]] = 2.5          # 40000 equal scores > 16384 candidate slots
    s = s.cuda()
    k = int((s > 2.5).sum()) + 10000                                 # the threshold falls inside the tie
    got = torch.full((1, k), -1, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s, k, got) == 0, L.last_error()
    want = T.topk(s, k, ws)
    assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)
    torch.cuda.synchronize()
    assert ws.status() == 0 and L.lib.tidal_topk_static_status(0, None) == 0


def test_static_topk_fault_word_can_be_read_and_cleared():
    from tidaldecode_b200 import _lib as L

    torch.cuda.set_device(0)
    assert L.lib.tidal_topk_static_status(1, None) == 0
    # NaN scores order above +inf and are legal; a clean call leaves the word at zero
    s = torch.randn(1, 4096, device="cuda")
    out = torch.zeros(1, 16, dtype=torch.int32, device="cuda")
    assert _static_topk(L, s, 16, out) == 0
    torch.cuda.synchronize()
    assert L.lib.tidal_topk_static_status(1, None) == 0


def test_static_topk_on_a_second_device():
    """The array's address is looked up per device; the first call on device 1 must not reuse device 0's."""
    import tidaldecode_b200.ops as T
    from tidaldecode_b200 import _lib as L

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with torch.cuda.device(1):
        s = torch.randn(2, 20000, device="cuda:1")
        got = torch.full((2, 64), -1, dtype=torch.int32, device="cuda:1")
        assert _static_topk(L, s, 64, got) == 0, L.last_error()
        ws = T.Workspace(1, 1, 64, 2, 20000, device="cuda:1")
        want = T.topk(s, 64, ws)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    torch.cuda.set_device(0)
