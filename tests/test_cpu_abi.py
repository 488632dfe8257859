"""CPU tier: the C-ABI library loads, exports every declared symbol, its structs
match the ctypes mirror, and host-side argument checks answer without a GPU."""
from __future__ import annotations

import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tidal_b200.h")


@pytest.fixture(scope="module")
def L():
    from tidaldecode_b200 import build
    build.build()
    from tidaldecode_b200 import _lib
    return _lib


def test_every_declared_symbol_is_exported(L):
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(tidal_[a-z_0-9]+)\s*\(", text))
    declared -= {"tidal_attn_args", "tidal_topk_args", "tidal_rope_append_args"}
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(L.lib, name), f"{name} declared in the header but not exported"
    assert set(L.EXPORTS) >= declared
    assert L.lib.tidal_version() >= 100


def test_struct_layouts_match_header(L, tmp_path):
    structs = {"tidal_attn_args": L.AttnArgs, "tidal_topk_args": L.TopkArgs, "tidal_rope_append_args": L.RopeAppendArgs,
               "tidal_linear_args": L.LinearArgs, "tidal_exchange_args": L.ExchangeArgs, "tidal_prefill_args": L.PrefillArgs}
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for cname, st in structs.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for f, _ in st._fields_:
            lines.append(f'printf("{cname}.{f} %zu\\n", offsetof({cname}, {f}));')
    lines.append("return 0;}")
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    got = dict(l.split() for l in out.strip().splitlines())
    for cname, st in structs.items():
        assert int(got[cname]) == C.sizeof(st), cname
        for f, _ in st._fields_:
            assert int(got[f"{cname}.{f}"]) == getattr(st, f).offset, f"{cname}.{f}"


def test_chunk_planner_is_pure_host_arithmetic(L):
    plan = L.lib.tidal_plan_chunks
    assert plan(1, 1, 32768, 4, 148) == 148          # one wave, one CTA per SM
    assert plan(8, 1, 1 << 20, 16, 148) == 18
    assert plan(1, 32, 257, 64, 148) == 4            # per-head lists: 148 // 32
    assert plan(1, 1, 256, 4, 148) == 64             # small lists are bounded by work
    assert plan(1, 1, 0, 4, 148) == 1
    assert plan(0, 1, 10, 4, 148) == L.ERR_ARG


def test_argument_errors_without_gpu(L):
    a = L.AttnArgs()
    assert L.lib.tidal_decode_attention(C.byref(a), None, 0, None) == L.ERR_ARG
    assert "q and kv" in L.last_error()
    a.d_q, a.d_kv, a.d_o = 0x1000, 0x2000, 0x3000
    a.batch, a.num_qo_heads, a.num_kv_heads, a.head_dim, a.page_size, a.num_pages = 1, 32, 5, 128, 1, 10
    assert L.lib.tidal_decode_attention(C.byref(a), None, 0, None) == L.ERR_ARG
    assert "multiple" in L.last_error()                 # reference: std::invalid_argument, decode_attn.cuh:1143-1148
    a.num_kv_heads, a.head_dim = 32, 96
    assert L.lib.tidal_decode_attention(C.byref(a), None, 0, None) == L.ERR_ARG
    assert "head_dim" in L.last_error()
    a.head_dim, a.extra_page = 128, -1
    # a workspace that was never initialised is refused before anything is launched
    # (reference: std::runtime_error when forward precedes begin_forward, decode_handler.cuh:228-233)
    assert L.lib.tidal_decode_attention(C.byref(a), 0x4000, 1 << 20, None) == L.ERR_WORKSPACE
    t = L.TopkArgs()
    assert L.lib.tidal_topk(C.byref(t), 0x4000, 1 << 20, None) == L.ERR_ARG
    lin = L.LinearArgs()
    assert L.lib.tidal_decode_linear(C.byref(lin), None) == L.ERR_ARG          # null pointers
    lin.d_x = lin.d_w = lin.d_y = 256
    lin.M, lin.N, lin.K, lin.dtype = 9, 16, 64, L.DTYPE_F16
    assert L.lib.tidal_decode_linear(C.byref(lin), None) == L.ERR_ARG and "M 9" in L.last_error()
    lin.M, lin.K = 1, 12
    assert L.lib.tidal_decode_linear(C.byref(lin), None) == L.ERR_ARG and "multiple of 8" in L.last_error()
    lin.K, lin.N, lin.epilogue = 64, 15, L.LINEAR_SILU_MUL
    assert L.lib.tidal_decode_linear(C.byref(lin), None) == L.ERR_ARG and "even N" in L.last_error()
    rq = L.RopeAppendArgs()
    assert L.lib.tidal_decode_qkv(C.byref(lin), C.byref(rq), None) == L.ERR_ARG            # no q output, no pool
    lin.K, lin.N, lin.epilogue, lin.M = 256, (8 + 2 * 2) * 64, L.LINEAR_PLAIN, 2
    rq.d_q = rq.d_kv = 256
    rq.batch, rq.tokens_per_seq, rq.num_qo_heads, rq.num_kv_heads, rq.head_dim, rq.dtype = 2, 1, 8, 2, 64, L.DTYPE_F32
    assert L.lib.tidal_decode_qkv(C.byref(lin), C.byref(rq), None) == L.ERR_ARG and "f16/bf16" in L.last_error()
    rq.dtype, rq.num_kv_heads = L.DTYPE_F16, 4
    assert L.lib.tidal_decode_qkv(C.byref(lin), C.byref(rq), None) == L.ERR_ARG and "rows" in L.last_error()
    x = L.ExchangeArgs()
    assert L.lib.tidal_peer_all_gather(C.byref(x), None) == L.ERR_ARG
    x.d_send = x.d_recv = x.d_peer_stage = x.d_peer_count = x.d_state = 256
    x.world, x.rank, x.bytes, x.slot_bytes = 1, 0, 64, 64
    assert L.lib.tidal_peer_all_gather(C.byref(x), None) == L.ERR_ARG and "world" in L.last_error()
    x.world, x.bytes = 2, 72
    assert L.lib.tidal_peer_all_gather(C.byref(x), None) == L.ERR_ARG and "multiples of 16" in L.last_error()
    pf = L.PrefillArgs()
    assert L.lib.tidal_prefill(C.byref(pf), None) == L.ERR_ARG
    pf.d_q = pf.d_o = pf.d_kv = pf.d_page_table = 256
    pf.dtype, pf.head_dim, pf.num_qo_heads, pf.num_kv_heads, pf.page_size, pf.n_q, pf.kv_len = 7, 128, 8, 2, 1, 4, 4
    assert L.lib.tidal_prefill(C.byref(pf), None) == L.ERR_ARG and "dtype" in L.last_error()
    pf.dtype = L.DTYPE_F32
    assert L.lib.tidal_prefill(C.byref(pf), None) == L.ERR_ARG and "num_pages" in L.last_error()     # the bounds of the page table entries
    pf.num_pages = 16
    pf.dtype, pf.head_dim = L.DTYPE_BF16, 96
    assert L.lib.tidal_prefill(C.byref(pf), None) == L.ERR_ARG and "head_dim" in L.last_error()
    pf.head_dim, pf.num_kv_heads = 128, 3
    assert L.lib.tidal_prefill(C.byref(pf), None) == L.ERR_ARG and "multiple" in L.last_error()
    pf.num_kv_heads, pf.kv_len = 2, 3          # the cache must already hold the new rows
    assert L.lib.tidal_prefill(C.byref(pf), None) == L.ERR_ARG and "kv_len" in L.last_error()
    r = L.RopeAppendArgs()
    assert L.lib.tidal_rope_append(C.byref(r), None) == L.ERR_ARG
    pm = L.PageMetaArgs()
    assert L.lib.tidal_update_page_meta(C.byref(pm), None) == L.ERR_ARG
    pm.d_kv = pm.d_meta = 256
    pm.batch, pm.num_kv_heads, pm.head_dim, pm.page_size, pm.meta_page_size, pm.num_pages, pm.num_meta_pages = 1, 8, 128, 16, 16, 4, 1
    pm.seq_len, pm.first_pos = 10, 10
    assert L.lib.tidal_update_page_meta(C.byref(pm), None) == L.ERR_ARG and "first_pos" in L.last_error()
    es = L.EstimateArgs()
    assert L.lib.tidal_estimate(C.byref(es), None) == L.ERR_ARG
    es.d_q = es.d_meta = es.d_out = 256
    es.batch, es.num_qo_heads, es.num_kv_heads, es.head_dim, es.meta_page_size, es.num_meta_pages = 1, 8, 3, 128, 16, 1
    assert L.lib.tidal_estimate(C.byref(es), None) == L.ERR_ARG and "multiple" in L.last_error()
    es.num_kv_heads, es.n_entries, es.out_stride = 8, 5, 4
    assert L.lib.tidal_estimate(C.byref(es), None) == L.ERR_ARG and "out_stride" in L.last_error()
    assert L.lib.tidal_ws_bytes(1, 32, 128, 32, 32768) > 0
    assert L.lib.tidal_ws_bytes(0, 32, 128, 32, 32768) == 0
    assert L.lib.tidal_ws_init(None, 0, 1, 32, 128, 32, 32768, None) == L.ERR_ARG
    with pytest.raises(RuntimeError):
        L.check(L.ERR_ARG, "x")


def test_missing_library_fails_loudly(tmp_path):
    """No CPU or PyTorch fallback: without the shared library the import raises."""
    code = (
        "import importlib.util, sys\n"
        f"spec = importlib.util.spec_from_file_location('x', r'{os.path.join(ROOT, 'tidaldecode_b200', '_lib.py')}')\n"
        "m = importlib.util.module_from_spec(spec)\n"
        f"import os; os.path.exists = (lambda p, _e=os.path.exists: False if p.endswith('libtidal_b200.so') else _e(p))\n"
        "try:\n    spec.loader.exec_module(m)\nexcept ImportError as e:\n    print('IMPORTERROR', e); sys.exit(0)\nsys.exit(1)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode == 0 and "IMPORTERROR" in r.stdout, r.stdout + r.stderr
