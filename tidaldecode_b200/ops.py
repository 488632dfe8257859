"""Tensor-level wrappers of the C ABI: torch supplies device memory and the
current stream, every computation happens in libtidal_b200.so.

These are the calls the reference-shaped layers (`tidaldecode_b200.utils`,
`tidaldecode_b200.models`) are written on; they add batch > 1, GQA, bf16/fp32,
head-summed selection scores and sequence-sharded KV to what the reference's
operators offer (tidal/utils/__init__.py:26-287).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import AttnArgs, RopeAppendArgs, TopkArgs, check, lib

_DTYPES = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {t.dtype} (float16, bfloat16, float32)") from None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("tidaldecode_b200 runs on CUDA tensors only (there is no CPU path)")
        if t is not None and not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")


class Workspace:
    """Caller-owned scratch for the split-KV partials and the top-k, allocated once
    (the reference allocates per call: decode_handler.cuh:104-117, controller.py:149-168)."""

    def __init__(self, max_batch: int, num_qo_heads: int, head_dim: int, max_rows: int, max_n: int, device="cuda"):
        self.geometry = (int(max_batch), int(num_qo_heads), int(head_dim), int(max_rows), int(max_n))
        self.nbytes = lib.tidal_ws_bytes(*self.geometry)
        if self.nbytes == 0:
            raise RuntimeError(f"bad workspace geometry {self.geometry}: {_lib.last_error()}")
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        if self.buf.data_ptr() % 256:
            raise RuntimeError("allocator returned a buffer that is not 256-byte aligned")
        self.max_rows = int(max_rows)
        # per-row first-digit histograms the attention kernel may fill for the top-k
        self.hist = torch.zeros((max_rows, _lib.TOPK_BINS), dtype=torch.int32, device=device)
        self.reset()

    def reset(self) -> None:
        with torch.cuda.device(self.buf.device):
            check(lib.tidal_ws_init(self.buf.data_ptr(), self.nbytes, *self.geometry, _stream()), "tidal_ws_init")
        self.hist.zero_()

    def status(self) -> int:
        """Blocking read of the device-side fault bits (0 = clean)."""
        with torch.cuda.device(self.buf.device):
            rc = lib.tidal_ws_status(self.buf.data_ptr(), self.nbytes, _stream())
        check(rc, "tidal_ws_status")
        return rc

    def __del__(self):
        try:
            lib.tidal_ws_release(self.buf.data_ptr())
        except Exception:
            pass


def decode_attention(
    q: torch.Tensor,                 # [B, Hq, D]
    kv: torch.Tensor,                # [pages, 2, page_size, Hkv, D]
    seq_len: int,
    ws: Workspace,
    *,
    out: Optional[torch.Tensor] = None,
    page_table: Optional[torch.Tensor] = None,   # int32 [B, max_pages]
    pages_per_seq: Optional[int] = None,          # identity mapping: sequence b starts at page b*pages_per_seq
    seq_lens: Optional[torch.Tensor] = None,      # int32 [B]
    sel_idx: Optional[torch.Tensor] = None,       # int32 [B, k] or [B, Hq, k]
    sel_counts: Optional[torch.Tensor] = None,    # int32 [B] or [B, Hq]
    sel_physical: bool = False,
    extra_page: int = -1,
    scores: Optional[torch.Tensor] = None,        # fp32 [B, N] (head-summed) or [B, Hq, N]
    hist: Optional[torch.Tensor] = None,          # int32 [rows, 4096] zeroed, rows = B or B*Hq
    force_last: bool = False,
    partials: Optional[tuple] = None,             # (m [B,Hq], l [B,Hq], o [B,Hq,D]) fp32 outputs
    sm_scale: float = 0.0,
    num_chunks: int = 0,
    heads_per_cta: int = 0,
    use_tensor_cores: int = 0,
    want_out: bool = True,
) -> Optional[torch.Tensor]:
    """One decode step of attention; see tidal_decode_attention in include/tidal_b200.h."""
    _need_cuda(q, kv, out, page_table, seq_lens, sel_idx, sel_counts, scores, hist)
    if q.dim() != 3 or kv.dim() != 5 or kv.shape[1] != 2:
        raise RuntimeError("q must be [B,Hq,D] and kv [pages,2,page_size,Hkv,D]")
    if kv.dtype != q.dtype:
        raise RuntimeError("q and kv must share a dtype")
    B, Hq, D = q.shape
    pages, _, page_size, Hkv, Dk = kv.shape
    if Dk != D:
        raise RuntimeError("head_dim of q and kv differ")
    if out is None and want_out:
        out = torch.empty_like(q)
    a = AttnArgs()
    a.d_q, a.d_o, a.d_kv = q.data_ptr(), _ptr(out), kv.data_ptr()
    if page_table is not None:
        if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.shape[0] != B:
            raise RuntimeError("page_table must be int32 [B, max_pages]")
        a.d_page_table, a.page_table_stride = page_table.data_ptr(), page_table.shape[1]
    else:
        a.d_page_table = None
        a.page_table_stride = pages_per_seq if pages_per_seq is not None else (pages // B)
    a.d_seq_lens, a.seq_len = _ptr(seq_lens), int(seq_len)
    if sel_idx is not None:
        if sel_idx.dtype != torch.int32:
            raise RuntimeError("sel_idx must be int32")
        if sel_idx.dim() == 2:
            a.sel_rows = 1
        elif sel_idx.dim() == 3 and sel_idx.shape[1] == Hq:
            a.sel_rows = Hq
        else:
            raise RuntimeError("sel_idx must be [B,k] or [B,Hq,k]")
        a.d_sel_idx, a.sel_count, a.sel_stride = sel_idx.data_ptr(), sel_idx.shape[-1], sel_idx.shape[-1]
        a.sel_physical = 1 if sel_physical else 0
        a.d_sel_counts = _ptr(sel_counts)
    a.extra_page = int(extra_page)
    if scores is not None:
        if scores.dtype != torch.float32:
            raise RuntimeError("scores must be float32")
        a.d_scores = scores.data_ptr()
        a.score_rows = 1 if scores.dim() == 2 else Hq
        a.score_stride = scores.shape[-1]
        if hist is not None:
            a.d_hist = hist.data_ptr()
        a.force_last = 1 if force_last else 0
    if partials is not None:
        m, l, o = partials
        _need_cuda(m, l, o)
        a.d_part_m, a.d_part_l, a.d_part_o = m.data_ptr(), l.data_ptr(), o.data_ptr()
    a.batch, a.num_qo_heads, a.num_kv_heads, a.head_dim = B, Hq, Hkv, D
    a.page_size, a.dtype, a.num_pages = page_size, _dtype_code(q), pages
    a.sm_scale, a.num_chunks, a.heads_per_cta = float(sm_scale), int(num_chunks), int(heads_per_cta)
    a.use_tensor_cores = int(use_tensor_cores)
    with torch.cuda.device(q.device):
        check(lib.tidal_decode_attention(C.byref(a), ws.buf.data_ptr(), ws.nbytes, _stream()), "tidal_decode_attention")
    return out


def topk(
    scores: torch.Tensor,            # fp32 [rows, n] (any leading dims are flattened)
    k: int,
    ws: Workspace,
    *,
    n: Optional[int] = None,
    in_idx: Optional[torch.Tensor] = None,
    out_idx: Optional[torch.Tensor] = None,
    out_val: Optional[torch.Tensor] = None,
    idx_offset: int = 0,
    force_last: bool = False,
    own_range: Optional[tuple] = None,
    out_count: Optional[torch.Tensor] = None,
    hist: Optional[torch.Tensor] = None,
    segments: Optional[tuple] = None,     # (rows, seg_len, seg_stride, row_stride): rows scattered over equal blocks
    row_len: Optional[torch.Tensor] = None,   # int32 [rows] on the device; n is then their upper bound
) -> torch.Tensor:
    """Row-wise top-k index sets; see tidal_topk in include/tidal_b200.h."""
    _need_cuda(out_idx, out_val, out_count, hist)
    if scores.dtype != torch.float32:
        raise RuntimeError("scores must be float32")
    if segments is not None:
        rows, seg_len, seg_stride, stride = (int(x) for x in segments)
        if n is None:
            raise RuntimeError("segmented rows need n")
    else:
        _need_cuda(scores, in_idx)
        stride = scores.shape[-1]
        rows = scores.numel() // stride
    n = stride if n is None else int(n)
    kk = min(int(k), n)
    if out_idx is None:
        out_idx = torch.empty((rows, kk) if segments is not None else scores.shape[:-1] + (kk,), dtype=torch.int32,
                              device=scores.device)
    if out_idx.dtype != torch.int32:
        raise RuntimeError("out_idx must be int32")
    a = TopkArgs()
    a.d_scores, a.d_in_idx, a.rows, a.n, a.row_stride, a.k = scores.data_ptr(), _ptr(in_idx), rows, n, stride, int(k)
    if in_idx is not None:
        if in_idx.dtype != torch.int32:
            raise RuntimeError("in_idx must be int32")
        a.in_idx_stride = stride if segments is not None else (0 if in_idx.dim() == 1 else in_idx.shape[-1])
    if segments is not None:
        a.seg_len, a.seg_stride = seg_len, seg_stride
    a.d_out_idx, a.d_out_val, a.out_stride = out_idx.data_ptr(), _ptr(out_val), out_idx.shape[-1]
    a.idx_offset, a.force_last = int(idx_offset), 1 if force_last else 0
    if own_range is not None:
        a.own_lo, a.own_hi = int(own_range[0]), int(own_range[1])
    a.d_out_count, a.d_hist = _ptr(out_count), _ptr(hist)
    a.d_row_len = _ptr(row_len)
    with torch.cuda.device(scores.device):
        check(lib.tidal_topk(C.byref(a), ws.buf.data_ptr(), ws.nbytes, _stream()), "tidal_topk")
    return out_idx


def rope_append(
    q: Optional[torch.Tensor],       # [n_tokens, Hq, D], rotated in place
    k: torch.Tensor,                 # [n_tokens, Hkv, D]
    v: Optional[torch.Tensor],       # [n_tokens, Hkv, D]
    kv: Optional[torch.Tensor],      # pool [pages, 2, page_size, Hkv, D] or None (rotate only)
    *,
    batch: int = 1,
    pos0: int = 0,
    pos0_dev: Optional[torch.Tensor] = None,
    page_table: Optional[torch.Tensor] = None,
    pages_per_seq: Optional[int] = None,
    rope_theta: float = 1e4,
    rope_scale: float = 1.0,
    rope_mode: int = 1,
    inv_freq: Optional[torch.Tensor] = None,
    rotate_k_in_place: bool = True,
    status: Optional[torch.Tensor] = None,
    q_src: Optional[torch.Tensor] = None,         # [n_tokens, Hq, D]: read the queries here, write them rotated to q
    kv_pos_base: int = 0,                         # position held by the pool's first slot per sequence (a shard's lo)
) -> None:
    """RoPE on q and k fused with the KV append; see tidal_rope_append in include/tidal_b200.h."""
    _need_cuda(q, k, v, kv, pos0_dev, page_table, inv_freq, status, q_src)
    if q_src is not None and (q is None or q_src.shape != q.shape or q_src.dtype != q.dtype):
        raise RuntimeError("q_src must have the shape and dtype of q")
    if k.dim() != 3:
        raise RuntimeError("k must be [n_tokens, Hkv, D]")
    n_tokens, Hkv, D = k.shape
    if n_tokens % batch:
        raise RuntimeError("n_tokens must be a multiple of batch")
    a = RopeAppendArgs()
    a.d_q, a.d_k, a.d_v, a.d_kv = _ptr(q), k.data_ptr(), _ptr(v), _ptr(kv)
    if page_table is not None:
        a.d_page_table, a.page_table_stride = page_table.data_ptr(), page_table.shape[1]
    elif kv is not None:
        a.page_table_stride = pages_per_seq if pages_per_seq is not None else kv.shape[0] // batch
    a.d_pos0, a.pos0, a.d_inv_freq = _ptr(pos0_dev), int(pos0), _ptr(inv_freq)
    a.rope_theta, a.rope_scale, a.rope_mode = float(rope_theta), float(rope_scale), int(rope_mode)
    a.rotate_k_in_place = 1 if rotate_k_in_place else 0
    a.batch, a.tokens_per_seq = int(batch), n_tokens // batch
    a.num_qo_heads = q.shape[1] if q is not None else 0
    a.num_kv_heads, a.head_dim = Hkv, D
    a.page_size = kv.shape[2] if kv is not None else 1
    a.num_pages = kv.shape[0] if kv is not None else 1
    a.dtype = _dtype_code(k)
    a.d_status = _ptr(status)
    a.d_q_src = _ptr(q_src)
    a.kv_pos_base = int(kv_pos_base)
    with torch.cuda.device(k.device):
        check(lib.tidal_rope_append(C.byref(a), _stream()), "tidal_rope_append")


def update_page_meta(kv: torch.Tensor, meta: torch.Tensor, seq_len: int, first_pos: int, *, batch: int = 1,
                     page_table: Optional[torch.Tensor] = None, pages_per_seq: Optional[int] = None,
                     meta_table: Optional[torch.Tensor] = None, meta_pages_per_seq: Optional[int] = None,
                     status: Optional[torch.Tensor] = None) -> None:
    """Per-page key bounds (Quest metadata) of the KV pages that hold positions [first_pos, seq_len), recomputed
    from the pool; see tidal_update_page_meta in include/tidal_b200.h.  kv [pages,2,page,Hkv,D],
    meta [meta_pages,2,meta_page,Hkv,D] (plane 0 maxima, plane 1 minima, one entry per KV page)."""
    _need_cuda(kv, meta, page_table, meta_table, status)
    if kv.dim() != 5 or meta.dim() != 5 or kv.shape[1] != 2 or meta.shape[1] != 2 or kv.shape[3:] != meta.shape[3:] or kv.dtype != meta.dtype:
        raise RuntimeError("kv and meta must be [pages,2,page,Hkv,D] pools of one dtype and head geometry")
    a = _lib.PageMetaArgs()
    a.d_kv, a.d_meta = kv.data_ptr(), meta.data_ptr()
    if page_table is not None:
        a.d_page_table, a.page_table_stride = page_table.data_ptr(), page_table.shape[-1]
    else:
        a.page_table_stride = pages_per_seq if pages_per_seq is not None else kv.shape[0] // batch
    if meta_table is not None:
        a.d_meta_table, a.meta_table_stride = meta_table.data_ptr(), meta_table.shape[-1]
    else:
        a.meta_table_stride = meta_pages_per_seq if meta_pages_per_seq is not None else meta.shape[0] // batch
    a.batch, a.num_kv_heads, a.head_dim = int(batch), kv.shape[3], kv.shape[4]
    a.page_size, a.meta_page_size, a.dtype = kv.shape[2], meta.shape[2], _dtype_code(kv)
    a.num_pages, a.num_meta_pages = kv.shape[0], meta.shape[0]
    a.first_pos, a.seq_len = int(first_pos), int(seq_len)
    a.d_status = _ptr(status)
    with torch.cuda.device(kv.device):
        check(lib.tidal_update_page_meta(C.byref(a), _stream()), "tidal_update_page_meta")


def estimate(q: torch.Tensor, meta: torch.Tensor, n_entries: int, *, out: Optional[torch.Tensor] = None,
             meta_table: Optional[torch.Tensor] = None, meta_pages_per_seq: Optional[int] = None,
             status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Quest's upper bound of q.k per KV page from the page metadata; see tidal_estimate in include/tidal_b200.h.
    q [B,Hq,D]; returns out [B,Hq,>= n_entries] (q's dtype unless `out` is given)."""
    _need_cuda(q, meta, out, meta_table, status)
    if q.dim() != 3 or meta.dim() != 5 or meta.shape[1] != 2 or meta.shape[4] != q.shape[2] or meta.dtype != q.dtype:
        raise RuntimeError("q must be [B,Hq,D] and meta [meta_pages,2,meta_page,Hkv,D] of the same dtype")
    B, Hq, D = q.shape
    if out is None:
        out = torch.empty(B, Hq, max(int(n_entries), 1), dtype=q.dtype, device=q.device)
    a = _lib.EstimateArgs()
    a.d_q, a.d_meta, a.d_out, a.out_stride = q.data_ptr(), meta.data_ptr(), out.data_ptr(), out.shape[-1]
    if meta_table is not None:
        a.d_meta_table, a.meta_table_stride = meta_table.data_ptr(), meta_table.shape[-1]
    else:
        a.meta_table_stride = meta_pages_per_seq if meta_pages_per_seq is not None else meta.shape[0] // B
    a.batch, a.num_qo_heads, a.num_kv_heads, a.head_dim = B, Hq, meta.shape[3], D
    a.meta_page_size, a.n_entries, a.dtype, a.out_dtype = meta.shape[2], int(n_entries), _dtype_code(q), _dtype_code(out)
    a.num_meta_pages, a.d_status = meta.shape[0], _ptr(status)
    with torch.cuda.device(q.device):
        check(lib.tidal_estimate(C.byref(a), _stream()), "tidal_estimate")
    return out


def merge_partials(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor, dtype: torch.dtype,
                   out: Optional[torch.Tensor] = None, geometry: Optional[tuple] = None) -> torch.Tensor:
    """LSE-merge of [shards, B, Hq(, D)] partials; see tidal_merge_partials.  With
    geometry = (shards, B, Hq, D, shard_stride) the three tensors are views whose first element is
    shard 0's block and whose shards lie shard_stride elements apart (a packed receive buffer)."""
    if geometry is None:
        _need_cuda(m, l, o, out)
        shards, B, Hq, D = o.shape
        stride = 0
    else:
        shards, B, Hq, D, stride = (int(x) for x in geometry)
    if out is None:
        out = torch.empty((B, Hq, D), dtype=dtype, device=o.device)
    with torch.cuda.device(o.device):
        check(lib.tidal_merge_partials_strided(m.data_ptr(), l.data_ptr(), o.data_ptr(), stride, shards, B, Hq, D,
                                               out.data_ptr(), _DTYPES[dtype], _stream()), "tidal_merge_partials")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
             round_before_weight: bool = True) -> torch.Tensor:
    """RMSNorm over the last dimension; see tidal_rms_norm in include/tidal_b200.h."""
    _need_cuda(x, weight, out)
    if weight.dtype != x.dtype:
        raise RuntimeError("input and weight must share a dtype")
    hidden = x.shape[-1]
    if weight.numel() != hidden:
        raise RuntimeError("weight length differs from the last dimension of the input")
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib.tidal_rms_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), x.numel() // hidden, hidden, float(eps),
                                 _dtype_code(x), 1 if round_before_weight else 0, _stream()), "tidal_rms_norm")
    return out


def prefill(q: torch.Tensor, kv_pool: torch.Tensor, page_table: torch.Tensor, kv_len: int, *, causal: bool = True,
            sm_scale: float = 0.0, out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the new rows q [n_q, Hq, D] of one sequence over its paged KV (which already
    holds their K,V); see tidal_prefill in include/tidal_b200.h.  kv_pool [pages, 2, page_size, Hkv, D],
    page_table int32 [>= ceil(kv_len / page_size)]; f16/bf16 (tensor cores) or f32 (CUDA cores), D 64 or 128."""
    _need_cuda(q, kv_pool, page_table, out, status)
    if q.dim() != 3 or kv_pool.dim() != 5 or kv_pool.shape[1] != 2:
        raise RuntimeError("q must be [n_q, Hq, D] and kv_pool [pages, 2, page_size, Hkv, D]")
    if kv_pool.dtype != q.dtype or page_table.dtype != torch.int32:
        raise RuntimeError("q and kv_pool must share a dtype, page_table must be int32")
    if not (q.is_contiguous() and kv_pool.is_contiguous() and page_table.is_contiguous()):
        raise RuntimeError("q, kv_pool and page_table must be contiguous")
    n_q, Hq, D = q.shape
    page_size, Hkv = kv_pool.shape[2], kv_pool.shape[3]
    if kv_pool.shape[4] != D:
        raise RuntimeError("q and kv_pool disagree on head_dim")
    if page_table.numel() * page_size < kv_len:
        raise RuntimeError("page_table does not cover kv_len tokens")
    if out is None:
        out = torch.empty_like(q)
    a = _lib.PrefillArgs()
    a.d_q, a.d_o, a.d_kv, a.d_page_table = q.data_ptr(), out.data_ptr(), kv_pool.data_ptr(), page_table.data_ptr()
    a.d_status = status.data_ptr() if status is not None else None
    a.kv_len, a.n_q, a.num_qo_heads, a.num_kv_heads, a.head_dim = int(kv_len), n_q, Hq, Hkv, D
    a.page_size, a.dtype, a.causal, a.sm_scale = page_size, _dtype_code(q), 1 if causal else 0, float(sm_scale)
    a.num_pages = kv_pool.shape[0]
    with torch.cuda.device(q.device):
        check(lib.tidal_prefill(C.byref(a), _stream()), "tidal_prefill")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, *, out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
           norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6, round_before_weight: bool = True,
           silu_mul: bool = False, static_weights: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode-step projection y = x W^T for up to 8 rows of x, with the optional RMSNorm of x, residual
    add and SiLU(gate) * up folded in; see tidal_decode_linear in include/tidal_b200.h.
    x [..., K] (at most 8 rows in all), weight [N, K]; returns [..., N] (or [..., N/2] with silu_mul)."""
    _need_cuda(x, weight, out, residual, norm_weight)
    if weight.dtype != x.dtype or weight.dim() != 2:
        raise RuntimeError("weight must be a [N, K] matrix of the input's dtype")
    N, K = weight.shape
    if x.shape[-1] != K:
        raise RuntimeError(f"input has {x.shape[-1]} features, the weight {K}")
    M = x.numel() // K
    if not (x.is_contiguous() and weight.is_contiguous()):
        raise RuntimeError("input and weight must be contiguous")
    n_out = N // 2 if silu_mul else N
    if out is None:
        out = torch.empty(*x.shape[:-1], n_out, dtype=x.dtype, device=x.device)
    elif out.numel() != M * n_out or out.dtype != x.dtype or not out.is_contiguous():
        raise RuntimeError("out has the wrong size, dtype or layout")
    if residual is not None and (residual.numel() != M * n_out or residual.dtype != x.dtype or not residual.is_contiguous()):
        raise RuntimeError("residual has the wrong size, dtype or layout")
    if norm_weight is not None and (norm_weight.numel() != K or norm_weight.dtype != x.dtype):
        raise RuntimeError("norm weight must have K elements of the input's dtype")
    a = _lib.LinearArgs()
    a.d_x, a.d_w, a.d_y = x.data_ptr(), weight.data_ptr(), out.data_ptr()
    a.d_residual = _ptr(residual)
    a.d_norm_weight = _ptr(norm_weight)
    a.norm_eps, a.norm_round_before_weight = float(eps), 1 if round_before_weight else 0
    a.M, a.N, a.K, a.dtype = M, N, K, _dtype_code(x)
    a.epilogue = _lib.LINEAR_SILU_MUL if silu_mul else _lib.LINEAR_PLAIN
    a.static_weights = 1 if static_weights else 0       # model weights: may be fetched ahead of stream order
    a.d_status = _ptr(status)                           # uint32 [1], fault bits are OR-ed in
    with torch.cuda.device(x.device):
        check(lib.tidal_decode_linear(C.byref(a), _stream()), "tidal_decode_linear")
    return out


def qkv_rope_append(x: torch.Tensor, weight: torch.Tensor, q_out: torch.Tensor, kv: torch.Tensor, *,
                    num_kv_heads: int, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                    round_before_weight: bool = True, pos0: int = 0, pos0_dev: Optional[torch.Tensor] = None,
                    page_table: Optional[torch.Tensor] = None, pages_per_seq: Optional[int] = None, rope_theta: float = 1e4,
                    rope_scale: float = 1.0, rope_mode: int = 1, inv_freq: Optional[torch.Tensor] = None,
                    static_weights: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The q|k|v projection of one new token per sequence with RoPE and the KV append folded in; see
    tidal_decode_qkv in include/tidal_b200.h.  x [B, K]; weight [(Hq + 2 Hkv) D, K] (q heads, k heads, v
    heads); q_out [B, Hq, D] receives the rotated queries; k and v land in the pool."""
    _need_cuda(x, weight, q_out, kv, norm_weight, pos0_dev, page_table, inv_freq, status)
    B, Hq, D = q_out.shape
    N, K = weight.shape
    if x.numel() != B * K or weight.dtype != x.dtype or q_out.dtype != x.dtype or kv.dtype != x.dtype:
        raise RuntimeError("x must be [B, K] and share its dtype with the weight, q_out and the pool")
    a = _lib.LinearArgs()
    a.d_x, a.d_w = x.data_ptr(), weight.data_ptr()
    a.d_norm_weight = _ptr(norm_weight)
    a.norm_eps, a.norm_round_before_weight = float(eps), 1 if round_before_weight else 0
    a.M, a.N, a.K, a.dtype = B, N, K, _dtype_code(x)
    a.static_weights = 1 if static_weights else 0
    r = RopeAppendArgs()
    r.d_q, r.d_kv = q_out.data_ptr(), kv.data_ptr()
    if page_table is not None:
        r.d_page_table, r.page_table_stride = page_table.data_ptr(), page_table.shape[1]
    else:
        r.page_table_stride = pages_per_seq if pages_per_seq is not None else kv.shape[0] // B
    r.d_pos0, r.pos0, r.d_inv_freq = _ptr(pos0_dev), int(pos0), _ptr(inv_freq)
    r.rope_theta, r.rope_scale, r.rope_mode = float(rope_theta), float(rope_scale), int(rope_mode)
    r.batch, r.tokens_per_seq = B, 1
    r.num_qo_heads, r.num_kv_heads, r.head_dim = Hq, int(num_kv_heads), D
    r.page_size, r.num_pages = kv.shape[2], kv.shape[0]
    r.dtype = _dtype_code(x)
    r.d_status = _ptr(status)
    with torch.cuda.device(x.device):
        check(lib.tidal_decode_qkv(C.byref(a), C.byref(r), _stream()), "tidal_decode_qkv")
    return q_out


class PeerExchange:
    """Buffers and peer mappings of tidal_peer_all_gather for one process group: staging and arrival
    flag words live in symmetric memory (torch.distributed._symmetric_memory: CUDA memory mapped on every
    rank of the group), the pointer tables on the device.  One object per (group, slot size); every rank
    must construct it at the same point of the program (the constructor is a collective)."""

    def __init__(self, slot_bytes: int, group, device, wait_limit: int = 0):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.group = group
        stage_bytes, count_off = self._geometry(slot_bytes, self.world)
        with torch.cuda.device(device):
            self.buf = symm_mem.empty(count_off + self._flag_bytes(self.world), dtype=torch.uint8, device=device)
            self.buf.zero_()
            hdl = symm_mem.rendezvous(self.buf, group)
            self._hdl = hdl
            self._tables([int(p) for p in hdl.buffer_ptrs], count_off, device)
            torch.cuda.synchronize()
        self.wait_limit = int(wait_limit)
        dist.barrier(group)                      # every rank's flag words are zero before anyone writes to them

    @staticmethod
    def _flag_bytes(world: int) -> int:
        return 2 * world * _lib.XCHG_MAX_CTAS * 4          # one flag word per (parity, source rank, CTA)

    def _geometry(self, slot_bytes: int, world: int):
        if slot_bytes % 16:
            raise RuntimeError("slot_bytes must be a multiple of 16")
        self.slot_bytes = int(slot_bytes)
        stage_bytes = 2 * world * self.slot_bytes
        return stage_bytes, (stage_bytes + 255) // 256 * 256

    def _tables(self, ptrs, count_off: int, device) -> None:
        i64 = dict(dtype=torch.int64, device=device)
        self.peer_stage = torch.tensor(ptrs, **i64)
        self.peer_count = torch.tensor([p + count_off for p in ptrs], **i64)
        self._own_count = ptrs[self.rank] + count_off
        self.state = torch.zeros(4, dtype=torch.int32, device=device)

    @classmethod
    def loopback(cls, slot_bytes: int, world: int, device, wait_limit: int = 0) -> "PeerExchange":
        """Rank 0 of a `world`-rank exchange whose every table entry is this GPU's own buffer: no other
        rank exists, so an exchange completes only if the missing ranks' blocks and flags were written by the
        host beforehand (`stage`, `flags`), and otherwise runs into its wait limit.  For tests of the
        timeout and reset behaviour on one GPU; nothing in it waits on another kernel."""
        self = cls.__new__(cls)
        self.world, self.rank, self.group, self._hdl = int(world), 0, None, None
        stage_bytes, count_off = self._geometry(slot_bytes, self.world)
        with torch.cuda.device(device):
            self.buf = torch.zeros(count_off + self._flag_bytes(self.world), dtype=torch.uint8, device=device)
            self._tables([self.buf.data_ptr()] * self.world, count_off, device)
        self.wait_limit = int(wait_limit)
        self.stage = self.buf[:stage_bytes].view(2, self.world, self.slot_bytes)       # [parity][rank][slot]
        self.flags = self.buf[count_off:count_off + self._flag_bytes(self.world)].view(torch.int32).view(
            2, self.world, _lib.XCHG_MAX_CTAS)                                          # [parity][source rank][CTA]
        return self

    def reset(self) -> None:
        """Flag words and exchange count back to zero after a timed-out exchange.  A collective in
        effect: every rank calls it, with none of the group's exchanges in flight."""
        import torch.distributed as dist

        if self.group is not None:
            torch.cuda.synchronize()
            dist.barrier(self.group)
        with torch.cuda.device(self.state.device):
            check(lib.tidal_peer_exchange_reset(self._own_count, self.state.data_ptr(), self.world, _stream()),
                  "tidal_peer_exchange_reset")
        if self.group is not None:
            torch.cuda.synchronize()
            dist.barrier(self.group)

    def all_gather(self, send: torch.Tensor, recv: Optional[torch.Tensor], nbytes: Optional[int] = None,
                   status: Optional[torch.Tensor] = None, merge: Optional[tuple] = None,
                   candidates: Optional[dict] = None) -> None:
        """recv [world, slot] (any dtype, slot_bytes per row) <- the first nbytes of every rank's `send`.
        merge = (out [rows, D], m_off, l_off, o_off): the blocks hold softmax partials at these fp32 word offsets
        and their merge goes to `out` in the same launch; recv may then be None.
        candidates = dict(rows, k, select, score_off, idx_off, own=(lo, hi), out=int32 [rows, >= select],
        count=int32 [rows]): the blocks also hold top-k candidates, ranked in the same launch (see
        tidal_exchange_args in include/tidal_b200.h)."""
        _need_cuda(send, recv, status)
        nbytes = send.numel() * send.element_size() if nbytes is None else int(nbytes)
        if recv is not None and recv.numel() * recv.element_size() < self.world * self.slot_bytes:
            raise RuntimeError("recv is smaller than world x slot_bytes")
        a = _lib.ExchangeArgs()
        a.d_send, a.d_recv, a.bytes, a.slot_bytes = send.data_ptr(), _ptr(recv), nbytes, self.slot_bytes
        if merge is not None:
            out, m_off, l_off, o_off = merge
            _need_cuda(out)
            a.d_merge_out, a.merge_m_off, a.merge_l_off, a.merge_o_off = out.data_ptr(), int(m_off), int(l_off), int(o_off)
            a.merge_head_dim = out.shape[-1]
            a.merge_rows, a.merge_dtype = out.numel() // out.shape[-1], _dtype_code(out)
        a.d_peer_stage, a.d_peer_count = self.peer_stage.data_ptr(), self.peer_count.data_ptr()
        a.d_state, a.d_status = self.state.data_ptr(), _ptr(status)
        a.rank, a.world = self.rank, self.world
        a.wait_limit = self.wait_limit
        if candidates is not None:
            c = candidates
            _need_cuda(c["out"], c["count"])
            if c["out"].dtype != torch.int32 or c["count"].dtype != torch.int32:
                raise RuntimeError("candidate outputs must be int32")
            a.cand_rows, a.cand_k, a.cand_select = int(c["rows"]), int(c["k"]), int(c["select"])
            a.cand_score_off, a.cand_idx_off = int(c["score_off"]), int(c["idx_off"])
            a.own_lo, a.own_hi = int(c["own"][0]), int(c["own"][1])
            a.d_sel_out, a.sel_stride, a.d_sel_count = c["out"].data_ptr(), c["out"].shape[-1], c["count"].data_ptr()
        with torch.cuda.device(send.device):
            check(lib.tidal_peer_all_gather(C.byref(a), _stream()), "tidal_peer_all_gather")
