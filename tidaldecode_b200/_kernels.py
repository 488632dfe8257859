"""Drop-in for the reference's pybind module `tidal._kernels`
(tidal/ops/csrc/bsk_ops.cu:4-20): the same seven functions and one class, same
argument order and tensor contracts, errors as RuntimeError — implemented on
libtidal_b200.so through its C ABI.

Differences a caller can observe, all of them repairs of reference defects:
  * every op launches on torch's current stream, not the legacy default stream
    (reference: approx_attn.cu:141, page.cu:89,200,244);
  * float16, bfloat16 and float32 are accepted (reference: float16 only,
    pytorch_extension_utils.h:25-35), any head count (reference: 32, topk.cu:26),
    and grouped-query heads (reference: decode_handler.cuh:83);
  * a `qk_product` buffer passed to `forward` IS written (the reference passes it
    on only when it is empty, approx_attn.cu:137): row h, column j holds the
    logit q_h.k/sqrt(D) of the j-th listed page, the newest token last;
  * the Quest metadata pool (per-page key bounds) is maintained by the append calls when one
    is passed, and `estimate_attn_score` reads it, as in the reference; passing None for
    `metadata_data` skips it (TidalDecode's own layers never read it).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops as _ops

_NHD, _HND = 0, 1


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_input(t: torch.Tensor, name: str) -> None:
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _check_layout(layout: int) -> None:
    _check(layout == _NHD, "only the NHD layout is built (the reference's controller uses no other: "
                           "tidal/utils/controller.py:40)")


_ws_cache = {}          # device index -> the Workspace per-token calls on that device use


def _fits(ws: _ops.Workspace, batch: int, hq: int, d: int, rows: int, n: int) -> bool:
    g = ws.geometry
    return batch * hq * d <= g[0] * g[1] * g[2] and batch * hq <= g[0] * g[1] and rows <= g[3] and n <= g[4]


def adopt_workspace(ws: _ops.Workspace) -> None:
    """Let `forward` and `topk_filtering` on ws's device use a workspace the caller owns already
    (an InferenceController's) instead of reserving a second one."""
    _ws_cache[ws.buf.device.index] = ws


def reserve_workspace(device, num_qo_heads: int, head_dim: int, rows: int, n: int, batch: int = 1) -> _ops.Workspace:
    """Make sure scratch for this geometry exists on `device`: split-KV partials for `batch` x `num_qo_heads` x
    `head_dim`, top-k lists for `rows` rows of up to `n` scores.  This is the only place of this module that
    allocates device memory, and only when what is there does not fit; `begin_forward` calls it, as the
    reference's handler allocates in BeginForward (decode_handler.cuh:104-117), so that the per-token calls
    find everything in place."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ws = _ws_cache.get(device.index)
    if ws is None or not _fits(ws, batch, num_qo_heads, head_dim, rows, n):
        g = ws.geometry if ws is not None else (1, 1, 1, 1, 1)
        ws = _ops.Workspace(max(batch, g[0]), max(num_qo_heads, g[1]), max(head_dim, g[2]), max(rows, g[3]), max(n, g[4]),
                            device=device)
        _ws_cache[device.index] = ws
    return ws


def _reserved(device: torch.device, batch: int, hq: int, d: int, rows: int, n: int, first_use_reserves: bool = False) -> _ops.Workspace:
    """The scratch for a per-token call; never allocates once a workspace exists on the device."""
    ws = _ws_cache.get(device.index)
    if ws is None and first_use_reserves:
        return reserve_workspace(device, hq, d, rows, n, batch)
    _check(ws is not None and _fits(ws, batch, hq, d, rows, n),
           f"no scratch reserved for {batch} x {hq} heads x {d}, {rows} rows of {n} scores on {device}: call begin_forward "
           "(or tidaldecode_b200._kernels.reserve_workspace) with this geometry first; per-token calls do not allocate")
    return ws


def apply_rope_in_place(q: torch.Tensor, k: torch.Tensor, past_kv_len: int, rope_scale: float, rope_theta: float) -> None:
    """q, k [seq, H, D] rotated in place, positions past_kv_len .. past_kv_len+seq-1
    (tidal/ops/csrc/page.cu:212-253).  fp32 rotation rounded once, like the reference kernel."""
    _check_input(q, "q")
    _check_input(k, "k")
    _check(q.dim() == 3 and k.dim() == 3, "q and k must be [seq, heads, head_dim]")
    _check(q.shape[0] == k.shape[0] and q.shape[2] == k.shape[2], "q and k disagree on seq or head_dim")
    _ops.rope_append(q, k, None, None, batch=1, pos0=int(past_kv_len), rope_theta=float(rope_theta),
                     rope_scale=float(rope_scale), rope_mode=2, rotate_k_in_place=True)


def _append(k, v, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx, metadata_data, metadata_indices,
            metadata_last_page_len, layout, decode: bool) -> None:
    for t, n in ((k, "k"), (v, "v"), (kv_data, "kv_data"), (kv_indices, "kv_indices")):
        _check_input(t, n)
    _check(k.dim() == 3 and v.dim() == 3, "k and v must be [seq, heads, head_dim]")
    _check(kv_data.dim() == 5 and kv_data.shape[1] == 2, "kv_data must be [pages, 2, page_size, heads, head_dim]")
    _check(kv_indices.dim() == 1 and kv_indices.dtype == torch.int32, "kv_indices must be int32 [num_pages]")
    _check(kv_indptr.dtype == torch.int32, "kv_indptr must be int32")
    _check_layout(layout)
    _check(kv_data.shape[3] == k.shape[1] and kv_data.shape[4] == k.shape[2], "kv_data and k disagree on heads or head_dim")
    _check(k.shape == v.shape, "k and v must have one shape")
    page_size = kv_data.shape[2]
    n_pages = kv_indices.numel()
    seq_len = (n_pages - 1) * page_size + int(kv_last_page_len)
    if decode:
        _check(k.shape[0] == 1, "append_kv_cache_decode takes one token")
        pos0 = int(kv_last_page_idx) * page_size + int(kv_last_page_len) - 1
        _ops.rope_append(None, k, v, kv_data, batch=1, pos0=pos0, pages_per_seq=kv_data.shape[0], rope_mode=0)
    else:
        _check(k.shape[0] <= seq_len, "more new tokens than the sequence holds")
        _ops.rope_append(None, k, v, kv_data, batch=1, pos0=seq_len - k.shape[0], page_table=kv_indices.view(1, -1),
                         rope_mode=0)
    if metadata_data is not None and isinstance(metadata_data, torch.Tensor) and metadata_data.numel() > 0:
        # Quest's per-page key bounds: one metadata entry per KV page (decode_page.cuh:417-441); the entries of the
        # pages the new tokens landed in are recomputed from the pool
        _check_input(metadata_data, "metadata_data")
        _check_input(metadata_indices, "metadata_indices")
        _check(metadata_data.dim() == 5 and metadata_data.shape[1] == 2 and metadata_data.shape[3:] == kv_data.shape[3:]
               and metadata_data.dtype == kv_data.dtype, "metadata_data must be [pages, 2, page_size, heads, head_dim] like kv_data")
        _check(metadata_indices.dim() == 1 and metadata_indices.dtype == torch.int32, "metadata_indices must be int32 [num_pages]")
        entries = (metadata_indices.numel() - 1) * metadata_data.shape[2] + int(metadata_last_page_len)
        _check(entries == n_pages, f"the metadata must hold one entry per KV page ({entries} entries, {n_pages} pages)")
        _ops.update_page_meta(kv_data, metadata_data, seq_len, seq_len - k.shape[0], batch=1,
                              page_table=kv_indices.view(1, -1), meta_table=metadata_indices.view(1, -1))


def append_kv_cache_decode(k, v, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx,
                           metadata_data, metadata_indices, metadata_indptr, metadata_last_page_len,
                           metadata_last_page_idx, layout) -> None:
    """Write the new token's k,v [1,H,D] into slot (kv_last_page_idx, kv_last_page_len-1) and fold its key into
    the page's metadata entry (tidal/ops/csrc/page.cu:6-99)."""
    _append(k, v, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx, metadata_data, metadata_indices,
            metadata_last_page_len, layout, True)


def append_kv_cache_prefill(k, v, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx,
                            metadata_data, metadata_indices, metadata_indptr, metadata_last_page_len,
                            metadata_last_page_idx, layout) -> None:
    """Write the last seq tokens' k,v [seq,H,D] into the pages listed by kv_indices and rebuild the metadata
    entries of those pages (tidal/ops/csrc/page.cu:101-210)."""
    _append(k, v, kv_data, kv_indices, kv_indptr, kv_last_page_len, kv_last_page_idx, metadata_data, metadata_indices,
            metadata_last_page_len, layout, False)


def topk_filtering(estimated_value: torch.Tensor, estimated_indices: torch.Tensor, d_out: torch.Tensor,
                   indices_out: torch.Tensor, buf: torch.Tensor, page_budget: int, length: Optional[int] = None) -> None:
    """Per row, the page_budget largest values and `estimated_indices` gathered at their
    places (tidal/ops/csrc/topk.cu:7-44).  `buf` is unused (the workspace is internal);
    `length` limits the columns considered (the reference always scans the full row,
    including columns beyond the sequence)."""
    _check_input(estimated_value, "estimated_value")
    _check_input(indices_out, "indices_out")
    _check(estimated_value.dim() == 2 and estimated_indices.dim() == 2, "value and indices must be 2-D")
    _check(estimated_indices.dtype == torch.int32 and indices_out.dtype == torch.int32, "indices must be int32")
    _check(estimated_value.shape[0] == estimated_indices.shape[0], "value and indices disagree on rows")
    _check(d_out.shape[1] == page_budget and indices_out.shape[1] == page_budget, "outputs must have page_budget columns")
    rows, width = estimated_value.shape
    n = width if length is None else int(length)
    _check(0 < n <= width and n <= estimated_indices.shape[1], "length out of range")
    val = estimated_value if estimated_value.dtype == torch.float32 else estimated_value.float()
    if estimated_indices.stride(0) == 0:
        in_idx = estimated_indices[0].contiguous()         # one row shared by all heads
    else:
        _check(estimated_indices.is_contiguous(), "estimated_indices must be contiguous or row-broadcast")
        _check(estimated_indices.shape[1] == width, "value and indices disagree on columns")
        in_idx = estimated_indices
    # scratch: reserved by the first call for this row count and width (the reference's callers pass rows of
    # max_seq_len columns, so the width never changes afterwards); later calls find it and allocate nothing
    ws = _reserved(val.device, 1, 1, 64, rows, width, first_use_reserves=True)
    out_val = d_out if d_out.dtype == torch.float32 else torch.empty(d_out.shape, dtype=torch.float32, device=d_out.device)
    _ops.topk(val, int(page_budget), ws, n=n, in_idx=in_idx, out_idx=indices_out, out_val=out_val)
    if out_val is not d_out:
        d_out.copy_(out_val)


def estimate_attn_score(q, o, metadata_data, metadata_indices, metadata_indptr, metadata_last_page_len,
                        metadata_last_page_idx, layout) -> None:
    """Quest's per-page upper bound of q.k (tidal/ops/csrc/estimate.cu:6-84): o [heads, entries - 1] receives, for
    every query head and every metadata entry but the last (the page still being filled, estimate.cu:52-54),
    sum_d max(q_d * max_d, q_d * min_d)."""
    _check_input(q, "q")
    _check_input(o, "o")
    _check_input(metadata_data, "metadata_data")
    _check_input(metadata_indices, "metadata_indices")
    _check(q.dim() == 3 and q.shape[0] == 1, "q must be [1, heads, head_dim]")
    _check(metadata_data.dim() == 5 and metadata_data.shape[1] == 2, "metadata_data must be [pages, 2, page_size, heads, head_dim]")
    _check(metadata_indices.dim() == 1 and metadata_indices.dtype == torch.int32, "metadata_indices must be int32 [num_pages]")
    _check_layout(layout)
    _check(metadata_data.shape[4] == q.shape[2], "head_dim of q and the metadata differ")
    n = (metadata_indices.numel() - 1) * metadata_data.shape[2] + int(metadata_last_page_len) - 1
    _check(o.dim() == 2 and o.shape[0] == q.shape[1] and o.shape[1] >= n, "o must be [heads, >= entries - 1]")
    _ops.estimate(q, metadata_data, n, out=o.view(1, o.shape[0], o.shape[1]), meta_table=metadata_indices.view(1, -1))


def prefill_with_paged_kv_cache(q, kv_data, kv_indices, kv_last_page_len, causal, layout, allow_fp16_qk_reduction,
                                rope_scale, rope_theta) -> torch.Tensor:
    """Causal attention of q [seq,H,D] over the paged KV that already holds these tokens
    (tidal/ops/csrc/batch_prefill.cu:27-117) by this library's own kernels (tidal_prefill): tcgen05 for
    fp16/bf16, CUDA cores for fp32; head_dim 64 or 128 (anything else is refused, as the reference's
    head-dim dispatch refuses what it was not built for)."""
    _check_input(q, "q")
    _check_input(kv_data, "kv_data")
    _check_input(kv_indices, "kv_indices")
    _check(q.dim() == 3 and kv_data.dim() == 5, "q must be [seq,H,D], kv_data [pages,2,page,H,D]")
    _check_layout(layout)
    page_size = kv_data.shape[2]
    n_pages = kv_indices.numel()
    seq_len = (n_pages - 1) * page_size + int(kv_last_page_len)
    D = kv_data.shape[4]
    _check(q.dtype == kv_data.dtype and q.dtype in (torch.float16, torch.bfloat16, torch.float32), "q and kv_data must share a dtype (f16, bf16, f32)")
    _check(D in (64, 128), f"head_dim {D} is not built (64, 128)")
    return _ops.prefill(q.contiguous(), kv_data, kv_indices.to(torch.int32).contiguous(), seq_len, causal=bool(causal))


def rms_norm_forward(input: torch.Tensor, weight: torch.Tensor, output: torch.Tensor, epsilon: float) -> None:
    """RMSNorm with fp32 statistics into `output` (tidal/ops/csrc/rms_norm.cu:185-213).  The normalised
    value is rounded to the storage type before the weight, as the reference's PyTorch model does."""
    _check_input(input, "input")
    _check_input(weight, "weight")
    _check_input(output, "output")
    _check(output.shape == input.shape and output.dtype == input.dtype, "output must match input")
    _ops.rms_norm(input, weight, float(epsilon), out=output, round_before_weight=True)


class BatchDecodeWithPagedKVCachePyTorchWrapper:
    """tidal/ops/csrc/bsk_ops.h:88-118, tidal/ops/csrc/approx_attn.cu:27-151."""

    def __init__(self, layout: int):
        _check_layout(layout)
        self._layout = layout
        self._begun = False
        self._geom = None
        self._ws = None
        self._max_list = 4096          # shortest list the scratch is sized for

    def begin_forward(self, indptr: torch.Tensor, num_qo_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                      empty_data: torch.Tensor, max_pages: int = 0, device=None) -> None:
        """Records the geometry and makes sure the scratch for it exists, so that `forward` allocates
        nothing (the reference allocates two buffers and uploads a partition plan here on every call:
        decode_handler.cuh:73-121; this allocates only when the geometry outgrows what is reserved).
        `indptr` ([0, pages listed per head], as the reference passes it) gives the list length when it
        is a host tensor or a list; a device tensor is not read back (no sync) and `max_pages` — or the
        longest list seen so far — is used instead."""
        if num_qo_heads % num_kv_heads != 0:
            raise ValueError(f"num_qo_heads {num_qo_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self._geom = (int(num_qo_heads), int(num_kv_heads), int(head_dim), int(page_size), empty_data.dtype)
        n = int(max_pages)
        if indptr is not None and not (isinstance(indptr, torch.Tensor) and indptr.is_cuda):
            ip = [int(x) for x in (indptr.tolist() if isinstance(indptr, torch.Tensor) else indptr)]
            if len(ip) >= 2:
                n = max(n, max(b - a for a, b in zip(ip[:-1], ip[1:])))
        self._max_list = max(self._max_list, n)
        dev = device if device is not None else (indptr.device if isinstance(indptr, torch.Tensor) and indptr.is_cuda
                                                 else torch.device("cuda", torch.cuda.current_device()))
        self._ws = reserve_workspace(dev, num_qo_heads, head_dim, num_qo_heads, self._max_list + 1)
        self._begun = True

    def end_forward(self) -> None:
        self._begun = False

    def forward(self, q: torch.Tensor, o: torch.Tensor, paged_kv_data: torch.Tensor, paged_kv_indices: torch.Tensor,
                paged_kv_indptr: torch.Tensor, paged_kv_last_page_len: int, paged_kv_last_page_idx: int,
                qk_product: torch.Tensor, rope_scale: float, rope_theta: float) -> None:
        if not self._begun:
            raise RuntimeError("forward() before begin_forward()")          # decode_handler.cuh:228-233
        _check_input(q, "q")
        _check_input(o, "o")
        _check_input(paged_kv_data, "paged_kv_data")
        _check_input(paged_kv_indices, "paged_kv_indices")
        _check(q.dim() == 3 and q.shape[0] == 1, "q must be [1, heads, head_dim]")
        _check(paged_kv_indices.dim() == 2 and paged_kv_indices.dtype == torch.int32, "paged_kv_indices must be int32 [heads, n]")
        _check(paged_kv_data.dim() == 5 and paged_kv_data.shape[1] == 2, "paged_kv_data must be [pages,2,page,H,D]")
        _check(paged_kv_data.shape[4] == q.shape[2], "head_dim of q and kv differ")
        _check(paged_kv_data.shape[2] == 1, "page lists are built for page_size 1 (tidal/utils/controller.py:20)")
        Hq, D = q.shape[1], q.shape[2]
        _check(paged_kv_indices.shape[0] == Hq, "paged_kv_indices needs one row per query head")
        n = paged_kv_indices.shape[1]
        scores = None
        tmp = None
        if qk_product is not None and qk_product.numel() > 0:
            _check(qk_product.dim() == 2 and qk_product.shape[0] == Hq and qk_product.shape[1] >= n + 1,
                   "qk_product must be [heads, >= listed pages + 1]")
            if qk_product.dtype == torch.float32 and qk_product.is_contiguous():
                scores = qk_product.view(1, Hq, -1)
            else:
                tmp = torch.empty(1, Hq, n + 1, dtype=torch.float32, device=q.device)
                scores = tmp
        ws = _reserved(q.device, 1, Hq, D, 1, 1)          # the attention call needs the split-KV partials only
        _ops.decode_attention(q, paged_kv_data, n + 1, ws, out=o, sel_idx=paged_kv_indices.view(1, Hq, n),
                              sel_physical=True, extra_page=int(paged_kv_last_page_idx), scores=scores)
        if tmp is not None:
            qk_product[:, : n + 1].copy_(tmp[0])
