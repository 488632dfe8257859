"""ctypes binding of libtidal_b200.so (the C ABI declared in include/tidal_b200.h).

There is no fallback: if the library is missing or a symbol cannot be resolved,
importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# TIDAL_B200_LIB names another build of the same library (e.g. one compiled with extra -D flags)
LIB_PATH = os.environ.get("TIDAL_B200_LIB") or os.path.join(_HERE, "libtidal_b200.so")

DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
ERR_ARG, ERR_WORKSPACE, ERR_CUDA = -1, -2, -3
DEV_WAIT_TIMEOUT, DEV_BAD_INDEX, DEV_TOPK_OVERFLOW = 1, 2, 4
TOPK_BINS = 4096
XCHG_MAX_CTAS = 64

EXPORTS = (
    "tidal_version", "tidal_last_error", "tidal_launch_count", "tidal_ws_bytes", "tidal_ws_init", "tidal_ws_release", "tidal_ws_status",
    "tidal_decode_attention", "tidal_plan_chunks", "tidal_topk", "tidal_topk_static", "tidal_topk_static_status", "tidal_rope_append", "tidal_update_page_meta", "tidal_estimate", "tidal_merge_partials", "tidal_merge_partials_strided", "tidal_rms_norm", "tidal_decode_linear", "tidal_decode_qkv", "tidal_peer_all_gather", "tidal_peer_exchange_reset", "tidal_prefill",
)


class AttnArgs(C.Structure):
    _fields_ = [
        ("d_q", C.c_void_p), ("d_o", C.c_void_p), ("d_kv", C.c_void_p),
        ("d_page_table", C.c_void_p), ("page_table_stride", C.c_int64),
        ("d_seq_lens", C.c_void_p), ("seq_len", C.c_int32),
        ("d_sel_idx", C.c_void_p), ("sel_rows", C.c_int32), ("sel_count", C.c_int32), ("sel_stride", C.c_int64),
        ("sel_physical", C.c_int32), ("d_sel_counts", C.c_void_p), ("extra_page", C.c_int32),
        ("d_scores", C.c_void_p), ("score_rows", C.c_int32), ("score_stride", C.c_int64),
        ("d_hist", C.c_void_p), ("force_last", C.c_int32),
        ("d_part_m", C.c_void_p), ("d_part_l", C.c_void_p), ("d_part_o", C.c_void_p),
        ("batch", C.c_int32), ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("page_size", C.c_int32), ("dtype", C.c_int32),
        ("num_pages", C.c_int64), ("sm_scale", C.c_float), ("num_chunks", C.c_int32), ("heads_per_cta", C.c_int32),
        ("use_tensor_cores", C.c_int32),
    ]


class TopkArgs(C.Structure):
    _fields_ = [
        ("d_scores", C.c_void_p), ("d_in_idx", C.c_void_p), ("in_idx_stride", C.c_int64), ("rows", C.c_int32),
        ("n", C.c_int64), ("row_stride", C.c_int64), ("k", C.c_int32),
        ("d_out_idx", C.c_void_p), ("d_out_val", C.c_void_p), ("out_stride", C.c_int64),
        ("idx_offset", C.c_int32), ("force_last", C.c_int32), ("own_lo", C.c_int32), ("own_hi", C.c_int32),
        ("d_out_count", C.c_void_p), ("d_hist", C.c_void_p),
        ("seg_len", C.c_int32), ("seg_stride", C.c_int64), ("d_row_len", C.c_void_p),
    ]


class RopeAppendArgs(C.Structure):
    _fields_ = [
        ("d_q", C.c_void_p), ("d_k", C.c_void_p), ("d_v", C.c_void_p), ("d_kv", C.c_void_p),
        ("d_page_table", C.c_void_p), ("page_table_stride", C.c_int64),
        ("d_pos0", C.c_void_p), ("pos0", C.c_int32), ("d_inv_freq", C.c_void_p),
        ("rope_theta", C.c_float), ("rope_scale", C.c_float), ("rope_mode", C.c_int32), ("rotate_k_in_place", C.c_int32),
        ("batch", C.c_int32), ("tokens_per_seq", C.c_int32), ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("page_size", C.c_int32), ("dtype", C.c_int32),
        ("num_pages", C.c_int64), ("d_status", C.c_void_p), ("d_q_src", C.c_void_p), ("kv_pos_base", C.c_int32),
    ]


class PageMetaArgs(C.Structure):
    _fields_ = [
        ("d_kv", C.c_void_p), ("d_meta", C.c_void_p), ("d_page_table", C.c_void_p), ("page_table_stride", C.c_int64),
        ("d_meta_table", C.c_void_p), ("meta_table_stride", C.c_int64),
        ("batch", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("page_size", C.c_int32),
        ("meta_page_size", C.c_int32), ("dtype", C.c_int32),
        ("num_pages", C.c_int64), ("num_meta_pages", C.c_int64), ("first_pos", C.c_int32), ("seq_len", C.c_int32),
        ("d_status", C.c_void_p),
    ]


class EstimateArgs(C.Structure):
    _fields_ = [
        ("d_q", C.c_void_p), ("d_meta", C.c_void_p), ("d_meta_table", C.c_void_p), ("meta_table_stride", C.c_int64),
        ("d_out", C.c_void_p), ("out_stride", C.c_int64),
        ("batch", C.c_int32), ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("meta_page_size", C.c_int32), ("n_entries", C.c_int32), ("dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("num_meta_pages", C.c_int64), ("d_status", C.c_void_p),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("d_x", C.c_void_p), ("d_w", C.c_void_p), ("d_y", C.c_void_p), ("d_residual", C.c_void_p), ("d_norm_weight", C.c_void_p),
        ("norm_eps", C.c_float), ("norm_round_before_weight", C.c_int32),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("dtype", C.c_int32), ("epilogue", C.c_int32),
        ("d_status", C.c_void_p), ("static_weights", C.c_int32),
    ]


LINEAR_PLAIN, LINEAR_SILU_MUL = 0, 1


class ExchangeArgs(C.Structure):
    _fields_ = [
        ("d_send", C.c_void_p), ("d_recv", C.c_void_p), ("bytes", C.c_int64), ("slot_bytes", C.c_int64),
        ("d_peer_stage", C.c_void_p), ("d_peer_count", C.c_void_p), ("d_state", C.c_void_p), ("d_status", C.c_void_p),
        ("rank", C.c_int32), ("world", C.c_int32),
        ("d_merge_out", C.c_void_p), ("merge_m_off", C.c_int64), ("merge_l_off", C.c_int64), ("merge_o_off", C.c_int64),
        ("merge_rows", C.c_int32), ("merge_head_dim", C.c_int32), ("merge_dtype", C.c_int32),
        ("wait_limit", C.c_int32),
        ("cand_rows", C.c_int32), ("cand_k", C.c_int32), ("cand_select", C.c_int32),
        ("cand_score_off", C.c_int64), ("cand_idx_off", C.c_int64), ("own_lo", C.c_int32), ("own_hi", C.c_int32),
        ("d_sel_out", C.c_void_p), ("sel_stride", C.c_int64), ("d_sel_count", C.c_void_p),
    ]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("d_q", C.c_void_p), ("d_o", C.c_void_p), ("d_kv", C.c_void_p), ("d_page_table", C.c_void_p), ("d_status", C.c_void_p),
        ("kv_len", C.c_int64),
        ("n_q", C.c_int32), ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("page_size", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32), ("sm_scale", C.c_float),
        ("num_pages", C.c_int64),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m tidaldecode_b200.build` "
            "(tidaldecode_b200 has no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}")
    lib.tidal_version.restype = C.c_int
    lib.tidal_last_error.restype = C.c_char_p
    lib.tidal_launch_count.restype = C.c_uint64
    lib.tidal_ws_bytes.restype = C.c_size_t
    lib.tidal_ws_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64]
    lib.tidal_ws_init.restype = C.c_int
    lib.tidal_ws_init.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p]
    lib.tidal_ws_release.restype = C.c_int
    lib.tidal_ws_release.argtypes = [C.c_void_p]
    lib.tidal_ws_status.restype = C.c_int
    lib.tidal_ws_status.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    lib.tidal_decode_attention.restype = C.c_int
    lib.tidal_decode_attention.argtypes = [C.POINTER(AttnArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.tidal_plan_chunks.restype = C.c_int
    lib.tidal_plan_chunks.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.tidal_topk.restype = C.c_int
    lib.tidal_topk.argtypes = [C.POINTER(TopkArgs), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.tidal_topk_static.restype = C.c_int
    lib.tidal_topk_static.argtypes = [C.POINTER(TopkArgs), C.c_void_p, C.c_void_p]
    lib.tidal_topk_static_status.restype = C.c_int
    lib.tidal_topk_static_status.argtypes = [C.c_int, C.c_void_p]
    lib.tidal_rope_append.restype = C.c_int
    lib.tidal_rope_append.argtypes = [C.POINTER(RopeAppendArgs), C.c_void_p]
    lib.tidal_update_page_meta.restype = C.c_int
    lib.tidal_update_page_meta.argtypes = [C.POINTER(PageMetaArgs), C.c_void_p]
    lib.tidal_estimate.restype = C.c_int
    lib.tidal_estimate.argtypes = [C.POINTER(EstimateArgs), C.c_void_p]
    lib.tidal_merge_partials.restype = C.c_int
    lib.tidal_merge_partials.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p, C.c_int, C.c_void_p]
    lib.tidal_merge_partials_strided.restype = C.c_int
    lib.tidal_merge_partials_strided.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int,
                                                 C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    lib.tidal_rms_norm.restype = C.c_int
    lib.tidal_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_int, C.c_int, C.c_void_p]
    lib.tidal_decode_linear.restype = C.c_int
    lib.tidal_decode_linear.argtypes = [C.POINTER(LinearArgs), C.c_void_p]
    lib.tidal_decode_qkv.restype = C.c_int
    lib.tidal_decode_qkv.argtypes = [C.POINTER(LinearArgs), C.POINTER(RopeAppendArgs), C.c_void_p]
    lib.tidal_peer_all_gather.restype = C.c_int
    lib.tidal_peer_all_gather.argtypes = [C.POINTER(ExchangeArgs), C.c_void_p]
    lib.tidal_peer_exchange_reset.restype = C.c_int
    lib.tidal_peer_exchange_reset.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.tidal_prefill.restype = C.c_int
    lib.tidal_prefill.argtypes = [C.POINTER(PrefillArgs), C.c_void_p]
    return lib


lib = _load()


def last_error() -> str:
    return lib.tidal_last_error().decode()


def check(rc: int, what: str) -> None:
    """Negative return codes become RuntimeError, as TORCH_CHECK failures do in
    the reference's extension (tidal/ops/csrc/page.cu:20-41)."""
    if rc < 0:
        raise RuntimeError(f"{what} failed ({rc}): {last_error()}")
