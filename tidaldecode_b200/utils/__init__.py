"""Operator façade with the reference's names and call signatures
(tidal/utils/__init__.py:11-287), implemented on the sm_100a kernels.

The reference's attention modules call exactly these functions
(tidal/models/SearchAttention.py:133-181, SparseAttention.py:133-187,
FullAttention.py:133-181); `tidaldecode_b200.attention` calls them the same way.
q is [tokens, Hq, D] for one sequence as in the reference, or [B, Hq, D] when the
controller was built with batch_size B (decode only).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _kernels, ops
from .controller import InferenceController
from .decode_wrapper import BatchDecodeWithPagedKVCacheWrapper
from .kv_cache import KvCache
from .utils import TensorLayout

__all__ = [
    "TensorLayout", "KvCache", "InferenceController", "BatchDecodeWithPagedKVCacheWrapper", "append_kv",
    "prefill_forward", "decode_estimate", "decode_topk", "decode_sparse_attn", "rms_norm_forward",
    "apply_rope_in_place", "rope_append_kv",
]


def apply_rope_in_place(q: torch.Tensor, k: torch.Tensor, past_kv_len: int, rope_scale: Optional[float] = None,
                        rope_theta: Optional[float] = None):
    """RoPE on q, k [N, H, D] in place (tidal/utils/__init__.py:26-53)."""
    _kernels.apply_rope_in_place(q, k, past_kv_len, 1.0 if rope_scale is None else rope_scale,
                                 1e4 if rope_theta is None else rope_theta)


def rms_norm_forward(input: torch.Tensor, weight: torch.Tensor, epsilon: float) -> torch.Tensor:
    o = torch.empty_like(input)
    _kernels.rms_norm_forward(input, weight, o, epsilon)
    return o


def _tokens_per_seq(k: torch.Tensor, c: InferenceController) -> int:
    if k.shape[0] % c.batch_size:
        raise RuntimeError("token count is not a multiple of the controller's batch size")
    return k.shape[0] // c.batch_size


def append_kv(k: torch.Tensor, v: torch.Tensor, iController: InferenceController, layer_idx: int):
    """Write the new tokens' k, v into the layer's pool (tidal/utils/__init__.py:72-128).
    The slots were reserved by iController.prepare_metadata()."""
    c = iController
    tps = _tokens_per_seq(k, c)
    ops.rope_append(None, k, v, c.kv_cache.buf_layer(layer_idx), batch=c.batch_size, pos0=c.kv_cache.seqlen - tps,
                    page_table=c.kv_cache.page_table, rope_mode=0)
    _update_quest_metadata(c, layer_idx, tps)


def rope_append_kv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, iController: InferenceController, layer_idx: int,
                   rope_scale: Optional[float] = None, rope_theta: Optional[float] = None, rope_mode: int = 2,
                   inv_freq: Optional[torch.Tensor] = None):
    """apply_rope_in_place + append_kv in one launch (no reference counterpart: the
    reference launches RoPE and append separately with a device sync around each)."""
    c = iController
    tps = _tokens_per_seq(k, c)
    ops.rope_append(q, k, v, c.kv_cache.buf_layer(layer_idx), batch=c.batch_size, pos0=c.kv_cache.seqlen - tps,
                    page_table=c.kv_cache.page_table, rope_theta=1e4 if rope_theta is None else rope_theta,
                    rope_scale=1.0 if rope_scale is None else rope_scale, rope_mode=rope_mode, inv_freq=inv_freq)
    _update_quest_metadata(c, layer_idx, tps)


def _update_quest_metadata(c: InferenceController, layer_idx: int, new_tokens: int) -> None:
    """Per-page key bounds of the pages the new tokens landed in (only for controllers that keep them)."""
    if c.metadata_cache is None:
        return
    n = c.kv_cache.seqlen
    ops.update_page_meta(c.kv_cache.buf_layer(layer_idx), c.metadata_cache[layer_idx // c.kv_cache.layer_alias], n, n - new_tokens,
                         batch=c.batch_size, page_table=c.kv_cache.page_table, meta_pages_per_seq=c.metadata_cache.shape[1] // c.batch_size)


def prefill_forward(q: torch.Tensor, iController: InferenceController, layer_idx: int, rope_scale: Optional[float] = None,
                    rope_theta: Optional[float] = None) -> torch.Tensor:
    """Causal attention of the prompt over the KV just appended (tidal/utils/__init__.py:131-173)."""
    c = iController
    return _kernels.prefill_with_paged_kv_cache(q, c.kv_cache.buf_layer(layer_idx), c.kv_indices_with_last,
                                                c.kv_cache.last_page_len, True, c.layout, False,
                                                1.0 if rope_scale is None else rope_scale,
                                                1e4 if rope_theta is None else rope_theta)


def decode_estimate(q: torch.Tensor, iController: InferenceController, layer_idx: int) -> torch.Tensor:
    """Quest's page-criticality estimate (tidal/utils/__init__.py:176-214): per query head, an upper bound of
    q.k for every KV page but the newest.  Needs a controller built with quest_metadata=True (the reference
    always allocates the metadata pool; TidalDecode's own layers never read it, so here it is optional).
    q [1, Hq, D] -> [Hq, pages - 1] in q's dtype."""
    c = iController
    if c.metadata_cache is None:
        raise RuntimeError("decode_estimate needs InferenceController(..., quest_metadata=True)")
    n = c.kv_cache.num_pages - 1
    o = torch.empty(q.shape[1], max(n, 1), dtype=q.dtype, device=q.device)
    ops.estimate(q[:1].contiguous(), c.metadata_cache[layer_idx // c.kv_cache.layer_alias], n, out=o.view(1, *o.shape),
                 meta_pages_per_seq=c.metadata_cache.shape[1] // c.batch_size)
    return o[:, :n]


def decode_topk(iController: InferenceController):
    """Select the token set from the logits the last selection layer wrote
    (tidal/utils/__init__.py:217-245): into iController.topk_dindices_buffer, as token
    positions, newest token forced in if the controller says so."""
    c = iController
    n = c.kv_cache.seqlen
    k = c.inference_token_budget
    ops.topk(c.qk_product, k, c.workspace, n=n, out_idx=c._topk_indices_full, out_val=c._topk_values_full,
             force_last=c.force_last_token, hist=c.workspace.hist)
    c._selection_valid = True


def decode_sparse_attn(q: torch.Tensor, iController: InferenceController, layer_idx: int, topk_indices: torch.Tensor,
                       output_qk_product: bool, rope_scale: Optional[float] = None,
                       rope_theta: Optional[float] = None) -> torch.Tensor:
    """Decode attention over the listed tokens (tidal/utils/__init__.py:248-287).

    topk_indices is iController.kv_indices_without_last  -> every cached token (full and
                 selection layers; with output_qk_product the fp32 logits land in
                 iController.qk_product for decode_topk);
    topk_indices is iController.topk_dindices_buffer     -> the set decode_topk chose;
    any other int32 [Hq, n] tensor                       -> pool page ids per head plus the
                 newest token, the reference's literal contract (bsk_ops.h:103-112).
    """
    c = iController
    o = torch.empty_like(q)
    pool = c.kv_cache.buf_layer(layer_idx)
    n = c.kv_cache.seqlen
    if topk_indices is c.kv_indices_without_last or topk_indices is c.kv_indices_with_last:
        if output_qk_product:
            ops.decode_attention(q, pool, n, c.workspace, out=o, page_table=c.kv_cache.page_table, scores=c.qk_product,
                                 hist=c.workspace.hist, force_last=c.force_last_token)
        else:
            ops.decode_attention(q, pool, n, c.workspace, out=o, page_table=c.kv_cache.page_table)
    elif topk_indices is c.topk_dindices_buffer:
        if not c._selection_valid:
            raise RuntimeError("sparse layer before a selection layer of this step")   # modify_llama.py:123-124
        if output_qk_product:
            raise RuntimeError("logits are written by selection layers only")
        ops.decode_attention(q, pool, n, c.workspace, out=o, page_table=c.kv_cache.page_table,
                             sel_idx=c._topk_indices_full, sel_counts=c._counts_full)
    else:
        c._decode_handler.forward(q, o, pool, topk_indices, None, c.kv_cache.last_page_len, c.kv_last_page_idx,
                                  c.qk_product.view(c.num_heads, -1) if (output_qk_product and c.head_reduce == "none"
                                                                         and c.batch_size == 1) else None,
                                  rope_scale, rope_theta)
    return o
