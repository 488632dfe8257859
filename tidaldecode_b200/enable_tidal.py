"""Drop-in for the reference's public switch (src/enable_tidal.py:1-11):

    enable_tidal(model, attn_type="tidal", top_k=256, sparse_layer_start=2, correction_layer=13)

on a Hugging Face Llama model.  As in the reference (src/tidal_build/modify_llama.py:331-391)
every attention module keeps its original forward as `module.flash_forward` and, for
attn_type == "tidal", gets a new `module.forward`:

  * prefill (more than one new token), and any call without a cache: the original forward,
    whose new K,V rows are then copied into this package's paged pool;
  * decode (one new token per sequence): projections and RoPE as the module does them, the
    new K,V row appended to the pool, and attention by the sm_100a kernels —
      layer <  sparse_layer_start                    full attention           (:84-102)
      layer == sparse_layer_start / correction_layer  full attention + top-k   (:116-120)
      other layers                                   the selected tokens only (:121-133)

Selection follows the reference: per query head, budget min(N, top_k), the newest token
competes like any other, the set persists until the next selection layer and is forgotten at
the start of the next forward.  `head_reduce="sum"` / `force_last_token=True` switch to the
shared-set and kernel-path rules.  The forward signature is that of the installed
`transformers` (hidden_states, position_embeddings, attention_mask, past_key_values,
**kwargs) -> (attn_output, None); the reference pins transformers 4.45, whose positional
order differs, so keyword calls are the portable way to invoke it.

`keep_hf_cache=True` (default) also appends the new K,V to the Hugging Face cache during
decode so that everything that reads it (sequence length, position ids in `generate`) keeps
working; the copy it makes every step is not needed by the kernels, and a caller that
passes its own position ids can switch it off.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import utils as tidal_utils
from .utils import InferenceController


class _TidalState:
    """Per-model decode state shared by the patched attention modules."""

    def __init__(self, top_k, sparse_layer_start, correction_layer, head_reduce, force_last_token, max_seq_len,
                 keep_hf_cache):
        self.top_k, self.start, self.correction = top_k, sparse_layer_start, correction_layer
        self.head_reduce, self.force_last_token = head_reduce, force_last_token
        self.max_seq_len, self.keep_hf_cache = max_seq_len, keep_hf_cache
        self.controller: Optional[InferenceController] = None
        self.first_layer = 0
        self.num_layers = 0

    def controller_for(self, module, batch, dtype, device) -> InferenceController:
        c = self.controller
        if c is None or c.batch_size != batch or c.dtype != dtype or torch.device(c.device) != torch.device(device):
            cfg = module.config
            hq = cfg.num_attention_heads
            self.controller = c = InferenceController(
                num_layers=self.num_layers, num_heads=hq, head_dim=module.head_dim, page_size=1, token_budget=self.top_k,
                max_seq_len=self.max_seq_len, dtype=dtype, device=device,
                num_kv_heads=getattr(cfg, "num_key_value_heads", hq) or hq, batch_size=batch, head_reduce=self.head_reduce,
                force_last_token=self.force_last_token)
        return c


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def _make_forward(module, state: _TidalState):
    def tidal_forward(hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, **kwargs):
        bsz, q_len = hidden_states.shape[:2]
        layer = module.layer_idx
        cache = past_key_values if past_key_values is not None else kwargs.get("past_key_value")
        if cache is None or not hidden_states.is_cuda:
            return module.flash_forward(hidden_states, position_embeddings=position_embeddings,
                                        attention_mask=attention_mask, past_key_values=past_key_values, **kwargs)
        c = state.controller_for(module, bsz, hidden_states.dtype, hidden_states.device)
        if layer == state.first_layer:
            if cache.get_seq_length(layer) == 0:
                c.clean_states()                       # a new sequence
            if c.kv_cache.seqlen + q_len > state.max_seq_len:
                raise RuntimeError(f"sequence length {c.kv_cache.seqlen + q_len} exceeds max_seq_len={state.max_seq_len} "
                                   "given to enable_tidal")
            c.prepare_metadata(q_len)
            c.begin_forward(q_len)

        if q_len > 1:
            # prefill: the module's own attention; its new K,V rows go into the pool as well
            out = module.flash_forward(hidden_states, position_embeddings=position_embeddings,
                                       attention_mask=attention_mask, past_key_values=cache, **kwargs)
            lay = cache.layers[layer]
            k_new = lay.keys[:, :, -q_len:].transpose(1, 2).reshape(bsz * q_len, -1, module.head_dim).contiguous()
            v_new = lay.values[:, :, -q_len:].transpose(1, 2).reshape(bsz * q_len, -1, module.head_dim).contiguous()
            tidal_utils.append_kv(k_new, v_new, c, layer)
            return out

        # decode
        D = module.head_dim
        q = module.q_proj(hidden_states).view(bsz, 1, -1, D).transpose(1, 2)      # [B,Hq,1,D]
        k = module.k_proj(hidden_states).view(bsz, 1, -1, D).transpose(1, 2)
        v = module.v_proj(hidden_states).view(bsz, 1, -1, D).transpose(1, 2)
        cos, sin = position_embeddings
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        q = (q * cos) + (_rotate_half(q) * sin)
        k = (k * cos) + (_rotate_half(k) * sin)
        if state.keep_hf_cache:
            cache.update(k, v, layer)
        qn = q[:, :, 0].contiguous()
        tidal_utils.append_kv(k[:, :, 0].contiguous(), v[:, :, 0].contiguous(), c, layer)
        if layer < state.start:
            o = tidal_utils.decode_sparse_attn(qn, c, layer, c.kv_indices_without_last, False)
        elif layer == state.start or layer == state.correction:
            o = tidal_utils.decode_sparse_attn(qn, c, layer, c.kv_indices_without_last, True)
            tidal_utils.decode_topk(c)
        else:
            if not c._selection_valid:
                raise ValueError("pos dict should be set up in sparse attn layers")     # modify_llama.py:123-124
            if c.need_estimate():
                o = tidal_utils.decode_sparse_attn(qn, c, layer, c.topk_dindices_buffer, False)
            else:
                o = tidal_utils.decode_sparse_attn(qn, c, layer, c.kv_indices_without_last, False)
        out = module.o_proj(o.reshape(bsz, 1, -1))
        return out, None

    return tidal_forward


def _is_llama_attention(m) -> bool:
    return all(hasattr(m, a) for a in ("q_proj", "k_proj", "v_proj", "o_proj", "layer_idx", "head_dim"))


def enable_tidal(model, attn_type="tidal", top_k=256, sparse_layer_start=2, correction_layer=13, *,
                 head_reduce: str = "none", force_last_token: bool = False, max_seq_len: Optional[int] = None,
                 keep_hf_cache: bool = True):
    model_type = model.config.model_type
    print(f"token budget: {top_k}")
    print(f"sparse layer starts from: Layer {sparse_layer_start}")
    print(f"reselection layer: {correction_layer}")
    if "llama" not in model_type:
        return
    if max_seq_len is None:
        max_seq_len = min(int(getattr(model.config, "max_position_embeddings", 4096)), 1 << 17)
    state = _TidalState(top_k, sparse_layer_start, correction_layer, head_reduce, force_last_token, max_seq_len, keep_hf_cache)
    mods = [m for m in model.modules() if _is_llama_attention(m)]
    if not mods:
        raise RuntimeError("no Llama attention modules found to patch")
    state.first_layer = min(m.layer_idx for m in mods)
    state.num_layers = max(m.layer_idx for m in mods) + 1
    model._tidal_state = state
    for m in mods:
        if not hasattr(m, "flash_forward"):
            m.flash_forward = m.forward
        if attn_type == "tidal":
            m.forward = _make_forward(m, state)
        else:
            m.forward = m.flash_forward
    return
