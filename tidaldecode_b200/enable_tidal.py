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

A second family, as in the reference (modify_llama.py:150-325, 379-391): attention modules whose class is
named "LlamaAttention" but which are not the installed transformers' (the YaRN model file's: their own
`rotary_emb(q, k, past_len)`, a cache that is the tuple `(kv [B, capacity, 2, heads, D], length)`, the forward
signature `(hidden_states, attention_mask, position_ids, past_key_value, output_attentions, use_cache,
is_padded_inputs)`) get the YaRN form of the hook: prefill and the layers below sparse_layer_start keep the
module's own forward; the other layers' decode steps run on the kernels, their history imported from the
tuple cache the first time.

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
        self.filled = {}              # YaRN form: tokens of each layer's history already in the pool

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


def _make_forward_yarn(module, state: _TidalState):
    """llama_tidal_forward_yarn (modify_llama.py:150-325) on the kernels."""

    def tidal_forward_yarn(hidden_states, attention_mask=None, position_ids=None, past_key_value=None, output_attentions=False,
                           use_cache=False, is_padded_inputs=False):
        bsz, q_len, _ = hidden_states.size()
        layer = module.layer_id
        # prefill and the dense layers: the module's own attention (:163-172)
        if q_len > 1 or layer < state.start or not hidden_states.is_cuda:
            return module.flash_forward(hidden_states, attention_mask, position_ids, past_key_value, output_attentions, use_cache,
                                        is_padded_inputs)
        past_kv, past_len = past_key_value if past_key_value is not None else (None, 0)
        D, Hq, Hkv = module.head_dim, module.num_heads, module.num_key_value_heads
        G = Hq // Hkv
        c = state.controller_for(module, bsz, hidden_states.dtype, hidden_states.device)
        first = layer == state.start
        if first:
            if past_len < c.kv_cache.seqlen:                 # a shorter history than the pool holds: a new sequence
                c.clean_states()
                state.filled.clear()
            if past_len + 1 > state.max_seq_len:
                raise RuntimeError(f"sequence length {past_len + 1} exceeds max_seq_len={state.max_seq_len} given to enable_tidal")
            c.prepare_metadata(past_len + 1 - c.kv_cache.seqlen)
            c.begin_forward(1)
        slot = layer - state.start
        q = module.q_proj(hidden_states).view(bsz, 1, Hq, D)
        k = module.k_proj(hidden_states).view(bsz, 1, Hkv, D)
        v = module.v_proj(hidden_states).view(bsz, 1, Hkv, D)
        q, k = module.rotary_emb(q, k, past_len)             # the module's own (YaRN) rotation (:217)
        # history this layer's pool does not hold yet (the prompt went through the module's own forward): the cache
        # stores every KV head `G` times (:219-236), the pool once
        have = state.filled.get(layer, 0)
        if have < past_len:
            old = past_kv[:, have:past_len, :, ::G]          # [B, n, 2, Hkv, D]
            n = past_len - have
            ko = old[:, :, 0].reshape(bsz * n, Hkv, D).contiguous()
            vo = old[:, :, 1].reshape(bsz * n, Hkv, D).contiguous()
            tidal_utils.ops.rope_append(None, ko, vo, c.kv_cache.buf_layer(slot), batch=bsz, pos0=have,
                                        page_table=c.kv_cache.page_table, rope_mode=0)
        if use_cache and state.keep_hf_cache:
            kv = torch.stack([k, v], 2)[:, :, :, :, None, :].expand(bsz, 1, 2, Hkv, G, D).reshape(bsz, 1, 2, Hq, D)
            if past_kv is None:
                past_kv = kv
            else:
                if past_len + 1 > past_kv.size(1):
                    past_kv = torch.cat([past_kv, torch.empty(bsz, 256, 2, Hq, D, dtype=kv.dtype, device=kv.device)], 1)
                past_kv[:, past_len:past_len + 1] = kv
        tidal_utils.append_kv(k[:, 0].contiguous(), v[:, 0].contiguous(), c, slot)
        state.filled[layer] = past_len + 1
        qn = q[:, 0].contiguous()
        if layer == state.start or layer == state.correction:
            o = tidal_utils.decode_sparse_attn(qn, c, slot, c.kv_indices_without_last, True)
            tidal_utils.decode_topk(c)
        else:
            if not c._selection_valid:
                raise ValueError("pos dict should be set up in sparse attn layers")     # modify_llama.py:286-289
            if c.need_estimate():
                o = tidal_utils.decode_sparse_attn(qn, c, slot, c.topk_dindices_buffer, False)
            else:
                o = tidal_utils.decode_sparse_attn(qn, c, slot, c.kv_indices_without_last, False)
        out = module.o_proj(o.reshape(bsz, 1, Hq * D))
        return out, None, ((past_kv, past_len + 1) if use_cache else None)

    return tidal_forward_yarn


def _is_llama_attention(m) -> bool:
    return all(hasattr(m, a) for a in ("q_proj", "k_proj", "v_proj", "o_proj", "layer_idx", "head_dim"))


def _is_yarn_attention(m) -> bool:
    """The reference's test for its second family: the class is called LlamaAttention (modify_llama.py:381) and it is
    not the kind handled above (no layer_idx, its own rotary_emb)."""
    return (m.__class__.__name__ == "LlamaAttention" and not hasattr(m, "layer_idx") and callable(getattr(m, "rotary_emb", None))
            and all(hasattr(m, a) for a in ("q_proj", "k_proj", "v_proj", "o_proj", "head_dim", "num_heads", "num_key_value_heads")))


def enable_tidal_yarn_modules(mods, attn_type="tidal", top_k=256, sparse_layer_start=2, correction_layer=13, *,
                              head_reduce: str = "none", force_last_token: bool = False, max_seq_len: int = 1 << 16,
                              keep_hf_cache: bool = True) -> _TidalState:
    """Install the YaRN form of the hook on a list of attention modules given in layer order (what enable_tidal does for
    the modules of that family it finds in a model).  Returns the shared decode state."""
    state = _TidalState(top_k, sparse_layer_start, correction_layer, head_reduce, force_last_token, max_seq_len, keep_hf_cache)
    state.num_layers = max(1, len(mods) - sparse_layer_start)        # only the layers from sparse_layer_start on use the pool
    state.filled = {}
    for i, m in enumerate(mods):
        m.layer_id = i
        m.token_budget, m.sparse_layer_start, m.correction_layer = top_k, sparse_layer_start, correction_layer
        if not hasattr(m, "flash_forward"):
            m.flash_forward = m.forward
        m.forward = _make_forward_yarn(m, state) if attn_type == "tidal" else m.flash_forward
    return state


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
    yarn = [m for m in model.modules() if _is_yarn_attention(m)]
    if yarn:
        model._tidal_state = enable_tidal_yarn_modules(yarn, attn_type, top_k, sparse_layer_start, correction_layer,
                                                       head_reduce=head_reduce, force_last_token=force_last_token,
                                                       max_seq_len=max_seq_len, keep_hf_cache=keep_hf_cache)
        return
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
