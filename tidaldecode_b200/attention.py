"""The three attention modules of the kernel path, with the reference's names,
constructor and forward signature (tidal/models/FullAttention.py:75-209,
SearchAttention.py:75-216, SparseAttention.py:75-222):

    forward(hidden_states, attention_mask, position_ids, past_key_value,
            output_attentions, use_cache, iController) -> (attn_output, None, past_key_value)

    FullAttention    every cached token (layers before the first selection layer)
    SearchAttention  every cached token, and writes the logits from which the
                     token set of the following layers is chosen (selection layers)
    SparseAttention  only the tokens the last SearchAttention chose

Same sequence of operator calls as the reference (projection, RoPE, append,
attention, top-k, output projection) through `tidaldecode_b200.utils`, minus the
`torch.cuda.synchronize()` the reference wraps around every call
(SearchAttention.py:156-182); RoPE and append are one fused launch.  The NVTX
range names are the reference's.  Grouped-query heads and a batch of sequences
decoded in lockstep are accepted (the reference asserts batch 1).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from . import utils as tidal_utils


class _TidalAttention(nn.Module):
    layer_kind = "full"

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.config = config
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = getattr(config, "head_dim", None) or self.hidden_size // self.num_heads
        self.num_key_value_heads = getattr(config, "num_key_value_heads", None) or self.num_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.pretraining_tp = getattr(config, "pretraining_tp", 1)
        self.max_position_embeddings = getattr(config, "max_position_embeddings", 4096)
        if self.head_dim * self.num_heads != self.hidden_size:
            raise ValueError(f"hidden_size must be divisible by num_heads (got `hidden_size`: {self.hidden_size}"
                             f" and `num_heads`: {self.num_heads}).")
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=False)
        self._init_rope()

    def _init_rope(self):
        scaling = getattr(self.config, "rope_scaling", None)
        self.rope_theta = float(getattr(self.config, "rope_theta", 1e4) or 1e4)
        if scaling is None:
            self.rope_scale = 1.0
        else:
            scaling_type = scaling.get("type", scaling.get("rope_type"))
            if scaling_type == "linear":
                self.rope_scale = scaling["factor"]
            elif scaling_type in (None, "default"):
                self.rope_scale = 1.0
            else:
                raise ValueError(f"Unknown RoPE scaling type {scaling_type}")
        # how the rotation is rounded: 2 = fp32 rotation rounded once (the reference kernel),
        # 1 = the rounding order of the reference's PyTorch model
        self.rope_mode = int(getattr(self.config, "tidal_rope_mode", 2))
        # fp32 always (a module-wide .to(dtype) must not round it), so not a registered buffer
        self._inv_freq = 1.0 / (self.rope_theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.int64).float() / self.head_dim))

    def _inv_freq_on(self, device) -> torch.Tensor:
        if self._inv_freq.device != device:
            self._inv_freq = self._inv_freq.to(device)
        return self._inv_freq

    def _attend(self, q: torch.Tensor, iController) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.LongTensor] = None, past_key_value: Optional[Tuple[torch.Tensor]] = None,
                output_attentions: bool = False, use_cache: bool = False, iController=None,
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[Tuple[torch.Tensor]]]:
        bsz, q_len, _ = hidden_states.size()
        c = iController
        assert c is not None, "the tidal attention modules need an InferenceController"
        assert bsz == c.batch_size, "batch size differs from the controller's"
        assert q_len == 1 or bsz == 1, "prefill takes one sequence at a time"

        torch.cuda.nvtx.range_push("qkv_proj")
        query_states = self.q_proj(hidden_states)
        key_states = self.k_proj(hidden_states)
        value_states = self.v_proj(hidden_states)
        torch.cuda.nvtx.range_pop()

        # NHD, tokens of all sequences flattened: [bsz*q_len, H, D]
        query_states = query_states.view(bsz * q_len, self.num_heads, self.head_dim)
        key_states = key_states.view(bsz * q_len, self.num_key_value_heads, self.head_dim)
        value_states = value_states.view(bsz * q_len, self.num_key_value_heads, self.head_dim)

        torch.cuda.nvtx.range_push("RoPE")
        torch.cuda.nvtx.range_push("append_kv")
        tidal_utils.rope_append_kv(query_states, key_states, value_states, c, self.layer_idx, rope_scale=self.rope_scale,
                                   rope_theta=self.rope_theta, rope_mode=self.rope_mode,
                                   inv_freq=self._inv_freq_on(hidden_states.device))
        torch.cuda.nvtx.range_pop()
        torch.cuda.nvtx.range_pop()

        if q_len > 1:
            torch.cuda.nvtx.range_push("prefill_attn")
            attn_output = tidal_utils.prefill_forward(query_states, c, self.layer_idx)
            torch.cuda.nvtx.range_pop()
        else:
            attn_output = self._attend(query_states, c)

        attn_output = attn_output.reshape(bsz, q_len, self.hidden_size)
        torch.cuda.nvtx.range_push("o_proj")
        attn_output = self.o_proj(attn_output)
        torch.cuda.nvtx.range_pop()
        return attn_output, None, past_key_value


class FullAttention(_TidalAttention):
    layer_kind = "full"

    def _attend(self, q, c):
        torch.cuda.nvtx.range_push("full_attn")
        o = tidal_utils.decode_sparse_attn(q, c, self.layer_idx, c.kv_indices_without_last, False)
        torch.cuda.nvtx.range_pop()
        return o


class SearchAttention(_TidalAttention):
    layer_kind = "search"

    def _attend(self, q, c):
        torch.cuda.nvtx.range_push("search_attn")
        o = tidal_utils.decode_sparse_attn(q, c, self.layer_idx, c.kv_indices_without_last, True)
        torch.cuda.nvtx.range_pop()
        torch.cuda.nvtx.range_push("arg_topk")
        tidal_utils.decode_topk(c)
        torch.cuda.nvtx.range_pop()
        return o


class SparseAttention(_TidalAttention):
    layer_kind = "sparse"

    def _attend(self, q, c):
        torch.cuda.nvtx.range_push("sparse_attn")
        if c.need_estimate():
            o = tidal_utils.decode_sparse_attn(q, c, self.layer_idx, c.topk_dindices_buffer, False)
        else:
            # the budget covers the whole context: nothing to leave out
            o = tidal_utils.decode_sparse_attn(q, c, self.layer_idx, c.kv_indices_without_last, False)
        torch.cuda.nvtx.range_pop()
        return o
