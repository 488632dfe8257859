"""The caller of the attention path: a Llama decoder with the reference's kernel-path
entry points (tidal/models/llama.py): `LlamaForCausalLM.tidal_init(page_size,
max_seq_len, token_budget, dtype, device)`, `tidal_clear()`, per-forward latency
lists on `model.model.iController`, and the per-layer choice of
Full / Search / Sparse attention (llama.py:351-360).

What differs from the reference: the layer schedule is a parameter
(`selection_layers`; the reference hard-codes Search at layers 2 and 12), the
token budget is not toggled by re-running `begin_forward` four times per token
(llama.py:505-520) because full layers simply ignore it, there is no device
synchronisation inside the layer loop, and grouped-query heads, bf16/fp32 and a
batch of sequences are accepted.  Parameter names match the Hugging Face Llama
state dict, so checkpoints and the oracle's seeded weights load unchanged.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import torch
from torch import nn

from .attention import FullAttention, SearchAttention, SparseAttention
from .utils import InferenceController, rms_norm_forward


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e4
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 4096
    pretraining_tp: int = 1
    # TidalDecode schedule: full attention below selection_layers[0]; the listed layers select
    selection_layers: Tuple[int, ...] = (2, 12)
    head_reduce: str = "none"          # "none": a set per query head (reference); "sum": one shared set
    force_last_token: bool = True      # kernel-path rule; False = the PyTorch path's rule
    tidal_rope_mode: int = 2
    layer_alias: int = 1

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads


class LlamaRMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states):
        return rms_norm_forward(hidden_states, self.weight, self.variance_epsilon)


class LlamaMLP(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig, layer_idx: int, Attention=FullAttention):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.self_attn = Attention(config=config, layer_idx=layer_idx)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, iController: Optional[InferenceController] = None):
        residual = hidden_states
        hidden_states = self.input_layernorm(hidden_states)
        hidden_states, _, _ = self.self_attn(hidden_states=hidden_states, attention_mask=attention_mask,
                                             position_ids=position_ids, past_key_value=past_key_value,
                                             output_attentions=output_attentions, use_cache=use_cache,
                                             iController=iController)
        hidden_states = residual + hidden_states
        residual = hidden_states
        hidden_states = self.post_attention_layernorm(hidden_states)
        hidden_states = self.mlp(hidden_states)
        return (residual + hidden_states,)


def attention_class_for(layer_idx: int, selection_layers: Sequence[int]):
    """Full below the first selection layer, Search at the listed layers, Sparse elsewhere
    (the reference's fixed instance of this rule: tidal/models/llama.py:351-360)."""
    if not selection_layers or layer_idx < min(selection_layers):
        return FullAttention
    if layer_idx in selection_layers:
        return SearchAttention
    return SparseAttention


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([
            LlamaDecoderLayer(config, i, attention_class_for(i, config.selection_layers))
            for i in range(config.num_hidden_layers)])
        self.norm = LlamaRMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.iController: Optional[InferenceController] = None

    def forward(self, input_ids=None, inputs_embeds=None):
        assert self.iController is not None, "call tidal_init() first"
        c = self.iController
        hidden_states = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        bsz, q_len, _ = hidden_states.shape
        t0 = time.perf_counter()
        c.prepare_metadata(q_len)
        c.begin_forward(q_len)
        for layer in self.layers:
            hidden_states = layer(hidden_states, iController=c)[0]
        c.end_forward()
        hidden_states = self.norm(hidden_states)
        if self.record_latency:
            torch.cuda.synchronize()
            (c.prefill_latency if q_len > 1 else c.decode_latency).append((time.perf_counter() - t0) * 1e3)
        return hidden_states

    record_latency = False


class LlamaForCausalLM(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.model = LlamaModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self._config = config

    def tidal_init(self, page_size: int, max_seq_len: int, token_budget: int = 512, dtype: torch.dtype = torch.float16,
                   device=torch.device("cuda:0"), batch_size: int = 1):
        """Allocates the KV pools, the workspace and every per-step buffer; must precede forward
        (tidal/models/llama.py:616-648)."""
        assert self.model.iController is None, "Can't init tidal Controller twice."
        cfg = self._config
        self.model.iController = InferenceController(
            num_layers=cfg.num_hidden_layers, num_heads=cfg.num_attention_heads,
            head_dim=cfg.hidden_size // cfg.num_attention_heads, page_size=page_size, token_budget=token_budget,
            max_seq_len=max_seq_len, dtype=dtype, device=device, num_kv_heads=cfg.num_key_value_heads,
            batch_size=batch_size, head_reduce=cfg.head_reduce, force_last_token=cfg.force_last_token,
            layer_alias=cfg.layer_alias)

    def tidal_clear(self):
        """Forget the cached sequence(s), ready for a new conversation (llama.py:650-656)."""
        assert self.model.iController is not None, "Must be called after init."
        self.model.iController.clean_states()

    def forward(self, input_ids=None, inputs_embeds=None, last_token_only: bool = True):
        h = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds)
        if last_token_only:
            h = h[:, -1:, :]
        return self.lm_head(h)

    @torch.inference_mode()
    def greedy_generate(self, prompt: torch.Tensor, steps: int):
        """Prefill + `steps` greedy tokens for one sequence; returns the token ids."""
        logits = self(input_ids=prompt)
        tok = logits.argmax(-1)
        out = [int(tok)]
        for _ in range(steps - 1):
            logits = self(input_ids=tok.view(1, 1))
            tok = logits.argmax(-1)
            out.append(int(tok))
        return out
