"""Decode-step runtime: the whole greedy decode step of `tidaldecode_b200.llama.LlamaForCausalLM` —
every layer, the sampling and the bookkeeping — captured once as a CUDA graph and replayed per token.

The reference runs a step as ~40 host-driven stages per layer with a device synchronisation
around each operator and four `begin_forward` re-plannings per token
(tidal/models/llama.py:505-576, tidal/utils/controller.py:93-177).  Here nothing on the host
changes between tokens: sequence lengths, positions, the token fed back and the output slot are
device tensors that the graph itself advances; pages for the whole generation are reserved
before capture; the kernels take their lengths from the device (`d_seq_lens`, `pos0_dev`,
`d_row_len`), their split-KV plan from the fixed maximum length.

    rt = GraphDecoder(model, max_seq_len=P + steps)      # model.tidal_init() is done for you
    rt.prefill(prompt_ids)                               # eager, through the attention modules
    tokens = rt.decode(steps)                            # [B, steps] greedy tokens, one replay per token
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .attention import FullAttention, SearchAttention, SparseAttention


class GraphDecoder:
    def __init__(self, model, max_seq_len: int, token_budget: Optional[int] = None, dtype: Optional[torch.dtype] = None,
                 device=None, batch_size: int = 1, fused_linear: bool = True):
        self.model = model
        p = next(model.parameters())
        self.dtype = dtype or p.dtype
        self.device = torch.device(device) if device is not None else p.device
        self.B = batch_size
        self.max_seq_len = int(max_seq_len)
        if model.model.iController is None:
            model.tidal_init(page_size=1, max_seq_len=self.max_seq_len, token_budget=token_budget or 256, dtype=self.dtype,
                             device=self.device, batch_size=batch_size)
        self.c = model.model.iController
        if self.c.max_seq_len < self.max_seq_len:
            raise RuntimeError("the model's controller was initialised for a shorter max_seq_len")
        if self.c.batch_size != batch_size:
            raise RuntimeError("batch size differs from the controller's")
        c = self.c
        self.k = min(int(c._token_budget), self.max_seq_len - 1)
        self.rows = c.batch_size * c.score_rows
        i32 = dict(dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros(self.B, **i32)          # tokens per sequence INCLUDING the one being decoded
        self.pos = torch.zeros(self.B, **i32)               # its position
        self.row_lens = torch.zeros(self.rows, **i32)       # seq_lens per score row
        self.sel_counts = torch.zeros(self.rows, **i32)
        self.tok = torch.zeros(self.B, 1, dtype=torch.int64, device=self.device)
        self.step_idx = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.out_tokens = torch.zeros(self.B, self.max_seq_len, dtype=torch.int64, device=self.device)
        self.graph = None
        self.logits = None
        # decode-step projections through tidal_decode_linear (norm, residual and SiLU*up folded in); False = torch ops
        self.fused_linear = fused_linear and batch_size <= 8
        self.lin_status = torch.zeros(1, dtype=torch.int32, device=self.device)      # fault bits of the linear kernels
        # one GEMV for q,k,v and one for gate,up per layer (three and two in the module): fewer launches per token
        self._wqkv, self._wgu = [], []
        for layer in model.model.layers:
            a, mlp = layer.self_attn, layer.mlp
            wqkv = torch.cat((a.q_proj.weight, a.k_proj.weight, a.v_proj.weight), dim=0).contiguous()
            wgu = torch.cat((mlp.gate_proj.weight, mlp.up_proj.weight), dim=0).contiguous()
            # the modules keep working (prefill runs through them) on row ranges of the stacked matrices: no second copy
            nq, nk = a.q_proj.weight.shape[0], a.k_proj.weight.shape[0]
            a.q_proj.weight.data, a.k_proj.weight.data, a.v_proj.weight.data = wqkv[:nq], wqkv[nq:nq + nk], wqkv[nq + nk:]
            f = mlp.gate_proj.weight.shape[0]
            mlp.gate_proj.weight.data, mlp.up_proj.weight.data = wgu[:f], wgu[f:]
            self._wqkv.append(wqkv)
            self._wgu.append(wgu)

    # ------------------------------------------------------------------ prefill
    @torch.inference_mode()
    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """Eager prefill through the model's attention modules; returns the first greedy token [B,1]."""
        c = self.c
        if prompt.shape[0] != self.B:
            raise RuntimeError("prompt batch differs from the decoder's")
        if self.B != 1:
            raise RuntimeError("prefill takes one sequence (decode a batch by prefilling each cache slot yourself)")
        c.clean_states()
        logits = self.model(input_ids=prompt.to(self.device))
        first = logits[:, -1:].argmax(-1)
        P = c.kv_cache.seqlen
        if P + 1 > self.max_seq_len:
            raise RuntimeError("prompt does not leave room for a decoded token")
        c.kv_cache.reserve(self.max_seq_len)                # page table filled once, never touched again
        self.seq_lens.fill_(P + 1)
        self.pos.fill_(P)
        self.row_lens.fill_(P + 1)
        self.tok.copy_(first.view(self.B, 1))
        self.step_idx.zero_()
        self._prefill_len = P
        return first

    @torch.inference_mode()
    def start_from_cache(self, seq_len: int, first_tokens: torch.Tensor) -> None:
        """Begin decoding with KV caches the caller has filled: every sequence holds `seq_len` tokens in the
        controller's cache (pages reserved here, to be written through `self.c.kv_cache.buf_layer(l)` and
        `self.c.kv_cache.page_table` before the first `decode`), and `first_tokens` [B] are fed first.
        The latency benchmark uses it for batches: the reference times decode steps on random data as well
        (scripts/bench_textgen.py:78-89), and prefill takes one sequence at a time."""
        c = self.c
        if seq_len + 1 > self.max_seq_len:
            raise RuntimeError("seq_len does not leave room for a decoded token")
        c.clean_states()
        c.kv_cache.reserve(self.max_seq_len)
        c.kv_cache._seqlen = seq_len
        self.seq_lens.fill_(seq_len + 1)
        self.pos.fill_(seq_len)
        self.row_lens.fill_(seq_len + 1)
        self.tok.copy_(first_tokens.view(self.B, 1).to(self.device))
        self.step_idx.zero_()
        self._prefill_len = seq_len

    # --------------------------------------------------------------- one step
    def _step(self):
        m, c = self.model, self.c
        B, k = self.B, self.k
        table = c.kv_cache.page_table
        ws = c.workspace
        h = m.model.embed_tokens(self.tok).view(B, -1).contiguous()          # [B, hidden], the residual stream (updated in place)
        cnt_shape = (B,) if c.score_rows == 1 else (B, c.num_heads)
        F = torch.nn.functional
        fused = self.fused_linear
        lin = dict(static_weights=True, status=self.lin_status)
        for li, layer in enumerate(m.model.layers):
            att = layer.self_attn
            nq, nkv = att.num_heads * att.head_dim, att.num_key_value_heads * att.head_dim
            ln1, ln2 = layer.input_layernorm, layer.post_attention_layernorm
            pool = c.kv_cache.buf_layer(att.layer_idx)
            rope = dict(pos0_dev=self.pos, page_table=table, rope_theta=att.rope_theta, rope_scale=att.rope_scale,
                        rope_mode=att.rope_mode, inv_freq=att._inv_freq_on(self.device))
            if fused and h.dtype != torch.float32:
                # norm, q|k|v projection, RoPE and the KV append in one launch
                q = torch.empty(B, att.num_heads, att.head_dim, dtype=h.dtype, device=h.device)
                ops.qkv_rope_append(h, self._wqkv[li], q, pool, num_kv_heads=att.num_key_value_heads, norm_weight=ln1.weight,
                                    eps=ln1.variance_epsilon, **rope, **lin)
            else:
                if fused:
                    qkv = ops.linear(h, self._wqkv[li], norm_weight=ln1.weight, eps=ln1.variance_epsilon, **lin)
                else:
                    qkv = F.linear(ln1(h), self._wqkv[li])
                q = qkv[:, :nq].contiguous().view(B, att.num_heads, att.head_dim)
                kk = qkv[:, nq:nq + nkv].contiguous().view(B, att.num_key_value_heads, att.head_dim)
                vv = qkv[:, nq + nkv:].contiguous().view(B, att.num_key_value_heads, att.head_dim)
                ops.rope_append(q, kk, vv, pool, batch=B, **rope)
            o = torch.empty_like(q)
            if isinstance(att, SearchAttention):
                ops.decode_attention(q, pool, self.max_seq_len, ws, out=o, page_table=table, seq_lens=self.seq_lens,
                                     scores=c.qk_product, hist=ws.hist, force_last=c.force_last_token)
                ops.topk(c.qk_product, k, ws, n=self.max_seq_len, out_idx=c._topk_indices_full.view(self.rows, -1),
                         out_val=c._topk_values_full.view(self.rows, -1), force_last=c.force_last_token, hist=ws.hist,
                         row_len=self.row_lens, out_count=self.sel_counts)
            elif isinstance(att, SparseAttention):
                ops.decode_attention(q, pool, self.max_seq_len, ws, out=o, page_table=table, seq_lens=self.seq_lens,
                                     sel_idx=c._topk_indices_full, sel_counts=self.sel_counts.view(cnt_shape))
            else:
                ops.decode_attention(q, pool, self.max_seq_len, ws, out=o, page_table=table, seq_lens=self.seq_lens)
            if fused:
                # o_proj into the residual stream; gate|up behind the second norm with SiLU(gate)*up; down into the stream
                ops.linear(o.view(B, -1), att.o_proj.weight, out=h, residual=h, **lin)
                act = ops.linear(h, self._wgu[li], norm_weight=ln2.weight, eps=ln2.variance_epsilon, silu_mul=True, **lin)
                ops.linear(act, layer.mlp.down_proj.weight, out=h, residual=h, **lin)
            else:
                h = h + att.o_proj(o.view(B, -1))
                gu = F.linear(ln2(h), self._wgu[li])
                ffn = gu.shape[-1] // 2
                h = h + layer.mlp.down_proj(F.silu(gu[..., :ffn]) * gu[..., ffn:])
        if fused:
            logits = ops.linear(h, m.lm_head.weight, norm_weight=m.model.norm.weight, eps=m.model.norm.variance_epsilon, **lin).view(B, 1, -1)
        else:
            logits = m.lm_head(m.model.norm(h)).view(B, 1, -1)
        nxt = logits.argmax(-1)                             # [B,1]
        self.out_tokens.index_copy_(1, self.step_idx, nxt)
        self.tok.copy_(nxt)
        self.step_idx.add_(1)
        self.seq_lens.add_(1)
        self.pos.add_(1)
        self.row_lens.add_(1)
        self.logits = logits

    # ------------------------------------------------------------------ decode
    @torch.inference_mode()
    def decode(self, steps: int, use_graph: bool = True) -> torch.Tensor:
        """`steps` more greedy tokens (the first call continues after the token `prefill` returned);
        returns those `steps` tokens, [B, steps] on the device."""
        asked = steps
        if self._prefill_len + 1 + steps > self.max_seq_len:
            raise RuntimeError("max_seq_len too small for this many steps")
        if not use_graph:
            for _ in range(steps):
                self._step()
        else:
            if self.graph is None:
                # one eager step warms allocator and kernels up (it is a real step: its token is kept)
                self._step()
                steps -= 1
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step()
                self.graph = g
                # the capture pass does not execute: nothing to undo
            for _ in range(steps):
                self.graph.replay()
        done = int(self.step_idx.item())
        self.c.kv_cache._seqlen = self._prefill_len + done      # host bookkeeping catches up with the device
        return self.out_tokens[:, done - asked:done]
