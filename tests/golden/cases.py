"""Seeded inputs of the golden attention cases.

The fixtures hold the reference's OUTPUTS plus a digest of the inputs; the inputs
themselves are regenerated from the seed by `make_case` (torch's CPU generator),
and a test that finds a different digest fails instead of comparing.
"""
from __future__ import annotations

import hashlib

import torch


def input_digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        h.update(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.float32 else t.numpy().tobytes())
    return h.hexdigest()


def make_case(seed, B, Hq, Hkv, D, N, k, dtype, planted=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, 1, D, generator=g)
    K = torch.randn(B, Hkv, N, D, generator=g)
    V = torch.randn(B, Hkv, N, D, generator=g)
    if planted:
        G = Hq // Hkv
        for b in range(B):
            pos = torch.randperm(N, generator=g)[:planted]
            for h in range(Hkv):
                qh = q[b, h * G, 0]
                K[b, h, pos] = 3.0 * qh / qh.norm() + 0.1 * torch.randn(planted, D, generator=g)
    return q.to(dtype), K.to(dtype), V.to(dtype)


ATTN_CASES = [
    # name, seed, B, Hq, Hkv, D, N, k, dtype, planted
    ("f32_mha_d64", 11, 1, 4, 4, 64, 300, 16, torch.float32, 0),
    ("f32_mha_d128", 12, 2, 4, 4, 128, 257, 32, torch.float32, 8),
    ("f16_mha_d128", 13, 1, 8, 8, 128, 1111, 64, torch.float16, 16),
    ("bf16_gqa4_d128", 14, 2, 8, 2, 128, 600, 32, torch.bfloat16, 8),
    ("f16_gqa8_d128", 15, 1, 16, 2, 128, 515, 128, torch.float16, 8),
    ("f32_k_ge_n", 16, 1, 4, 4, 64, 20, 128, torch.float32, 0),
    ("f16_mha_d64", 17, 1, 4, 4, 64, 777, 48, torch.float16, 4),
    # the single-layer benchmark configuration verbatim: Llama-2-7B attention shape, context 32768,
    # 64 planted keys 3*q/|q| + N(0,0.1), top_k 256 (per-q-head sets, as the reference selects)
    ("cfg2_f16_mha_32k", 2, 1, 32, 32, 128, 32768, 256, torch.float16, 64),
]


# ----------------------------------------------------------------------------------------------
# A YaRN-style attention module, as the reference's second hook expects to find it
# (src/tidal_build/modify_llama.py:150-325, 379-391): class name "LlamaAttention", q/k/v/o projections, a
# rotary_emb(q, k, past_len) that returns the rotated q and k itself, a cache that is the tuple
# (kv [B, capacity, 2, heads, D], length), and the forward signature of the YaRN model file.  It stands in
# for that model's module in the fixture generator (driven through the reference's own
# llama_tidal_forward_yarn) and in the tests of this package's hook.
class YarnRotary(torch.nn.Module):
    def __init__(self, dim, base=10000.0, scale=4.0, original_max=64, beta_fast=32.0, beta_slow=1.0):
        super().__init__()
        import math
        pos_freqs = base ** (torch.arange(0, dim, 2).float() / dim)
        extrapolation, interpolation = 1.0 / pos_freqs, 1.0 / (scale * pos_freqs)

        def correction_dim(rot):
            return (dim * math.log(original_max / (rot * 2 * math.pi))) / (2 * math.log(base))

        low, high = max(math.floor(correction_dim(beta_fast)), 0), min(math.ceil(correction_dim(beta_slow)), dim - 1)
        ramp = ((torch.arange(dim // 2).float() - low) / max(high - low, 1e-3)).clamp(0, 1)
        self.register_buffer("inv_freq", interpolation * ramp + extrapolation * (1 - ramp), persistent=False)
        self.mscale = 0.1 * math.log(scale) + 1.0

    def forward(self, q, k, past_len):
        """q [B, n, Hq, D], k [B, n, Hkv, D]; positions past_len .. past_len + n - 1."""
        n = q.shape[1]
        t = torch.arange(past_len, past_len + n, device=q.device, dtype=torch.float32)
        freqs = torch.outer(t, self.inv_freq.to(q.device))
        emb = torch.cat((freqs, freqs), dim=-1)
        cos, sin = (emb.cos() * self.mscale).to(q.dtype)[None, :, None, :], (emb.sin() * self.mscale).to(q.dtype)[None, :, None, :]

        def rot(x):
            h = x.shape[-1] // 2
            return torch.cat((-x[..., h:], x[..., :h]), dim=-1)

        return q * cos + rot(q) * sin, k * cos + rot(k) * sin


def make_yarn_style_attention_class():
    """The class is built on demand so that importing this file needs no torch.nn machinery at collection time."""
    import math
    import types

    nn = torch.nn

    class LlamaAttention(nn.Module):
        def __init__(self, hidden, heads, kv_heads, seed):
            super().__init__()
            self.config = types.SimpleNamespace(pretraining_tp=1, num_attention_heads=heads, num_key_value_heads=kv_heads)
            self.hidden_size, self.num_heads, self.num_key_value_heads = hidden, heads, kv_heads
            self.head_dim = hidden // heads
            self.num_key_value_groups = heads // kv_heads
            g = torch.Generator().manual_seed(seed)

            def lin(o, i):
                m = nn.Linear(i, o, bias=False)
                with torch.no_grad():
                    m.weight.copy_(torch.randn(o, i, generator=g) / math.sqrt(i))
                return m

            self.q_proj, self.k_proj = lin(heads * self.head_dim, hidden), lin(kv_heads * self.head_dim, hidden)
            self.v_proj, self.o_proj = lin(kv_heads * self.head_dim, hidden), lin(hidden, heads * self.head_dim)
            self.rotary_emb = YarnRotary(self.head_dim)
            self.pos_dict = None

        def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, output_attentions=False,
                    use_cache=False, is_padded_inputs=False):
            """Plain causal attention with the tuple cache of the YaRN model file (its flash path, in eager form)."""
            bsz, q_len, _ = hidden_states.shape
            past_kv, past_len = past_key_value if past_key_value is not None else (None, 0)
            q = self.q_proj(hidden_states).view(bsz, q_len, self.num_heads, self.head_dim)
            k = self.k_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim)
            v = self.v_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim)
            q, k = self.rotary_emb(q, k, past_len)
            G = self.num_key_value_groups
            kv = torch.stack([k, v], 2)[:, :, :, :, None, :].expand(bsz, q_len, 2, self.num_key_value_heads, G, self.head_dim)
            kv = kv.reshape(bsz, q_len, 2, self.num_heads, self.head_dim)
            if past_kv is not None:
                new_len = past_len + q_len
                if new_len > past_kv.size(1):
                    past_kv = torch.cat([past_kv, torch.empty(bsz, 256, 2, kv.size(3), kv.size(4), dtype=kv.dtype, device=kv.device)], 1)
                past_kv[:, past_len:new_len] = kv
                kv = past_kv[:, :new_len]
            else:
                past_kv = kv
            kk, vv = kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)
            n_all = kk.shape[2]
            mask = torch.ones(q_len, n_all, dtype=torch.bool, device=q.device).tril(diagonal=n_all - q_len)
            o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, attn_mask=mask)
            o = self.o_proj(o.transpose(1, 2).reshape(bsz, q_len, self.hidden_size))
            return o, None, ((past_kv, past_len + q_len) if use_cache else None)

    return LlamaAttention


YARN_CASE = dict(hidden=256, heads=4, kv_heads=2, layers=4, prompt=300, steps=6, top_k=32, sparse_layer_start=1,
                 correction_layer=3, seed=31)


def yarn_case_model_and_inputs(dtype=torch.float32):
    """(list of attention modules, prompt hidden states [1, P, hidden], per-step hidden states [steps, 1, 1, hidden])."""
    c = YARN_CASE
    cls = make_yarn_style_attention_class()
    mods = [cls(c["hidden"], c["heads"], c["kv_heads"], c["seed"] + i).to(dtype).eval() for i in range(c["layers"])]
    g = torch.Generator().manual_seed(c["seed"])
    prompt = torch.randn(1, c["prompt"], c["hidden"], generator=g).to(dtype)
    steps = torch.randn(c["steps"], 1, 1, c["hidden"], generator=g).to(dtype)
    return mods, prompt, steps


def run_attention_stack(mods, prompt, steps):
    """Residual stack of the attention modules (x = x + attn(x)) with the YaRN model's threading of the selected set from
    layer to layer (src/models/yarn_tidaldecoding.py:1151-1197).  Returns the last layer's outputs per decode step."""
    caches = [None] * len(mods)
    outs = []

    def forward(x):
        pos_dict = None
        for i, m in enumerate(mods):
            m.pos_dict = pos_dict
            o, _, caches[i] = m.forward(x, None, None, caches[i], False, True, False)
            pos_dict = m.pos_dict
            x = x + o
        return x

    with torch.no_grad():
        forward(prompt)
        for s in range(steps.shape[0]):
            outs.append(forward(steps[s]))
    return torch.cat(outs, dim=1)[0]           # [steps, hidden]
