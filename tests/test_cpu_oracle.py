"""CPU tier: the oracle restatement against the fixtures the reference produced."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import tidal_oracle as O
from tests.golden.cases import ATTN_CASES, input_digest, make_case
from tests.helpers import from_np, load_golden


@pytest.mark.parametrize("case", ATTN_CASES, ids=[c[0] for c in ATTN_CASES])
def test_oracle_reproduces_reference_attention(case):
    name, seed, B, Hq, Hkv, D, N, k, dtype, planted = case
    z = load_golden(f"attn_{name}.npz")
    q, K, V = make_case(seed, B, Hq, Hkv, D, N, k, dtype, planted)
    assert input_digest(q, K, V) == str(z["input_sha256"])
    o, idx, mask = O.selection_layer(q, K, V, k, "none")
    assert torch.equal(o, from_np(z["o_select"], dtype))
    sets = torch.sort(idx[:, :, 0, :], dim=-1).values.to(torch.int32)
    assert torch.equal(sets, torch.from_numpy(z["sel_idx"]))
    assert torch.equal(O.sparse_layer(q, K, V, mask), from_np(z["o_sparse"], dtype))


@pytest.mark.parametrize("name,dtype,D", [("f32_d64", torch.float32, 64), ("f16_d128", torch.float16, 128),
                                          ("bf16_d128", torch.bfloat16, 128)])
def test_oracle_reproduces_reference_rope(name, dtype, D):
    z = load_golden("rope.npz")
    q, k = from_np(z[f"{name}_q"], dtype), from_np(z[f"{name}_k"], dtype)
    pos = torch.from_numpy(z[f"{name}_pos"])
    cos, sin = O.rope_cos_sin(pos, D, float(z[f"{name}_theta"]), dtype)
    assert torch.equal(O.apply_rope_path_a(q, cos[:, None], sin[:, None]), from_np(z[f"{name}_qe"], dtype))
    assert torch.equal(O.apply_rope_path_a(k, cos[:, None], sin[:, None]), from_np(z[f"{name}_ke"], dtype))


def test_oracle_reproduces_reference_tiny_model():
    """Config 1: greedy tokens and the layer-3 index sets of the reference model."""
    z = load_golden("tiny_llama_cfg1.npz")
    W = O.TinyLlamaWeights()
    g = torch.Generator().manual_seed(int(z["prompt_seed"]))
    prompt = torch.randint(0, W.vocab, (1, 2048), generator=g)
    with torch.no_grad():
        toks, trace, logits = O.tiny_llama_greedy(W, prompt, 8, 128, 2, 3, return_trace=True, return_logits=True)
    assert toks == z["tokens"][:8].tolist()
    assert torch.equal(logits, torch.from_numpy(z["logits"][:8])), "last-position logits of every step, bit for bit"
    for layer, key in ((2, "layer2_sets"), (3, "layer3_sets")):
        mine = [t[2] for t in trace if t[1] == layer]
        assert len(mine) == 7
        for step, got in enumerate(mine):
            want = torch.from_numpy(z[key][step])
            assert torch.equal(torch.sort(got[0, :, 0, :], dim=-1).values.to(torch.int32), want)


def test_gathered_attention_equals_masked_dense():
    """Gather-based sparse attention == the reference's dense-masked formulation (fp32)."""
    q, K, V = make_case(3, 2, 8, 2, 64, 500, 32, torch.float32, 4)
    _, idx, mask = O.selection_layer(q, K, V, 32, "none")
    dense = O.sparse_layer(q, K, V, mask)
    sparse = O.gathered_attention(q, K, V, idx[:, :, 0, :].to(torch.int32))
    assert torch.allclose(dense, sparse, rtol=1e-5, atol=1e-6)
    _, idx, mask = O.selection_layer(q, K, V, 32, "sum")
    assert mask.shape == (2, 1, 1, 500) and idx.shape == (2, 1, 1, 32)
    dense = O.sparse_layer(q, K, V, mask)
    sparse = O.gathered_attention(q, K, V, idx[:, 0, 0, :].to(torch.int32))
    assert torch.allclose(dense, sparse, rtol=1e-5, atol=1e-6)


def test_force_last_semantics():
    q, K, V = make_case(4, 1, 4, 4, 64, 200, 16, torch.float32, 0)
    S = O.logits(q, K)
    idx, mask = O.select_topk(S, 16, "none", force_last=True)
    assert bool((idx[..., -1] == 199).all()) and int(mask.sum()) == 4 * 16
    ok, why = O.topk_sets_match(S[0, :, 0, :], idx[0, :, 0, :], 16, 0.0, force_last=True)
    assert ok, why


def test_sharded_merge_is_exact():
    """(m,l,o) partials and per-shard top-k candidates merge to the unsharded result."""
    q, K, V = make_case(5, 2, 8, 2, 64, 1000, 64, torch.float32, 8)
    bounds = [0, 1, 400, 400, 1000]          # includes a single-token and an empty shard
    parts, cs, ci = [], [], []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        parts.append(O.partial_attention(q, K[:, :, lo:hi], V[:, :, lo:hi]))
        s = O.scores_fp32(q, K[:, :, lo:hi], "sum")
        kk = min(64, hi - lo)
        if kk:
            v, i = torch.topk(s, kk, dim=-1)
            cs.append(v)
            ci.append(i + lo)
    o = O.merge_partials(parts)
    want = O.gathered_attention(q, K, V, torch.arange(1000, dtype=torch.int32)[None].expand(2, 1000))[:, :, 0]
    assert torch.allclose(o, want, rtol=1e-5, atol=1e-6)
    merged = O.merge_candidates(cs, ci, 64)
    ok, why = O.topk_sets_match(O.scores_fp32(q, K, "sum"), merged, 64, 0.0)
    assert ok, why


def test_paged_append_roundtrip():
    g = torch.Generator().manual_seed(0)
    H, D, page = 3, 8, 4
    pool = torch.zeros(10, 2, page, H, D)
    pages = [7, 2, 9]
    k = torch.randn(9, H, D, generator=g)
    v = torch.randn(9, H, D, generator=g)
    O.append_paged_kv(pool, pages, 9, k, v)
    K, V = O.paged_to_dense(pool, pages, 9)
    assert torch.equal(K[0].permute(1, 0, 2), k) and torch.equal(V[0].permute(1, 0, 2), v)
    assert O.kv_elem_offset(2, 1, 3, 1, 5, page, H, D) == (((2 * 2 + 1) * page + 3) * H + 1) * D + 5
    flat = pool.view(-1)
    assert flat[O.kv_elem_offset(9, 0, 0, 2, 7, page, H, D)] == k[8, 2, 7]


def test_causal_prefill_matches_the_reference_paths():
    """The prefill restatement against (a) the fused causal attention the reference's PyTorch path
    runs below the sparse layers (src/tidal_build/modify_llama.py:84-98) and (b), for a later chunk of
    a prompt, one decode-style full_layer call per row over that row's prefix — the mask of
    kernels/src/include/cpu_reference.h:127."""
    g = torch.Generator().manual_seed(3)
    n, Hq, Hkv, D = 37, 4, 2, 32
    q = torch.randn(n, Hq, D, generator=g)
    K = torch.randn(n, Hkv, D, generator=g)
    V = torch.randn(n, Hkv, D, generator=g)
    got = O.causal_prefill(q, K, V)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1)[None], O.repeat_kv(K.transpose(0, 1)[None], Hq // Hkv), O.repeat_kv(V.transpose(0, 1)[None], Hq // Hkv),
        is_causal=True)[0].transpose(0, 1)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)
    # a chunk: the last 5 rows over all 37 cached tokens
    chunk = O.causal_prefill(q[-5:], K, V)
    for i in range(5):
        upto = n - 5 + i + 1
        row = O.full_layer(q[-5 + i][None, :, None, :], K[:upto].transpose(0, 1)[None], V[:upto].transpose(0, 1)[None])
        assert torch.allclose(chunk[i], row[0, :, 0], rtol=1e-5, atol=1e-6)
    # non-causal: every row sees everything
    full = O.causal_prefill(q[:3], K, V, causal=False)
    row = O.full_layer(q[:3].transpose(0, 1)[None], K.transpose(0, 1)[None], V.transpose(0, 1)[None])
    assert torch.allclose(full, row[0].transpose(0, 1), rtol=1e-5, atol=1e-6)


def test_oracle_reproduces_reference_yarn_hook():
    """The reference's second hook (llama_tidal_forward_yarn, fixture yarn_hook.npz) on the YaRN-style attention stack:
    its decode-step arithmetic is the oracle's selection_layer / sparse_layer on the module's own rotated q, k."""
    import types

    from tests.golden.cases import YARN_CASE, run_attention_stack, yarn_case_model_and_inputs

    z = load_golden("yarn_hook.npz")
    mods, prompt, steps = yarn_case_model_and_inputs()
    c = YARN_CASE

    def hooked(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, output_attentions=False,
               use_cache=False, is_padded_inputs=False):
        bsz, q_len, _ = hidden_states.shape
        if q_len > 1 or self.layer_id < c["sparse_layer_start"]:
            return self.flash_forward(hidden_states, attention_mask, position_ids, past_key_value, output_attentions, use_cache,
                                      is_padded_inputs)
        past_kv, past_len = past_key_value
        q = self.q_proj(hidden_states).view(bsz, 1, self.num_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(bsz, 1, self.num_key_value_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(bsz, 1, self.num_key_value_heads, self.head_dim)
        q, k = self.rotary_emb(q, k, past_len)
        G = self.num_key_value_groups
        K = torch.cat((past_kv[:, :past_len, 0, ::G], k), dim=1).transpose(1, 2)       # [B,Hkv,N,D]
        V = torch.cat((past_kv[:, :past_len, 1, ::G], v), dim=1).transpose(1, 2)
        kv = torch.stack([k, v], 2)[:, :, :, :, None, :].expand(bsz, 1, 2, self.num_key_value_heads, G, self.head_dim)
        if past_len + 1 > past_kv.size(1):
            past_kv = torch.cat([past_kv, torch.empty(bsz, 256, 2, self.num_heads, self.head_dim)], 1)
        past_kv[:, past_len:past_len + 1] = kv.reshape(bsz, 1, 2, self.num_heads, self.head_dim)
        qq = q.transpose(1, 2)
        if self.layer_id in (c["sparse_layer_start"], c["correction_layer"]):
            o, _, self.pos_dict = O.selection_layer(qq, K, V, c["top_k"], "none")
        else:
            o = O.sparse_layer(qq, K, V, self.pos_dict)
        o = self.o_proj(o.transpose(1, 2).reshape(bsz, 1, self.hidden_size))
        return o, None, (past_kv, past_len + 1)

    for i, m in enumerate(mods):
        m.layer_id = i
        m.flash_forward = m.forward
        m.forward = types.MethodType(hooked, m)
    out = run_attention_stack(mods, prompt, steps)
    want = torch.from_numpy(z["out"])
    assert torch.allclose(out, want, rtol=0, atol=1e-5), (out - want).abs().max()
