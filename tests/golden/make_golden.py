"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Runs only where the TidalDecode checkout is present (pass its root with --ref);
the fixtures it writes are committed so that the tests never need the checkout.

What it does
  1. imports the reference's `llama_tidal_attention_forward`
     (src/tidal_build/modify_llama.py:19-148) with harness-side shims for the
     newer `transformers` in this image (nothing in the reference is edited);
  2. drives it directly, with projections that return seeded q / k / v, on small
     attention cases (fp32, fp16, bf16; MHA and GQA) and stores the outputs plus a
     digest of the seeded inputs (tests/golden/cases.py regenerates them);
  3. drives the reference's whole model (src/models/llama_tidaldecoding.py) on the
     tiny 4-layer decoder with weights from `oracle.tidal_oracle.TinyLlamaWeights`
     and stores the greedy tokens and the selected index sets;
  4. asserts that the restatement in oracle/tidal_oracle.py reproduces 2. and 3.
     bit for bit before anything is written.

    python tests/golden/make_golden.py --ref /path/to/TidalDecode
"""
from __future__ import annotations

import argparse
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import tidal_oracle as O  # noqa: E402
from tests.golden.cases import ATTN_CASES, make_case, input_digest  # noqa: E402


def import_reference(ref_root: str):
    """Shims: (1) `LlamaSdpaAttention` no longer exists in transformers 5 — the
    reference imports the name (modify_llama.py:10) but never uses it; (2) the
    "default" rope init was dropped from ROPE_INIT_FUNCTIONS
    (llama_tidaldecoding.py:175)."""
    import transformers.models.llama.modeling_llama as ml
    import transformers.modeling_rope_utils as ru

    if not hasattr(ml, "LlamaSdpaAttention"):
        ml.LlamaSdpaAttention = ml.LlamaAttention

    def _default_rope(config, device=None, seq_len=None, **kw):
        base = config.rope_theta
        dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.int64).float().to(device) / dim))
        return inv, 1.0

    ru.ROPE_INIT_FUNCTIONS.setdefault("default", _default_rope)
    sys.path.insert(0, ref_root)
    import src.tidal_build.modify_llama as mod
    import src.models.llama_tidaldecoding as lt
    return mod, lt


class _Cache:
    """Minimal cache the reference forward needs (modify_llama.py:75-80)."""

    def __init__(self, K, V):
        self.K, self.V = K, V          # [B,Hkv,N-1,D] history

    def update(self, k, v, layer_idx, kwargs=None):
        self.K = torch.cat((self.K, k), dim=2)
        self.V = torch.cat((self.V, v), dim=2)
        return self.K, self.V

    def get_seq_length(self, layer_idx=0):
        return self.K.shape[2]


def ref_attention(mod, q, K, V, top_k, kind, pos_dict=None):
    """Call the reference forward on explicit q [B,Hq,1,D], K,V [B,Hkv,N,D]
    (the newest token is K[:,:,-1]).  kind: 'select' | 'sparse'."""
    B, Hq, _, D = q.shape
    Hkv = K.shape[1]
    self = types.SimpleNamespace()
    self.num_heads, self.num_key_value_heads, self.head_dim = Hq, Hkv, D
    self.num_key_value_groups = Hq // Hkv
    self.attention_dropout, self.training = 0.0, False
    self.q_proj = lambda h: q.transpose(1, 2).reshape(B, 1, Hq * D)
    self.k_proj = lambda h: K[:, :, -1:].transpose(1, 2).reshape(B, 1, Hkv * D)
    self.v_proj = lambda h: V[:, :, -1:].transpose(1, 2).reshape(B, 1, Hkv * D)
    self.o_proj = lambda a: a
    self.pos_dict = pos_dict
    self.layer_idx = 2 if kind == "select" else 3
    cache = _Cache(K[:, :, :-1], V[:, :, :-1])
    cos = torch.ones(B, 1, D, dtype=q.dtype)
    sin = torch.zeros(B, 1, D, dtype=q.dtype)
    hidden = torch.zeros(B, 1, Hq * D, dtype=q.dtype)
    out, _, _ = mod.llama_tidal_attention_forward(
        self, hidden, None, None, cache, False, True, None, (cos, sin),
        top_k=top_k, sparse_layer_start=2, correction_layer=9)
    return out.view(B, 1, Hq, D).transpose(1, 2), self.pos_dict


def gen_attention(mod, outdir):
    for name, seed, B, Hq, Hkv, D, N, k, dtype, planted in ATTN_CASES:
        q, K, V = make_case(seed, B, Hq, Hkv, D, N, k, dtype, planted)
        o_sel, pos_dict = ref_attention(mod, q, K, V, k, "select")
        o_sp, _ = ref_attention(mod, q, K, V, k, "sparse", pos_dict=pos_dict)
        # restatement must agree bit for bit
        o2, idx2, mask2 = O.selection_layer(q, K, V, k, "none")
        assert torch.equal(o2, o_sel), name
        assert torch.equal(mask2, pos_dict), name
        assert torch.equal(O.sparse_layer(q, K, V, mask2), o_sp), name
        sel = torch.nonzero(pos_dict[:, :, 0, :])[:, 2].view(B, Hq, min(N, k)).to(torch.int32)
        as_np = (lambda t: t.view(torch.int16).numpy()) if dtype != torch.float32 else (lambda t: t.numpy())
        np.savez_compressed(
            os.path.join(outdir, f"attn_{name}.npz"),
            dtype=str(dtype).replace("torch.", ""), top_k=k,
            input_sha256=input_digest(q, K, V),
            o_select=as_np(o_sel.contiguous()), o_sparse=as_np(o_sp.contiguous()), sel_idx=sel.numpy())
        print("attn", name, "ok; |sel| per head", sel.shape[-1])


def gen_rope(lt, outdir):
    """apply_rotary_pos_emb of the reference model file on seeded q,k."""
    g = torch.Generator().manual_seed(21)
    out = {}
    for name, dtype, D, theta in [("f32_d64", torch.float32, 64, 1e4), ("f16_d128", torch.float16, 128, 1e4),
                                  ("bf16_d128", torch.bfloat16, 128, 5e5)]:
        H, n = 4, 6
        q = torch.randn(1, H, n, D, generator=g).to(dtype)
        k = torch.randn(1, H, n, D, generator=g).to(dtype)
        pos = torch.tensor([[0, 1, 17, 2047, 32768, 131071]])
        cfg = types.SimpleNamespace(rope_theta=theta, head_dim=D, hidden_size=H * D, num_attention_heads=H,
                                    rope_scaling=None, max_position_embeddings=1 << 20)
        rot = lt.LlamaRotaryEmbedding(config=cfg)
        cos, sin = rot(q, pos)
        qe, ke = lt.apply_rotary_pos_emb(q, k, cos, sin)
        c2, s2 = O.rope_cos_sin(pos, D, theta, dtype)
        assert torch.equal(c2, cos) and torch.equal(s2, sin), name
        assert torch.equal(O.apply_rope_path_a(q, c2[:, None], s2[:, None]), qe), name
        cv = (lambda t: t.view(torch.int16).numpy()) if dtype != torch.float32 else (lambda t: t.numpy())
        out[f"{name}_q"], out[f"{name}_k"] = cv(q), cv(k)
        out[f"{name}_qe"], out[f"{name}_ke"] = cv(qe.contiguous()), cv(ke.contiguous())
        out[f"{name}_pos"] = pos.numpy()
        out[f"{name}_theta"] = theta
        print("rope", name, "ok")
    np.savez_compressed(os.path.join(outdir, "rope.npz"), **out)


def gen_tiny_model(lt, mod, outdir):
    """Config 1: 4 layers, hidden 256, 4x64 MHA, FFN 688, vocab 1024, fp32,
    prompt 2048, selection at layer 2 and again at 3, top_k 128, 32 greedy steps."""
    from transformers import LlamaConfig
    from transformers.cache_utils import DynamicCache

    W = O.TinyLlamaWeights()
    cfg = LlamaConfig(vocab_size=W.vocab, hidden_size=W.hidden, intermediate_size=W.ffn, num_hidden_layers=W.layers,
                      num_attention_heads=W.heads, num_key_value_heads=W.kv_heads, rms_norm_eps=W.eps,
                      max_position_embeddings=4096, hidden_act="silu", tie_word_embeddings=False)
    cfg.rope_theta = W.theta
    cfg.rope_scaling = None
    cfg._attn_implementation = "sdpa"
    model = lt.LlamaForCausalLM(cfg).eval()
    missing = model.load_state_dict(W.hf_state_dict(), strict=False)
    assert not [m for m in missing.missing_keys if "inv_freq" not in m], missing
    import src.enable_tidal as et
    et.enable_tidal(model, attn_type="tidal", top_k=128, sparse_layer_start=2, correction_layer=3)
    patched = sum(hasattr(m, "flash_forward") for m in model.modules())
    assert patched == W.layers, patched

    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, W.vocab, (1, 2048), generator=g)
    steps = 32
    toks, sets, sets2, logits = [], [], [], []

    def sets_of(layer):
        pd = model.model.layers[layer].self_attn.pos_dict
        return torch.nonzero(pd[0, :, 0, :])[:, 1].view(W.heads, -1).to(torch.int32)

    with torch.no_grad():
        cache = DynamicCache()
        out = model(prompt, past_key_values=cache, use_cache=True)
        logits.append(out.logits[0, -1].clone())
        tok = out.logits[:, -1:].argmax(-1)
        toks.append(int(tok))
        for s in range(steps - 1):
            out = model(tok.view(1, 1), past_key_values=cache, use_cache=True)
            sets2.append(sets_of(2))
            sets.append(sets_of(3))
            logits.append(out.logits[0, -1].clone())
            tok = out.logits[:, -1:].argmax(-1)
            toks.append(int(tok))
    with torch.no_grad():
        toks2, trace, logits2 = O.tiny_llama_greedy(W, prompt, steps, 128, 2, 3, return_trace=True, return_logits=True)
    assert toks2 == toks, (toks, toks2)
    assert torch.equal(logits2, torch.stack(logits)), "the restatement's per-step logits differ from the reference model's"
    for layer, got in ((2, sets2), (3, sets)):
        mine = [t[2] for t in trace if t[1] == layer]
        assert len(mine) == len(got)
        for a, b in zip(got, mine):
            assert torch.equal(a, torch.sort(b[0, :, 0, :], dim=-1).values.to(torch.int32))
    # tokens, the last-position logits of every step (the prefill's first) and the sets selected at
    # layers 2 and 3 in every decode step, each sorted by position
    np.savez_compressed(os.path.join(outdir, "tiny_llama_cfg1.npz"), prompt_seed=0, tokens=np.array(toks, np.int64),
                        layer3_sets=torch.stack(sets).numpy(), layer2_sets=torch.stack(sets2).numpy(),
                        logits=torch.stack(logits).numpy())
    print("tiny model ok; tokens", toks)


def gen_yarn_hook(mod, outdir):
    """The reference's second hook, llama_tidal_forward_yarn (modify_llama.py:150-325), installed on a stack of YaRN-style
    attention modules exactly as enable_llama_tidal_attention does for that model family (:379-391): outputs of the last
    layer over a prompt and a few decode steps."""
    from tests.golden.cases import YARN_CASE, run_attention_stack, yarn_case_model_and_inputs

    mods, prompt, steps = yarn_case_model_and_inputs()
    for i, m in enumerate(mods):
        m.layer_id = i
        m.flash_forward = m.forward
        m.forward = types.MethodType(mod.llama_tidal_forward_yarn, m)
        m.token_budget = YARN_CASE["top_k"]
        m.sparse_layer_start = YARN_CASE["sparse_layer_start"]
        m.correction_layer = YARN_CASE["correction_layer"]
    out = run_attention_stack(mods, prompt, steps)
    # the same stack without the hook (dense attention everywhere) must differ: the budget is below the context
    dense_mods, _, _ = yarn_case_model_and_inputs()
    dense = run_attention_stack(dense_mods, prompt, steps)
    assert not torch.allclose(out, dense, atol=1e-4), "the hook did not change anything"
    np.savez_compressed(os.path.join(outdir, "yarn_hook.npz"), out=out.numpy(), dense=dense.numpy())
    print("yarn hook ok; |out - dense| max", float((out - dense).abs().max()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    torch.manual_seed(0)
    mod, lt = import_reference(a.ref)
    gen_attention(mod, a.out)
    gen_rope(lt, a.out)
    gen_tiny_model(lt, mod, a.out)
    gen_yarn_hook(mod, a.out)


if __name__ == "__main__":
    main()
