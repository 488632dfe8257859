"""enable_tidal on a Hugging Face Llama (the installed transformers): same call as the
reference's src/enable_tidal.py, same greedy tokens as the reference model produced
(fixture), attention by the sm_100a kernels during decode."""
from __future__ import annotations

import pytest
import torch

from oracle import tidal_oracle as O
from tests.helpers import load_golden

pytestmark = pytest.mark.gpu


def _hf_model(W, dtype):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=W.vocab, hidden_size=W.hidden, intermediate_size=W.ffn, num_hidden_layers=W.layers,
                      num_attention_heads=W.heads, num_key_value_heads=W.kv_heads, rms_norm_eps=W.eps,
                      max_position_embeddings=4096, hidden_act="silu", tie_word_embeddings=False, rope_theta=W.theta)
    cfg._attn_implementation = "sdpa"
    m = LlamaForCausalLM(cfg).eval()
    missing = m.load_state_dict(W.hf_state_dict(), strict=False)
    assert not [k for k in missing.missing_keys if "inv_freq" not in k], missing
    return m.to(dtype).cuda()


def _greedy(model, prompt, steps, logits_out=None):
    from transformers.cache_utils import DynamicCache

    toks = []
    with torch.inference_mode():
        cache = DynamicCache()
        out = model(prompt, past_key_values=cache, use_cache=True)
        if logits_out is not None:
            logits_out.append(out.logits[0, -1].float().cpu())
        tok = out.logits[:, -1:].argmax(-1)
        toks.append(int(tok))
        for _ in range(steps - 1):
            out = model(tok.view(1, 1), past_key_values=cache, use_cache=True)
            if logits_out is not None:
                logits_out.append(out.logits[0, -1].float().cpu())
            tok = out.logits[:, -1:].argmax(-1)
            toks.append(int(tok))
    return toks


def test_enable_tidal_on_hf_llama_matches_reference_tokens():
    from tidaldecode_b200.enable_tidal import enable_tidal

    z = load_golden("tiny_llama_cfg1.npz")
    W = O.TinyLlamaWeights()
    g = torch.Generator().manual_seed(int(z["prompt_seed"]))
    prompt = torch.randint(0, W.vocab, (1, 2048), generator=g).cuda()
    model = _hf_model(W, torch.float32)
    enable_tidal(model, attn_type="tidal", top_k=128, sparse_layer_start=2, correction_layer=3, max_seq_len=2048 + 64)
    attn = model.model.layers[0].self_attn
    assert hasattr(attn, "flash_forward")                       # the original forward is kept (modify_llama.py:366)
    step_logits = []
    toks = _greedy(model, prompt, 32, step_logits)
    assert toks == z["tokens"].tolist()
    want_logits = torch.from_numpy(z["logits"])
    err = (torch.stack(step_logits) - want_logits).abs().max().item()
    assert torch.allclose(torch.stack(step_logits), want_logits, rtol=1e-4, atol=1e-5), f"per-step logits differ by {err:.3e}"
    c = model._tidal_state.controller
    assert c.workspace.status() == 0
    sets = torch.sort(c.topk_dindices_buffer[0].cpu(), dim=-1).values
    want = torch.from_numpy(z["layer3_sets"][-1])
    diff = sum(len(set(sets[h].tolist()) ^ set(want[h].tolist())) for h in range(W.heads))
    assert diff <= 4, diff
    # a second sequence through the same model: state is reset when the cache is empty again
    assert _greedy(model, prompt, 4) == z["tokens"][:4].tolist()
    # attn_type other than "tidal" leaves the original forward in place
    enable_tidal(model, attn_type="full", top_k=128)
    assert model.model.layers[0].self_attn.forward == model.model.layers[0].self_attn.flash_forward


def test_enable_tidal_gqa_bf16_head_sum():
    """Shared-set mode on a GQA bf16 model: decode logits stay close to the dense model's
    when the budget covers the context (nothing is dropped)."""
    from tidaldecode_b200.enable_tidal import enable_tidal

    W = O.TinyLlamaWeights(vocab=256, hidden=512, layers=4, heads=8, kv_heads=2, ffn=256, seed=5, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, W.vocab, (1, 200), generator=g).cuda()
    dense = _hf_model(W, torch.bfloat16)
    want = _greedy(dense, prompt, 6)
    model = _hf_model(W, torch.bfloat16)
    enable_tidal(model, top_k=1024, sparse_layer_start=1, correction_layer=2, head_reduce="sum", max_seq_len=512)
    got = _greedy(model, prompt, 6)
    assert sum(a == b for a, b in zip(got, want)) >= 5, (got, want)
    assert model._tidal_state.controller.workspace.status() == 0


def test_enable_tidal_yarn_style_modules_match_reference():
    """The YaRN form of the hook (modules with their own rotary_emb(q, k, past_len) and a tuple cache) against the
    outputs the reference's llama_tidal_forward_yarn produced on the same attention stack (fixture yarn_hook.npz)."""
    from tests.golden.cases import YARN_CASE, run_attention_stack, yarn_case_model_and_inputs
    from tidaldecode_b200.enable_tidal import enable_tidal_yarn_modules

    z = load_golden("yarn_hook.npz")
    mods, prompt, steps = yarn_case_model_and_inputs()
    mods = [m.cuda() for m in mods]
    state = enable_tidal_yarn_modules(mods, "tidal", YARN_CASE["top_k"], YARN_CASE["sparse_layer_start"], YARN_CASE["correction_layer"],
                                      max_seq_len=512)
    assert all(hasattr(m, "flash_forward") for m in mods)
    out = run_attention_stack(mods, prompt.cuda(), steps.cuda()).float().cpu()
    want, dense = torch.from_numpy(z["out"]), torch.from_numpy(z["dense"])
    err = (out - want).abs().max().item()
    assert torch.allclose(out, want, rtol=1e-4, atol=2e-4), f"differs from the reference's hook by {err:.3e}"
    assert (out - dense).abs().max() > 0.1, "the outputs must be those of sparse attention, not of the dense stack"
    assert state.controller.workspace.status() == 0
    # a second sequence through the same modules: the pool is recognised as stale and refilled
    out2 = run_attention_stack(mods, prompt.cuda(), steps.cuda()).float().cpu()
    assert torch.allclose(out2, out, rtol=0, atol=1e-6)
