"""GPU parity of the reference-shaped layers: the `_kernels` drop-in, the operator
façade + InferenceController, the three attention modules and the decoder that
calls them — against the CPU oracle and the reference's fixtures."""
from __future__ import annotations

import pytest
import torch

from oracle import tidal_oracle as O
from tests.helpers import assert_close, load_golden, make_qkv

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    import tidaldecode_b200._kernels as k
    return k


def test_kernels_surface_matches_reference_names(K):
    """tidal/ops/csrc/bsk_ops.cu:4-20: seven functions and one class."""
    for name in ("apply_rope_in_place", "rms_norm_forward", "topk_filtering", "estimate_attn_score",
                 "append_kv_cache_prefill", "append_kv_cache_decode", "prefill_with_paged_kv_cache"):
        assert callable(getattr(K, name)), name
    w = K.BatchDecodeWithPagedKVCachePyTorchWrapper(0)
    for m in ("begin_forward", "end_forward", "forward"):
        assert callable(getattr(w, m)), m


def test_kernels_rope_append_roundtrip(K):
    """apply_rope_in_place + append_kv_cache_{prefill,decode} as the reference calls them
    (tidal/utils/__init__.py:46-52, 97-128), checked like kernels/src/test/test_page.cu does."""
    H, D, page = 32, 128, 1
    g = torch.Generator().manual_seed(0)
    n0 = 37
    pool = torch.zeros(64, 2, page, H, D, dtype=torch.float16, device="cuda")
    pages = torch.randperm(64, generator=g)[: n0 + 1].to(torch.int32)
    q = torch.randn(n0, H, D, generator=g).half()
    k = torch.randn(n0, H, D, generator=g).half()
    v = torch.randn(n0, H, D, generator=g).half()
    qd, kd = q.clone().cuda(), k.clone().cuda()
    K.apply_rope_in_place(qd, kd, 0, 1.0, 1e4)
    want_k = O.apply_rope_fp32(k, torch.arange(n0), 1e4)
    assert torch.allclose(kd.cpu().float(), want_k.float(), atol=2 ** -8, rtol=0)
    assert torch.allclose(qd.cpu().float(), O.apply_rope_fp32(q, torch.arange(n0), 1e4).float(), atol=2 ** -8, rtol=0)
    idx = pages[:n0].cuda()
    indptr = torch.tensor([0, n0], dtype=torch.int32, device="cuda")
    meta = torch.zeros_like(pool)               # Quest's per-page key bounds; with pages of one token both planes equal the key
    K.append_kv_cache_prefill(kd, v.cuda(), pool, idx, indptr, 1, int(pages[n0 - 1]), meta, idx, indptr, 1, 0, 0)
    # one decode token
    k1 = torch.randn(1, H, D, generator=g).half().cuda()
    v1 = torch.randn(1, H, D, generator=g).half().cuda()
    idx1 = pages[: n0 + 1].cuda()
    indptr1 = torch.tensor([0, n0 + 1], dtype=torch.int32, device="cuda")
    K.append_kv_cache_decode(k1, v1, pool, idx1, indptr1, 1, int(pages[n0]), meta, idx1, indptr1, 1, 0, 0)
    want = torch.zeros(64, 2, page, H, D, dtype=torch.float16)
    O.append_paged_kv(want, pages.tolist(), n0, kd.cpu(), v)
    O.append_paged_kv(want, pages.tolist(), n0 + 1, k1.cpu(), v1.cpu())
    assert torch.equal(pool.cpu(), want)
    assert torch.equal(meta.cpu()[:, 0], want[:, 0]) and torch.equal(meta.cpu()[:, 1], want[:, 0])
    # no metadata pool given: the append alone (TidalDecode's own layers never read the metadata)
    K.append_kv_cache_decode(k1, v1, pool, idx1, indptr1, 1, int(pages[n0]), None, None, None, 0, 0, 0)
    with pytest.raises(RuntimeError):
        K.append_kv_cache_decode(kd, v.cuda(), pool, idx1, indptr1, 1, 0, pool, idx1, indptr1, 1, 0, 0)   # more than one token


def test_kernels_wrapper_forward_and_topk_filtering(K):
    """The reference's literal decode contract: per-head page lists + the newest token's page,
    logits into qk_product, top-k gathering page ids (approx_attn.cu:68-151, topk.cu:7-44)."""
    B, H, D, N, budget = 1, 32, 128, 700, 64
    q, Kd, Vd = make_qkv(5, B, H, H, D, N, torch.float16, planted=16)
    g = torch.Generator().manual_seed(2)
    perm = torch.randperm(N + 5, generator=g)[:N].to(torch.int32)          # page of position j
    pool = torch.zeros(N + 5, 2, 1, H, D, dtype=torch.float16)
    pool[perm.long(), 0, 0] = Kd[0].permute(1, 0, 2)
    pool[perm.long(), 1, 0] = Vd[0].permute(1, 0, 2)
    pool = pool.cuda()
    w = K.BatchDecodeWithPagedKVCachePyTorchWrapper(0)
    qd = q[0, :, 0][None].contiguous().cuda()
    o = torch.empty_like(qd)
    hist_pages = perm[: N - 1].cuda()[None].expand(H, N - 1).contiguous()
    with pytest.raises(RuntimeError):
        w.forward(qd, o, pool, hist_pages, None, 1, int(perm[N - 1]), torch.empty(0), 1.0, 1e4)
    indptr = torch.tensor([0, N - 1], dtype=torch.int32, device="cuda")
    w.begin_forward(indptr, H, H, D, 1, torch.empty(0, dtype=torch.float16))
    qk = torch.zeros(H, N + 10, dtype=torch.float32, device="cuda")
    w.forward(qd, o, pool, hist_pages, indptr, 1, int(perm[N - 1]), qk, 1.0, 1e4)
    allidx = torch.arange(N, dtype=torch.int32)[None]
    assert_close(o, O.gathered_attention(q, Kd, Vd, allidx)[:, :, 0], torch.float16, "wrapper.forward over all pages")
    want_s = O.scores_fp32(q, Kd, "none")[0]
    assert torch.allclose(qk[:, :N].cpu(), want_s, rtol=1e-4, atol=2e-4)
    # top-k over the logits, gathering page ids (one shared row of ids, broadcast as the reference repeats it)
    ids = perm.cuda()[None].expand(H, N)
    d_out = torch.zeros(H, budget, dtype=torch.float32, device="cuda")
    i_out = torch.zeros(H, budget, dtype=torch.int32, device="cuda")
    K.topk_filtering(qk, ids, d_out, i_out, torch.empty(0), budget, length=N)
    inv = torch.empty(N + 5, dtype=torch.long)
    inv[perm.long()] = torch.arange(N)
    pos = inv[i_out.cpu().long()]
    ok, why = O.topk_sets_match(want_s, pos, budget, tie_band=1e-4)
    assert ok, why
    # sparse pass over the chosen pages (newest token appended by the wrapper)
    sel_pages = i_out[:, : budget - 1].contiguous()
    w.forward(qd, o, pool, sel_pages, indptr, 1, int(perm[N - 1]), torch.empty(0), 1.0, 1e4)
    sel_pos = torch.cat((pos[:, : budget - 1], torch.full((H, 1), N - 1)), dim=1)[None].to(torch.int32)
    assert_close(o, O.gathered_attention(q, Kd, Vd, sel_pos)[:, :, 0], torch.float16, "wrapper.forward over selected pages")
    w.end_forward()
    with pytest.raises(ValueError):
        w.begin_forward(indptr, 32, 5, D, 1, torch.empty(0, dtype=torch.float16))      # decode_attn.cuh:1143-1148
    with pytest.raises(RuntimeError):
        K.estimate_attn_score(qd, o, pool, hist_pages, indptr, 1, 0, 0)


def _tiny_model(W, dtype, selection_layers, head_reduce, force_last, rope_mode):
    from tidaldecode_b200.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=W.vocab, hidden_size=W.hidden, intermediate_size=W.ffn, num_hidden_layers=W.layers,
                      num_attention_heads=W.heads, num_key_value_heads=W.kv_heads, rms_norm_eps=W.eps, rope_theta=W.theta,
                      selection_layers=selection_layers, head_reduce=head_reduce, force_last_token=force_last,
                      tidal_rope_mode=rope_mode)
    m = LlamaForCausalLM(cfg)
    missing = m.load_state_dict(W.hf_state_dict(), strict=True)
    return m.to(dtype).cuda().eval()


def _set_differences_inside_tie_band(scores, got, want, band):
    """Indices present in only one of two top-k sets must all have scores within `band` of the k-th
    score (near-ties that fp32 on the device and on the host may order differently).  scores [N] fp32."""
    a, b = set(got.tolist()), set(want.tolist())
    only = sorted(a ^ b)
    if not only:
        return 0
    kth = torch.topk(scores, len(b)).values[-1]
    worst = (scores[torch.tensor(only)] - kth).abs().max().item()
    assert worst <= band, f"sets differ at {only} with scores {worst:.3e} away from the k-th"
    return len(only)


def test_tiny_llama_greedy_matches_reference():
    """Configuration 1 through the attention modules in reference-parity mode (per-head sets, newest token
    not forced, fp32) against what the reference model produced (fixture): the greedy tokens, the
    last-position logits of every step, and the sets selected at layers 2 and 3 in every decode step."""
    z = load_golden("tiny_llama_cfg1.npz")
    W = O.TinyLlamaWeights()
    g = torch.Generator().manual_seed(int(z["prompt_seed"]))
    prompt = torch.randint(0, W.vocab, (1, 2048), generator=g)
    m = _tiny_model(W, torch.float32, (2, 3), "none", False, 1)
    m.tidal_init(page_size=1, max_seq_len=2048 + 64, token_budget=128, dtype=torch.float32, device=torch.device("cuda"))
    steps = 32
    c = m.model.iController
    sets = {2: [], 3: []}
    scores = {2: [], 3: []}

    def grab(layer):
        def hook(mod, args, out):
            if c.kv_cache.seqlen > 2048:        # decode steps only
                sets[layer].append(torch.sort(c.topk_dindices_buffer[0].cpu(), dim=-1).values.clone())
                scores[layer].append(c.qk_product[0, :, : c.kv_cache.seqlen].cpu().clone())
        return hook

    for layer in (2, 3):
        m.model.layers[layer].self_attn.register_forward_hook(grab(layer))
    step_logits = []
    with torch.inference_mode():
        logits = m(input_ids=prompt.cuda())
        step_logits.append(logits[0, -1].float().cpu())
        tok = logits.argmax(-1)
        toks = [int(tok)]
        for _ in range(steps - 1):
            logits = m(input_ids=tok.view(1, 1))
            step_logits.append(logits[0, -1].float().cpu())
            tok = logits.argmax(-1)
            toks.append(int(tok))
    assert c.workspace.status() == 0
    assert toks == z["tokens"].tolist()
    want_logits = torch.from_numpy(z["logits"])
    err = (torch.stack(step_logits) - want_logits).abs().max().item()
    assert torch.allclose(torch.stack(step_logits), want_logits, rtol=1e-4, atol=1e-5), f"per-step logits differ by {err:.3e}"
    differing = 0
    for layer, key in ((2, "layer2_sets"), (3, "layer3_sets")):
        ref_sets = torch.from_numpy(z[key])               # [31, 4, 128]
        assert len(sets[layer]) == ref_sets.shape[0]
        for step, (got, want) in enumerate(zip(sets[layer], ref_sets)):
            for h in range(W.heads):
                differing += _set_differences_inside_tie_band(scores[layer][step][h], got[h], want[h], 1e-4)
    assert differing <= 0.01 * 2 * ref_sets.numel(), f"{differing} near-tied indices differ"
    m.tidal_clear()
    assert c.kv_cache.seqlen == 0


@pytest.mark.parametrize("dtype,heads,kv_heads,reduce,force", [
    (torch.bfloat16, 8, 2, "sum", True), (torch.float16, 4, 4, "none", True), (torch.float32, 8, 8, "sum", False)])
def test_llama_decode_matches_oracle_modes(dtype, heads, kv_heads, reduce, force):
    """GQA / 16-bit / head-summed / forced-newest-token modes against the oracle decoder
    fed the same weights: logits of every decode step within tolerance."""
    W = O.TinyLlamaWeights(vocab=512, hidden=heads * 64, layers=4, heads=heads, kv_heads=kv_heads, ffn=344, seed=3,
                           dtype=dtype)
    g = torch.Generator().manual_seed(1)
    P, steps, k = 300, 6, 32
    prompt = torch.randint(0, W.vocab, (1, P), generator=g)
    m = _tiny_model(W, dtype, (2,), reduce, force, 1)
    m.tidal_init(page_size=1, max_seq_len=P + 32, token_budget=k, dtype=dtype, device=torch.device("cuda"))
    with torch.inference_mode():
        toks = m.greedy_generate(prompt.cuda(), steps)
    assert m.model.iController.workspace.status() == 0
    with torch.no_grad():
        want = O.tiny_llama_greedy(W, prompt, steps, k, 2, 99, head_reduce=reduce, force_last=force)
    if dtype == torch.float32:
        assert toks == want
    else:
        # 16-bit logits of a random-init model are nearly flat; demand agreement on most steps
        agree = sum(a == b for a, b in zip(toks, want))
        assert agree >= steps - 2, (toks, want)


def test_batched_decode_equals_single_sequence_runs():
    """A batch decoded in lockstep gives each sequence what it gets alone."""
    from tidaldecode_b200.llama import LlamaConfig, LlamaForCausalLM
    from tidaldecode_b200 import utils as U

    B, Hq, Hkv, D, N, k = 3, 8, 2, 128, 257, 32
    dtype = torch.bfloat16
    c = U.InferenceController(num_layers=1, num_heads=Hq, head_dim=D, page_size=1, token_budget=k, max_seq_len=N + 8,
                              dtype=dtype, device=torch.device("cuda"), num_kv_heads=Hkv, batch_size=B, head_reduce="sum",
                              force_last_token=False)
    q, Kd, Vd = make_qkv(31, B, Hq, Hkv, D, N, dtype, planted=8)
    # fill the cache token by token group: prefill-like append of N-1 tokens per sequence, then one decode token
    c.prepare_metadata(N - 1)
    c.begin_forward(N - 1)
    kk = Kd[:, :, : N - 1].permute(0, 2, 1, 3).reshape(B * (N - 1), Hkv, D).contiguous().cuda()
    vv = Vd[:, :, : N - 1].permute(0, 2, 1, 3).reshape(B * (N - 1), Hkv, D).contiguous().cuda()
    U.append_kv(kk, vv, c, 0)
    c.prepare_metadata(1)
    c.begin_forward(1)
    U.append_kv(Kd[:, :, N - 1].contiguous().cuda(), Vd[:, :, N - 1].contiguous().cuda(), c, 0)
    qd = q[:, :, 0].contiguous().cuda()
    o_sel = U.decode_sparse_attn(qd, c, 0, c.kv_indices_without_last, True)
    U.decode_topk(c)
    o_sp = U.decode_sparse_attn(qd, c, 0, c.topk_dindices_buffer, False)
    assert c.workspace.status() == 0
    allidx = torch.arange(N, dtype=torch.int32)[None].expand(B, N)
    assert_close(o_sel, O.gathered_attention(q, Kd, Vd, allidx)[:, :, 0], dtype, "batched selection layer")
    idx = c.topk_dindices_buffer.cpu()
    ok, why = O.topk_sets_match(O.scores_fp32(q, Kd, "sum"), idx, k, tie_band=1e-4)
    assert ok, why
    assert_close(o_sp, O.gathered_attention(q, Kd, Vd, idx)[:, :, 0], dtype, "batched sparse layer")
    with pytest.raises(RuntimeError):
        c._selection_valid = False
        U.decode_sparse_attn(qd, c, 0, c.topk_dindices_buffer, False)       # modify_llama.py:123-124


@pytest.mark.parametrize("dtype,rows,hidden", [(torch.float16, 1, 4096), (torch.bfloat16, 7, 4096), (torch.float32, 3, 256),
                                               (torch.float16, 2048, 1024), (torch.bfloat16, 2, 8192)])
def test_rms_norm_matches_reference_model(K, dtype, rows, hidden):
    """rms_norm_forward against the reference model's LlamaRMSNorm arithmetic (oracle restatement of
    src/models/llama_tidaldecoding.py:122-127)."""
    g = torch.Generator().manual_seed(hidden + rows)
    x = (torch.randn(1, rows, hidden, generator=g) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    out = torch.empty_like(x, device="cuda")
    K.rms_norm_forward(x.cuda(), w.cuda(), out, 1e-6)
    want = O.rms_norm(x, w, 1e-6)
    if dtype == torch.float32:
        assert torch.allclose(out.cpu(), want, rtol=1e-5, atol=1e-6)
    else:
        ulp = 2 ** -7 if dtype == torch.bfloat16 else 2 ** -10
        assert torch.allclose(out.cpu().float(), want.float(), rtol=2 * ulp, atol=1e-6)
        assert (out.cpu() == want).float().mean() > 0.98
    with pytest.raises(RuntimeError):
        K.rms_norm_forward(x.cuda()[..., :-3].contiguous(), w.cuda()[:-3].contiguous(), out[..., :-3].contiguous(), 1e-6)


@pytest.mark.parametrize("fused_linear", [True, False])
def test_graph_decoder_matches_eager_and_reference(fused_linear):
    """The decode step captured as one CUDA graph (device-side lengths, positions and token feedback)
    produces the reference model's greedy tokens on configuration 1."""
    from tidaldecode_b200.runtime import GraphDecoder

    z = load_golden("tiny_llama_cfg1.npz")
    W = O.TinyLlamaWeights()
    g = torch.Generator().manual_seed(int(z["prompt_seed"]))
    prompt = torch.randint(0, W.vocab, (1, 2048), generator=g)
    m = _tiny_model(W, torch.float32, (2, 3), "none", False, 1)
    m.tidal_init(page_size=1, max_seq_len=2048 + 64, token_budget=128, dtype=torch.float32, device=torch.device("cuda"))
    rt = GraphDecoder(m, max_seq_len=2048 + 64, fused_linear=fused_linear)   # projections in one launch each, or torch ops
    first = rt.prefill(prompt)
    toks = [int(first)] + rt.decode(31).cpu()[0].tolist()
    assert toks == z["tokens"].tolist()
    assert rt.c.workspace.status() == 0
    assert rt.c.kv_cache.seqlen == 2048 + 31
    # the sets of the last step's re-selection layer against the reference's, near-ties excepted
    got = torch.sort(rt.c._topk_indices_full[0, :, :128].cpu(), dim=-1).values
    want = torch.from_numpy(z["layer3_sets"][-1])
    sc = rt.c.qk_product[0, :, : 2048 + 31].cpu()
    for h in range(W.heads):
        _set_differences_inside_tie_band(sc[h], got[h], want[h], 1e-4)
    # a second prompt through the same decoder: graph and buffers are reused
    first = rt.prefill(prompt[:, :700])
    again = [int(first)] + rt.decode(5).cpu()[0].tolist()
    with torch.no_grad():
        want = O.tiny_llama_greedy(W, prompt[:, :700], 6, 128, 2, 3)
    assert again == want


def test_graph_decoder_gqa_head_sum_bf16():
    from tidaldecode_b200.runtime import GraphDecoder

    W = O.TinyLlamaWeights(vocab=512, hidden=512, layers=4, heads=8, kv_heads=2, ffn=344, seed=3, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, W.vocab, (1, 300), generator=g)
    m = _tiny_model(W, torch.bfloat16, (2,), "sum", True, 1)
    rt = GraphDecoder(m, max_seq_len=340, token_budget=32)
    first = rt.prefill(prompt)
    graph_toks = [int(first)] + rt.decode(6).cpu()[0].tolist()
    m2 = _tiny_model(W, torch.bfloat16, (2,), "sum", True, 1)
    m2.tidal_init(page_size=1, max_seq_len=340, token_budget=32, dtype=torch.bfloat16, device=torch.device("cuda"))
    with torch.inference_mode():
        eager_toks = m2.greedy_generate(prompt.cuda(), 7)
    assert graph_toks == eager_toks, (graph_toks, eager_toks)
    assert rt.c.workspace.status() == 0


def test_graph_decoder_batch_from_filled_caches():
    """Sequences decoded in lockstep from caches the caller filled (GraphDecoder.start_from_cache): two
    sequences with the same cache content and first token produce the same tokens as one sequence alone."""
    from tidaldecode_b200.runtime import GraphDecoder

    W = O.TinyLlamaWeights(vocab=512, hidden=512, layers=4, heads=8, kv_heads=2, ffn=352, seed=5, dtype=torch.bfloat16)
    ctx, steps = 200, 6
    outs = []
    ref_pool = None
    for B in (1, 2):
        m = _tiny_model(W, torch.bfloat16, (2,), "sum", True, 1)
        rt = GraphDecoder(m, max_seq_len=ctx + steps + 4, token_budget=32, batch_size=B)
        rt.start_from_cache(ctx, torch.full((B,), 7))
        kv = rt.c.kv_cache
        g = torch.Generator(device="cuda").manual_seed(3)
        for layer in range(kv.pool.num_layers):
            buf = kv.pool.buf[layer]
            t0 = kv.page_table[0, :ctx].long()
            buf[t0] = torch.randn(ctx, *buf.shape[1:], generator=g, device="cuda").to(buf.dtype)
            for b in range(1, B):
                buf[kv.page_table[b, :ctx].long()] = buf[t0]
        toks = rt.decode(steps).cpu()
        assert rt.c.workspace.status() == 0 and int(rt.lin_status.item()) == 0
        outs.append(toks)
    assert torch.equal(outs[1][0], outs[1][1])
    assert torch.equal(outs[1][0], outs[0][0])
