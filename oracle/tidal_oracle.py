"""CPU restatement of TidalDecode's decode-time attention path (torch, CPU only).

TEST INFRASTRUCTURE, NOT PRODUCT.  Only the test-suite, the smoke check and the
benchmark's CPU-baseline leg may import this module; the shipped package never
does.  Every function cites the reference file:line it follows (paths are
relative to the TidalDecode repository root).

Parity pin: `selection_layer(..., head_reduce="none")` and `sparse_layer` are
checked bit-for-bit against the reference's own `llama_tidal_attention_forward`
(src/tidal_build/modify_llama.py:19-148), imported unmodified, by
tests/golden/make_golden.py; the outputs of that import are the committed
fixtures under tests/golden/.  The two modes that the reference has no code for
(`head_reduce="sum"`, `force_last`) differ from the pinned mode by one line
each, marked below.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

# ----------------------------------------------------------------------------
# RoPE
# ----------------------------------------------------------------------------


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq = 1 / theta^(2i/D), i in [0, D/2)  (transformers' "default" rope
    init that src/models/llama_tidaldecoding.py:175-177 looks up)."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype,
                 scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables the way path A builds them
    (src/models/llama_tidaldecoding.py:200-220): fp32 outer product of inv_freq
    and position, halves duplicated, cast to the model dtype.  `scale` is the
    linear position divisor of the kernel path (decode_page.cuh:650-656)."""
    inv_freq = rope_inv_freq(head_dim, theta)
    pos = positions.to(torch.float32) / scale
    freqs = pos[..., None] * inv_freq          # [..., D/2]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """src/models/llama_tidaldecoding.py:248-252."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope_path_a(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin in the model dtype
    (src/models/llama_tidaldecoding.py:255-279)."""
    return (x * cos) + (rotate_half(x) * sin)


def apply_rope_fp32(x: torch.Tensor, positions: torch.Tensor, theta: float, scale: float = 1.0) -> torch.Tensor:
    """Kernel-path RoPE: rotate in fp32, round once to the storage dtype
    (kernels/src/include/cpu_reference.h:36-53; decode_page.cuh:650-669).
    x: [n, H, D]; positions: [n]."""
    D = x.shape[-1]
    idx = torch.arange(D) % (D // 2)
    ang = (positions.to(torch.float32)[:, None] / scale) / torch.pow(
        torch.tensor(theta, dtype=torch.float32), (2 * idx).float() / D)[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    return (xf * cos + rotate_half(xf) * sin).to(x.dtype)


# ----------------------------------------------------------------------------
# Path-A attention (the semantic ground truth)
# ----------------------------------------------------------------------------


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,Hkv,N,D] -> [B,Hkv*n_rep,N,D]  (src/models/llama_tidaldecoding.py:316-325)."""
    if n_rep == 1:
        return x
    b, h, n, d = x.shape
    return x[:, :, None, :, :].expand(b, h, n_rep, n, d).reshape(b, h * n_rep, n, d)


def logits(q: torch.Tensor, K: torch.Tensor) -> torch.Tensor:
    """S = q K^T / sqrt(D) in the tensors' dtype (modify_llama.py:105-107).
    q [B,Hq,1,D]; K [B,Hq,N,D] -> [B,Hq,1,N]."""
    return torch.matmul(q, K.transpose(2, 3)) / math.sqrt(q.shape[-1])


def select_topk(S: torch.Tensor, top_k: int, head_reduce: str = "none",
                force_last: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k over pre-softmax logits (modify_llama.py:112-120).

    Returns (indices, mask): indices [B,R,1,budget] int64 with R = Hq ("none") or
    1 ("sum"); mask = the 0/1 `pos_dict` of shape [B,R,1,N].
    """
    N = S.size(-1)
    budget = min(N, top_k)                                    # :112-113
    if head_reduce == "sum":
        # NOT IN THE REFERENCE: one shared set from scores summed over q heads.
        S = S.float().sum(dim=1, keepdim=True)
    elif head_reduce != "none":
        raise ValueError(head_reduce)
    if force_last:
        # NOT IN PATH A: kernel-path semantics, newest token always kept and
        # budget-1 picked from history (decode_page.cuh:326-341, controller.py:140-147).
        hist = S[..., : N - 1]
        kk = min(budget - 1, N - 1)
        _, idx = torch.topk(hist, k=kk, dim=-1)
        last = torch.full(idx.shape[:-1] + (1,), N - 1, dtype=idx.dtype)
        idx = torch.cat((idx, last), dim=-1)
    else:
        _, idx = torch.topk(S, k=budget, dim=-1)              # :118
    mask = torch.zeros_like(S).scatter_(-1, idx, 1.0)          # :119
    return idx, mask


def softmax_pv(S: torch.Tensor, V: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """fp32 softmax, cast to the model dtype, then P·V (modify_llama.py:130-133)."""
    P = torch.nn.functional.softmax(S, dim=-1, dtype=torch.float32).to(dtype)
    return torch.matmul(P, V)


def selection_layer(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, top_k: int,
                    head_reduce: str = "none", force_last: bool = False):
    """Token-selection layer: full attention plus top-k (modify_llama.py:105-120,130-133).
    q [B,Hq,1,D]; K,V [B,Hkv,N,D].  Returns (o [B,Hq,1,D], idx, mask)."""
    G = q.shape[1] // K.shape[1]
    Kr, Vr = repeat_kv(K, G), repeat_kv(V, G)                 # :82-83
    S = logits(q, Kr)
    idx, mask = select_topk(S, top_k, head_reduce, force_last)
    o = softmax_pv(S, Vr, q.dtype)                            # unmasked: the layer itself sees all tokens
    return o, idx, mask


def sparse_layer(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Sparse layer as the reference computes it: dense logits, masked_fill with
    finfo.min where pos_dict == 0, fp32 softmax, P·V (modify_llama.py:121-133).
    mask [B,Hq or 1,1,N] (a shared set broadcasts over heads)."""
    G = q.shape[1] // K.shape[1]
    Kr, Vr = repeat_kv(K, G), repeat_kv(V, G)
    S = logits(q, Kr)
    S = S.masked_fill(mask.expand_as(S) == 0, torch.finfo(S.dtype).min)   # :125-128
    return softmax_pv(S, Vr, q.dtype)


def causal_prefill(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """Attention of qo_len new rows q [qo_len,Hq,D] over kv_len cached tokens K,V [kv_len,Hkv,D] of one
    sequence, fp32 arithmetic on the stored values: row i sees kv_idx <= kv_len + i - qo_len
    (kernels/src/include/cpu_reference.h:56-160, mask at :127; scale 1/sqrt(D), no rotary here because
    the modules rotate before they append: tidal/models/SearchAttention.py:121-163)."""
    n_q, Hq, D = q.shape
    kv_len, Hkv, _ = K.shape
    G = Hq // Hkv
    qq = q.float().transpose(0, 1)
    kk = K.float().transpose(0, 1).repeat_interleave(G, 0)
    vv = V.float().transpose(0, 1).repeat_interleave(G, 0)
    S = qq @ kk.transpose(1, 2) / math.sqrt(D)
    if causal:
        q_idx = torch.arange(n_q, device=q.device)[:, None]
        kv_idx = torch.arange(kv_len, device=q.device)[None, :]
        S = S.masked_fill(kv_idx > kv_len + q_idx - n_q, float("-inf"))
    return (torch.softmax(S, -1) @ vv).transpose(0, 1).contiguous()


def full_layer(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
    """Layers below sparse_layer_start: plain SDPA (modify_llama.py:84-98)."""
    G = q.shape[1] // K.shape[1]
    return torch.nn.functional.scaled_dot_product_attention(q, repeat_kv(K, G), repeat_kv(V, G))


# ----------------------------------------------------------------------------
# fp32 views used by the GPU parity tests
# ----------------------------------------------------------------------------


def scores_fp32(q: torch.Tensor, K: torch.Tensor, head_reduce: str) -> torch.Tensor:
    """fp32 logits of the stored (already rounded) q,K; [B,Hq,N] or [B,N]."""
    G = q.shape[1] // K.shape[1]
    S = logits(q.float(), repeat_kv(K, G).float())[:, :, 0, :]
    return S.sum(dim=1) if head_reduce == "sum" else S


def gathered_attention(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """Attention over an explicit index list, fp32 throughout — the arithmetic of
    `selected_single_mha` (kernels/src/include/cpu_reference.h:161-292) at
    page_size 1.  idx [B,Hq,k] or [B,k] (shared).  Returns [B,Hq,1,D] fp32."""
    B, Hq, _, D = q.shape
    G = Hq // K.shape[1]
    Kr, Vr = repeat_kv(K, G).float(), repeat_kv(V, G).float()
    if idx.dim() == 2:
        idx = idx[:, None, :].expand(B, Hq, idx.shape[-1])
    gi = idx.long()[..., None].expand(B, Hq, idx.shape[-1], D)
    Kg, Vg = torch.gather(Kr, 2, gi), torch.gather(Vr, 2, gi)
    S = torch.matmul(q.float(), Kg.transpose(2, 3)) / math.sqrt(D)
    return torch.matmul(torch.softmax(S, dim=-1), Vg)


def attention_chunked(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, head_reduce: Optional[str] = None,
                      chunk: int = 32768, return_partials: bool = False):
    """The same fp32 arithmetic as `scores_fp32` + `gathered_attention` over ALL positions, for contexts
    where materialising the G-fold repeated K,V (modify_llama.py:82-83) in fp32 would not fit the host:
    query heads are grouped on their KV head instead of repeating K,V, and the context is walked in
    chunks whose partials are merged by log-sum-exp (`merge_partials`).  q [B,Hq,1,D]; K,V [B,Hkv,N,D].
    Returns (o [B,Hq,D] fp32, scores: None, [B,N] ("sum") or [B,Hq,N] ("none") fp32); with
    return_partials the first item is the un-normalised (m [B,Hq], l [B,Hq], o [B,Hq,D]) of
    `partial_attention` instead (natural-log domain)."""
    B, Hq, _, D = q.shape
    Hkv, N = K.shape[1], K.shape[2]
    G = Hq // Hkv
    qg = q.float().view(B, Hkv, G, D)
    parts, sc = [], []
    for lo in range(0, N, chunk):
        Kc, Vc = K[:, :, lo:lo + chunk].float(), V[:, :, lo:lo + chunk].float()
        S = torch.matmul(qg, Kc.transpose(2, 3)) / math.sqrt(D)          # [B,Hkv,G,n]
        if head_reduce is not None:
            Sh = S.reshape(B, Hq, -1)
            sc.append(Sh.sum(dim=1) if head_reduce == "sum" else Sh)
        m = S.max(dim=-1).values
        p = torch.exp(S - m[..., None])
        parts.append((m.reshape(B, Hq), p.sum(-1).reshape(B, Hq), torch.matmul(p, Vc).reshape(B, Hq, D)))
    scores = torch.cat(sc, dim=-1) if sc else None
    if not parts:
        parts = [(torch.full((B, Hq), -float("inf")), torch.zeros(B, Hq), torch.zeros(B, Hq, D))]
    if return_partials:
        m = torch.stack([p[0] for p in parts]).max(dim=0).values
        wts = [torch.where(torch.isfinite(p[0]), torch.exp(p[0] - m), torch.zeros_like(m)) for p in parts]
        return (m, sum(w * p[1] for w, p in zip(wts, parts)), sum(w[..., None] * p[2] for w, p in zip(wts, parts))), scores
    return merge_partials(parts), scores


def gathered_attention_gqa(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """`gathered_attention` for a list shared by all heads of a sequence (idx [B,k]) without repeating
    K,V: the rows are gathered first, then the query heads of a group share them.  [B,Hq,D] fp32."""
    B, Hq, _, D = q.shape
    Hkv = K.shape[1]
    G = Hq // Hkv
    gi = idx.long()[:, None, :, None].expand(B, Hkv, idx.shape[-1], D)
    Kg, Vg = torch.gather(K, 2, gi).float(), torch.gather(V, 2, gi).float()
    S = torch.matmul(q.float().view(B, Hkv, G, D), Kg.transpose(2, 3)) / math.sqrt(D)
    return torch.matmul(torch.softmax(S, dim=-1), Vg).reshape(B, Hq, D)


def topk_sets_match(scores: torch.Tensor, got_idx: torch.Tensor, k: int, tie_band: float = 1e-4,
                    force_last: bool = False) -> Tuple[bool, str]:
    """Set equality of a row's top-k up to ties: every index whose score is more
    than `tie_band` above the k-th largest score must be present, no index more
    than `tie_band` below it may be present, there are exactly min(k,N) distinct
    in-range indices.  scores [R,N] fp32, got_idx [R,k']."""
    R, N = scores.shape
    budget = min(N, k)
    for r in range(R):
        s = scores[r]
        got = got_idx[r].long()
        if got.numel() != budget:
            return False, f"row {r}: {got.numel()} indices, want {budget}"
        if got.min() < 0 or got.max() >= N:
            return False, f"row {r}: index out of range"
        if torch.unique(got).numel() != budget:
            return False, f"row {r}: duplicate indices"
        if force_last:
            if (got == N - 1).sum() != 1:
                return False, f"row {r}: newest token not forced"
            got = got[got != N - 1]
            s = s[: N - 1]
            kk = budget - 1
        else:
            kk = budget
        if kk == 0:
            continue
        kth = torch.topk(s, kk).values[-1]
        must = torch.nonzero(s > kth + tie_band).flatten()
        present = torch.zeros(s.numel(), dtype=torch.bool)
        present[got] = True
        if not bool(present[must].all()):
            return False, f"row {r}: a score above the k-th by more than the band is missing"
        if bool((s[got] < kth - tie_band).any()):
            return False, f"row {r}: a selected score is below the k-th by more than the band"
    return True, "ok"


# ----------------------------------------------------------------------------
# Paged KV cache (kernel-path layout) and append
# ----------------------------------------------------------------------------


def kv_elem_offset(page: int, kv: int, entry: int, head: int, d: int, page_size: int, H: int, D: int) -> int:
    """NHD element offset inside one layer's pool
    (kernels/include/decode/decode_page.cuh:191-200,223-234)."""
    return (((page * 2 + kv) * page_size + entry) * H + head) * D + d


def append_paged_kv(kv_data: torch.Tensor, indices: Sequence[int], seq_len: int,
                    k_new: torch.Tensor, v_new: torch.Tensor) -> None:
    """Write the last `n` tokens' K,V rows into their page slots
    (kernels/src/include/cpu_reference.h:294-327).  kv_data [pages,2,page,H,D];
    k_new,v_new [n,H,D]; seq_len counts the appended tokens already."""
    page_size = kv_data.shape[2]
    n = k_new.shape[0]
    start = seq_len - n
    for j in range(n):
        t = start + j
        page = indices[t // page_size]
        kv_data[page, 0, t % page_size] = k_new[j]
        kv_data[page, 1, t % page_size] = v_new[j]


def paged_to_dense(kv_data: torch.Tensor, indices: Sequence[int], seq_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gather a sequence's K,V from the pool: returns [1,H,N,D] each."""
    page_size = kv_data.shape[2]
    idx = torch.as_tensor(list(indices), dtype=torch.long)
    pages = kv_data[idx]                                      # [P,2,page,H,D]
    K = pages[:, 0].reshape(-1, *kv_data.shape[3:])[:seq_len]
    V = pages[:, 1].reshape(-1, *kv_data.shape[3:])[:seq_len]
    return K.permute(1, 0, 2)[None], V.permute(1, 0, 2)[None]


def page_key_bounds(K: torch.Tensor, page_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quest's page metadata: element-wise maximum and minimum of the keys of every KV page
    (kernels/include/decode/decode_page.cuh:417-441 folds one key at a time into the same values).
    K [N,H,D] of one sequence -> (max [P,H,D], min [P,H,D]), P = ceil(N / page_size); a partly filled
    last page is bounded over the keys it holds."""
    N = K.shape[0]
    P = (N + page_size - 1) // page_size
    mx = torch.stack([K[p * page_size:min(N, (p + 1) * page_size)].max(dim=0).values for p in range(P)])
    mn = torch.stack([K[p * page_size:min(N, (p + 1) * page_size)].min(dim=0).values for p in range(P)])
    return mx, mn


def estimate_scores(q: torch.Tensor, kmax: torch.Tensor, kmin: torch.Tensor) -> torch.Tensor:
    """Quest's upper bound of q.k per page: sum_d max(q_d * max_d, q_d * min_d) in fp32
    (kernels/src/test/test_max_possible.cu:80-104; kernel kernels/include/decode/decode_attn.cuh:141-172).
    q [Hq,D]; kmax,kmin [P,Hkv,D] -> [Hq,P]."""
    Hq, Hkv = q.shape[0], kmax.shape[1]
    G = Hq // Hkv
    qf = q.float()[:, None, :]                                             # [Hq,1,D]
    mx = kmax.float().permute(1, 0, 2).repeat_interleave(G, 0)             # [Hq,P,D]
    mn = kmin.float().permute(1, 0, 2).repeat_interleave(G, 0)
    return torch.maximum(qf * mx, qf * mn).sum(-1)


# ----------------------------------------------------------------------------
# Sequence-sharded exact merge (no reference counterpart; the chunk merge it
# generalises is decode_attn.cuh:213-232 `sync_state` / `state_t::merge`)
# ----------------------------------------------------------------------------


def partial_attention(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor):
    """Un-normalised partials over one shard, fp32: m [B,Hq], l [B,Hq], o [B,Hq,D]
    with o = sum_j exp(s_j - m) v_j, l = sum_j exp(s_j - m)."""
    G = q.shape[1] // K.shape[1]
    S = logits(q.float(), repeat_kv(K, G).float())[:, :, 0, :]
    if S.shape[-1] == 0:
        B, Hq, D = q.shape[0], q.shape[1], q.shape[-1]
        return torch.full((B, Hq), -float("inf")), torch.zeros(B, Hq), torch.zeros(B, Hq, D)
    m = S.max(dim=-1).values
    p = torch.exp(S - m[..., None])
    return m, p.sum(-1), torch.einsum("bhn,bhnd->bhd", p, repeat_kv(V, G).float())


def merge_partials(parts) -> torch.Tensor:
    """o = sum_r e^{m_r-m*} o_r / sum_r e^{m_r-m*} l_r over shards r."""
    m_all = torch.stack([p[0] for p in parts])
    m_star = m_all.max(dim=0).values
    num, den = 0.0, 0.0
    for m, l, o in parts:
        w = torch.exp(m - m_star)
        w = torch.where(torch.isfinite(m), w, torch.zeros_like(w))
        num = num + w[..., None] * o
        den = den + w * l
    return num / den[..., None]


def merge_candidates(cand_scores: List[torch.Tensor], cand_idx: List[torch.Tensor], k: int) -> torch.Tensor:
    """Global top-k from per-shard top-k candidates: exact because the selection
    score is the raw logit, so the global top-k is a subset of the union of the
    shard-local top-k sets.  cand_scores[r] [R,kr] fp32, cand_idx[r] [R,kr] global."""
    s = torch.cat(cand_scores, dim=-1)
    i = torch.cat(cand_idx, dim=-1)
    kk = min(k, s.shape[-1])
    pick = torch.topk(s, kk, dim=-1).indices
    return torch.gather(i, -1, pick)


# ----------------------------------------------------------------------------
# Tiny Llama-style decoder (config 1 of the benchmark list), path-A arithmetic
# ----------------------------------------------------------------------------


class TinyLlamaWeights:
    """Seeded N(0, std) weights in a fixed order, independent of any model class,
    so the same tensors can be loaded into the reference model and into ours."""

    def __init__(self, vocab=1024, hidden=256, layers=4, heads=4, kv_heads=4, ffn=688, std=0.02,
                 seed=0, dtype=torch.float32):
        g = torch.Generator().manual_seed(seed)
        self.vocab, self.hidden, self.layers, self.heads, self.kv_heads, self.ffn = vocab, hidden, layers, heads, kv_heads, ffn
        self.head_dim = hidden // heads
        self.eps = 1e-6
        self.theta = 10000.0
        self.dtype = dtype

        def n(*shape):
            return (torch.randn(*shape, generator=g) * std).to(dtype)

        self.embed = n(vocab, hidden)
        self.layer = []
        for _ in range(layers):
            self.layer.append(dict(
                q=n(heads * self.head_dim, hidden), k=n(kv_heads * self.head_dim, hidden),
                v=n(kv_heads * self.head_dim, hidden), o=n(hidden, heads * self.head_dim),
                gate=n(ffn, hidden), up=n(ffn, hidden), down=n(hidden, ffn),
                ln1=torch.ones(hidden, dtype=dtype), ln2=torch.ones(hidden, dtype=dtype)))
        self.norm = torch.ones(hidden, dtype=dtype)
        self.lm_head = n(vocab, hidden)

    def hf_state_dict(self):
        """Names as in src/models/llama_tidaldecoding.py (`LlamaForCausalLM`)."""
        sd = {"model.embed_tokens.weight": self.embed, "model.norm.weight": self.norm, "lm_head.weight": self.lm_head}
        for i, L in enumerate(self.layer):
            p = f"model.layers.{i}."
            sd[p + "self_attn.q_proj.weight"] = L["q"]
            sd[p + "self_attn.k_proj.weight"] = L["k"]
            sd[p + "self_attn.v_proj.weight"] = L["v"]
            sd[p + "self_attn.o_proj.weight"] = L["o"]
            sd[p + "mlp.gate_proj.weight"] = L["gate"]
            sd[p + "mlp.up_proj.weight"] = L["up"]
            sd[p + "mlp.down_proj.weight"] = L["down"]
            sd[p + "input_layernorm.weight"] = L["ln1"]
            sd[p + "post_attention_layernorm.weight"] = L["ln2"]
        return sd


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """src/models/llama_tidaldecoding.py:122-127."""
    dt = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return w * (xf * torch.rsqrt(var + eps)).to(dt)


def tiny_llama_greedy(W: TinyLlamaWeights, prompt: torch.Tensor, steps: int, top_k: int,
                      sparse_layer_start: int, correction_layer: int, head_reduce: str = "none",
                      force_last: bool = False, return_trace: bool = False, return_logits: bool = False):
    """Prefill + greedy decode with path-A attention per layer
    (src/models/llama_tidaldecoding.py:914-1019 for the layer loop and pos_dict
    threading; modify_llama.py:19-148 for the attention).  prompt [1,P] int64."""
    F = torch.nn.functional
    B, P = prompt.shape
    H, Hkv, D = W.heads, W.kv_heads, W.head_dim
    Ks = [None] * W.layers
    Vs = [None] * W.layers
    out_tokens, trace, step_logits = [], [], []

    def forward(ids, pos0):
        n = ids.shape[1]
        h = F.embedding(ids, W.embed)
        pos = torch.arange(pos0, pos0 + n)[None]
        cos, sin = rope_cos_sin(pos, D, W.theta, W.dtype)
        cos, sin = cos[:, None], sin[:, None]
        mask = None                                           # pos_dict, reset per forward (:983)
        for i, L in enumerate(W.layer):
            x = rms_norm(h, L["ln1"], W.eps)
            q = F.linear(x, L["q"]).view(B, n, H, D).transpose(1, 2)
            k = F.linear(x, L["k"]).view(B, n, Hkv, D).transpose(1, 2)
            v = F.linear(x, L["v"]).view(B, n, Hkv, D).transpose(1, 2)
            q, k = apply_rope_path_a(q, cos, sin), apply_rope_path_a(k, cos, sin)
            Ks[i] = k if Ks[i] is None else torch.cat((Ks[i], k), dim=2)
            Vs[i] = v if Vs[i] is None else torch.cat((Vs[i], v), dim=2)
            N = Ks[i].shape[2]
            if i < sparse_layer_start or n == N:              # modify_llama.py:84
                G = H // Hkv
                a = F.scaled_dot_product_attention(q, repeat_kv(Ks[i], G), repeat_kv(Vs[i], G),
                                                   is_causal=(n > 1))
            elif i == sparse_layer_start or i == correction_layer:
                a, idx, mask = selection_layer(q, Ks[i], Vs[i], top_k, head_reduce, force_last)
                if return_trace:
                    trace.append((len(out_tokens), i, idx.clone()))
            else:
                a = sparse_layer(q, Ks[i], Vs[i], mask)
            a = a.transpose(1, 2).reshape(B, n, H * D)
            h = h + F.linear(a, L["o"])
            x = rms_norm(h, L["ln2"], W.eps)
            h = h + F.linear(F.silu(F.linear(x, L["gate"])) * F.linear(x, L["up"]), L["down"])
        h = rms_norm(h, W.norm, W.eps)
        return F.linear(h, W.lm_head)[:, -1:]               # logits of every position, as the reference computes them

    logit = forward(prompt, 0)
    step_logits.append(logit[0, -1].clone())
    tok = logit.argmax(-1)
    out_tokens.append(int(tok))
    for s in range(steps - 1):
        logit = forward(tok.view(1, 1), P + s)
        step_logits.append(logit[0, -1].clone())
        tok = logit.argmax(-1)
        out_tokens.append(int(tok))
    res = (out_tokens,) + ((trace,) if return_trace else ()) + ((torch.stack(step_logits),) if return_logits else ())
    return res if len(res) > 1 else out_tokens
