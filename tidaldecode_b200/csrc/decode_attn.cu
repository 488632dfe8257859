// Decode attention over a paged KV pool for sm_100a: one kernel serves full,
// token-selection and sparse layers (tidal_decode_attention), one kernel merges
// the split-KV partials.
//
// Data movement: a producer warp walks the CTA's token list and, per token,
// issues two one-dimensional TMA bulk copies (cp.async.bulk) — the K row and the
// V row of the CTA's KV heads, HC*D*sizeof(T) bytes each, contiguous in the
// [pages][2][page_size][Hkv][D] pool — into a ring of shared-memory stages
// tracked by full/empty mbarriers.  Consumer warps read the rows back with
// 128-bit shared loads, LPR = D*sizeof(T)/16 lanes per row ("slot"), reduce the
// dot product with warp shuffles and keep an online softmax per (slot, q head)
// in the log2 domain.  Every wait is bounded.
//
// Work split: grid = (chunks of the token list, head slices, sequences).  A CTA
// covers HC KV heads (all of them when logits are summed over heads, so the sum
// is formed in shared memory in a fixed order); its slots either own HPS heads
// each (HC = slots*HPS) or share a head among TG token groups (slots = HC*TG).
#include <cstdlib>

#include "attn_params.cuh"

namespace tidal {

__host__ __device__ inline size_t attn_smem_bytes(int S, int T, int row_bytes, int HC, int CW, int slots, int hps,
                                                  int G, int D, bool want_scores) {
    size_t stage = (size_t)S * 2 * T * row_bytes;
    size_t ep = (size_t)slots * hps * G * (D + 2) * sizeof(float) + cta_result_bytes(HC, G, D);
    size_t main_bytes = round16(stage > ep ? stage : ep);
    size_t sc = want_scores ? score_smem_bytes(T, HC) + sizeof(uint32_t) * TIDAL_TOPK_BINS : 0;
    return main_bytes + sc + 2 * S * sizeof(uint64_t) + 64;
}

// Tokens one slot processes per stage (unrolled): fewer under wide GQA groups,
// whose q and accumulator registers leave less room.
__host__ __device__ constexpr int attn_tps(int G) { return G >= 4 ? 2 : 4; }

// T: storage type; D: head dim; G: q heads per KV head handled by one slot;
// HPS: KV heads per slot.
// MPW: most producer warps the instance can be launched with (1 or kMaxProducerWarps); the instances
// with one producer keep the tighter launch bound, which the long streaming layers are tuned for.
template <typename T, int D, int G, int HPS, int MPW>
__global__ void __launch_bounds__(((G >= 4 ? 8 : 16) + MPW) * 32) decode_attn_kernel(const __grid_constant__ AttnParams p) {
    using V = Vec16<T>;
    constexpr int VEC = V::N;
    constexpr int LPR = D / VEC;          // lanes per row
    constexpr int SPW = 32 / LPR;         // slots per warp
    constexpr int TPS = attn_tps(G);      // tokens a slot takes from one stage
    static_assert(LPR <= 32 && (32 % LPR) == 0, "row must fit a warp");

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t src_row[2 * kAddrBlock];  // pool rows of the producers' current and next block of list entries
    const int row_bytes = p.HC * D * (int)sizeof(T);
    const int S = p.S, TT = p.T, TG = p.TG, HC = p.HC;
    const int slots = p.CW * SPW;
    // K rows then V rows, or token-major K|V when both arrive in one copy
    const int pitch = p.kv_fused ? 2 * row_bytes : row_bytes;
    const int v_base = p.kv_fused ? row_bytes : TT * row_bytes;
    const size_t stage_stride = (size_t)2 * TT * row_bytes;
    const size_t stage_bytes = (size_t)S * stage_stride;
    const size_t ep_bytes = (size_t)slots * HPS * G * (D + 2) * sizeof(float);
    const size_t main_bytes = round16(stage_bytes > ep_bytes + cta_result_bytes(p.HC, G, D) ? stage_bytes
                                                                                             : ep_bytes + cta_result_bytes(p.HC, G, D));
    float* cta_o = reinterpret_cast<float*>(smem + ep_bytes);                      // [HC*G][D], then [HC*G][2]
    float* cta_ml = cta_o + (size_t)p.HC * G * D;
    const bool want_scores = p.scores != nullptr;
    const bool sum_heads = want_scores && p.score_rows == 1;
    unsigned char* stage_base = smem;
    float* sc_smem = reinterpret_cast<float*>(smem + main_bytes);                  // [2][R*T][HC]
    const size_t sc_bytes = sum_heads ? score_smem_bytes(TT, HC) + sizeof(uint32_t) * TIDAL_TOPK_BINS : 0;
    uint32_t* sh_hist = reinterpret_cast<uint32_t*>(smem + main_bytes + score_smem_bytes(TT, HC));   // CTA-local digit counts
    const int R = score_block_stages(TT, HC);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + main_bytes + sc_bytes);
    uint64_t* empty_bar = full_bar + S;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + S);

    const int chunk = blockIdx.x, slice = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        TIDAL_STAMP(0);
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], p.CW);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (sum_heads && p.hist)
        for (int i = threadIdx.x; i < TIDAL_TOPK_BINS; i += blockDim.x) sh_hist[i] = 0;
    // the prologue above touched no global memory; from here on this kernel is ordered
    // after the earlier kernels of the stream (see common.cuh)
    // a cluster's CTAs write into each other's shared memory at the end: all of them must be running by then.
    // Arrive now, wait only before the first such store (store_attention_result).
    if (p.cluster > 1) cluster_arrive_relaxed();
    if (threadIdx.x == 0) TIDAL_STAMP(1);
    pdl_wait();
    if (threadIdx.x == 0) TIDAL_STAMP(2);
    pdl_launch_dependents();
    // ---- token list of this CTA
    const int sel_row = p.sel_idx ? (p.sel_rows == 1 ? 0 : slice) : 0;
    int list_len;
    if (p.sel_idx) {
        list_len = p.sel_counts ? p.sel_counts[(size_t)b * p.sel_rows + sel_row] : p.sel_count;
        if (list_len > p.sel_count) list_len = p.sel_count;
        if (list_len < 0) list_len = 0;
    } else {
        list_len = p.seq_lens ? p.seq_lens[b] : p.seq_len;
        if (list_len > p.seq_len) list_len = p.seq_len;
        if (list_len < 0) list_len = 0;
    }
    const int seq_len_b = p.seq_lens ? min(p.seq_lens[b], p.seq_len) : p.seq_len;
    const int ntok_all = list_len + (p.extra_page >= 0 ? 1 : 0);
    // index of the newest token in the score row: its position, or its place in the list
    const int last_index = (p.sel_idx ? ntok_all : seq_len_b) - 1;
    const int ctok = (ntok_all + p.nchunks - 1) / p.nchunks;
    const int tok0 = chunk * ctok;
    const int ntok = max(0, min(ntok_all, tok0 + ctok) - tok0);
    const int n_iters = (ntok + TT - 1) / TT;

    const int kvh0 = p.per_head ? slice / p.greal : slice * HC;   // first KV head of the CTA
    const int qh0 = p.per_head ? slice : kvh0 * G;                // first q head of the CTA

    const TokenList tl{b, sel_row, list_len, seq_len_b, tok0, ntok};
    fill_first_rows(p, tl, src_row);
    __syncthreads();
    if (threadIdx.x == 0) TIDAL_STAMP(3);

    if (warp < p.PW) {
        // ============================================================== producers
        produce_stages<MPW>(p, tl, src_row, warp, lane, S, TT, n_iters, (uint32_t)row_bytes, (uint32_t)pitch, (uint32_t)v_base, stage_stride,
                       (size_t)kvh0 * D * sizeof(T), (size_t)p.Hkv * D * sizeof(T), stage_base, full_bar, empty_bar, abort_flag);
    } else {
    // ================================================================= consumers
    const int cw = warp - p.PW;
    const int slot = cw * SPW + lane / LPR;
    const int sl = lane % LPR;                    // lane within the slot
    const unsigned slot_mask = (LPR == 32) ? 0xffffffffu : (((1u << LPR) - 1u) << ((lane / LPR) * LPR));
    int head_local, tg;                           // first KV head (within the CTA) and token group of this slot
    if (TG == 1) {
        head_local = slot * HPS;
        tg = 0;
    } else {
        head_local = slot % HC;
        tg = slot / HC;
    }
    const bool slot_active = head_local < HC;
    const int consumer_threads = p.CW * 32;
    const int ctid = threadIdx.x - 32 * p.PW;

    float qf[HPS][G][VEC], of[HPS][G][VEC], mrun[HPS][G], lrun[HPS][G];
#pragma unroll
    for (int hh = 0; hh < HPS; ++hh)
#pragma unroll
        for (int g = 0; g < G; ++g) {
            mrun[hh][g] = -INFINITY;
            lrun[hh][g] = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) of[hh][g][i] = 0.f;
            if (slot_active) {
                const int hq = qh0 + (head_local + hh) * G + g;
                const uint4 v = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const T*>(p.q) + ((size_t)b * p.Hq + hq) * D + sl * VEC);
                V::to_float(v, qf[hh][g]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) qf[hh][g][i] = 0.f;
            }
        }
    const float scale_log2 = p.sm_scale * kLog2e;

    for (int it = 0; it < n_iters; ++it) {
        const int s = it % S;
        mbar_wait_bounded(&full_bar[s], (it / S) & 1, abort_flag, p.status);
        if (ctid == 0 && it == 0) TIDAL_STAMP(6);
        const int valid = min(TT, ntok - it * TT);
        const unsigned char* kst = stage_base + (size_t)s * stage_stride;
        const unsigned char* vst = kst + v_base;
        float* sc = sc_smem + ((size_t)((it / R) & 1) * R + (it % R)) * TT * HC;   // this stage's rows of the super-block
        if (slot_active) {
            // The slot's TPS tokens of this stage are processed together: independent dot
            // products and shuffles overlap, and the running softmax is rescaled once.
#pragma unroll
            for (int hh = 0; hh < HPS; ++hh) {
                const size_t hoff = (size_t)(head_local + hh) * D * sizeof(T) + sl * 16;
                float d[TPS][G];
                {
                    float kf[TPS][VEC];
#pragma unroll
                    for (int j = 0; j < TPS; ++j)
                        V::to_float(*reinterpret_cast<const uint4*>(kst + (size_t)(tg + j * TG) * pitch + hoff), kf[j]);
#pragma unroll
                    for (int j = 0; j < TPS; ++j)
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            float acc = 0.f;
#pragma unroll
                            for (int i = 0; i < VEC; ++i) acc = fmaf(qf[hh][g][i], kf[j][i], acc);
                            d[j][g] = acc;
                        }
                }
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1)
#pragma unroll
                    for (int j = 0; j < TPS; ++j)
#pragma unroll
                        for (int g = 0; g < G; ++g) d[j][g] += __shfl_xor_sync(slot_mask, d[j][g], o);
                float vf[TPS][VEC];
#pragma unroll
                for (int j = 0; j < TPS; ++j) {
                    if (tg + j * TG < valid) {
                        V::to_float(*reinterpret_cast<const uint4*>(vst + (size_t)(tg + j * TG) * pitch + hoff), vf[j]);
                    } else {
                        // rows beyond the stage's valid tokens hold stale bytes: their weight is 0, and 0 * NaN is NaN
#pragma unroll
                        for (int i = 0; i < VEC; ++i) vf[j][i] = 0.f;
                    }
                }
                if (want_scores) {
#pragma unroll
                    for (int j = 0; j < TPS; ++j) {
                        const int t = tg + j * TG;
                        if (t >= valid) continue;
                        const int pos = tok0 + it * TT + t;   // position, or index into the list (score column)
                        if (sum_heads) {
                            float ssum = 0.f;
#pragma unroll
                            for (int g = 0; g < G; ++g) ssum += d[j][g] * p.sm_scale;
                            if (sl == 0) sc[t * HC + head_local + hh] = ssum;
                        } else if (sl == 0) {
#pragma unroll
                            for (int g = 0; g < G; ++g) {
                                const float sraw = d[j][g] * p.sm_scale;
                                const int hq = qh0 + (head_local + hh) * G + g;
                                const size_t row = (size_t)b * p.score_rows + hq;
                                p.scores[row * p.score_stride + pos] = sraw;
                                if (p.hist) {
                                    uint32_t bin = ordered_key(sraw) >> kDigit0Shift;
                                    if (p.force_last && pos == last_index) bin = TIDAL_TOPK_BINS - 1;
                                    atomicAdd(&p.hist[row * TIDAL_TOPK_BINS + bin], 1u);
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float s2[TPS];
                    float mnew = mrun[hh][g];
#pragma unroll
                    for (int j = 0; j < TPS; ++j) {
                        s2[j] = (tg + j * TG < valid) ? d[j][g] * scale_log2 : -INFINITY;
                        mnew = fmaxf(mnew, s2[j]);
                    }
                    const float msafe = (mnew == -INFINITY) ? 0.f : mnew;   // nothing seen yet: keep zeros, no NaN
                    const float alpha = fast_exp2(mrun[hh][g] - msafe);
                    float pe[TPS], psum = 0.f;
#pragma unroll
                    for (int j = 0; j < TPS; ++j) {
                        pe[j] = fast_exp2(s2[j] - msafe);
                        psum += pe[j];
                    }
                    mrun[hh][g] = mnew;
                    lrun[hh][g] = fmaf(lrun[hh][g], alpha, psum);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        float acc = of[hh][g][i] * alpha;
#pragma unroll
                        for (int j = 0; j < TPS; ++j) acc = fmaf(pe[j], vf[j][i], acc);
                        of[hh][g][i] = acc;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);          // the stage is free: the logits wait in their own buffer
        if (sum_heads && ((it % R) == R - 1 || it == n_iters - 1)) {
            // head sum in a fixed order for the whole super-block: 8 lanes per token, each adds every 8th
            // head, then a butterfly; one thread per token stores the logit and counts its first radix digit
            named_bar_sync(1, consumer_threads);
            const int sb = it / R;
            const float* blk = sc_smem + (size_t)(sb & 1) * R * TT * HC;
            const int rows = ((it % R) + 1) * TT;
            const int first = sb * R * TT;                  // token index (within the chunk) of row 0
            for (int base = 0; base < rows; base += consumer_threads / 8) {   // uniform per warp
                const int r = base + (ctid >> 3), j = ctid & 7;
                const bool in = r < rows && first + r < ntok;
                float a = 0.f;
                if (in)
                    for (int h = j; h < HC; h += 8) a += blk[r * HC + h];
                a += __shfl_xor_sync(0xffffffffu, a, 4);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                if (j == 0 && in) {
                    const int pos = tok0 + first + r;
                    p.scores[(size_t)b * p.score_stride + pos] = a;
                    if (p.hist) {
                        uint32_t bin = ordered_key(a) >> kDigit0Shift;
                        if (p.force_last && pos == last_index) bin = TIDAL_TOPK_BINS - 1;
                        atomicAdd(&sh_hist[bin], 1u);       // flushed to the row's global histogram once, below
                    }
                }
            }
        }
    }
    if (ctid == 0) TIDAL_STAMP(7);
    if (sum_heads && p.hist) {
        named_bar_sync(1, consumer_threads);
        for (int i = ctid; i < TIDAL_TOPK_BINS; i += consumer_threads)
            if (sh_hist[i]) atomicAdd(&p.hist[(size_t)b * TIDAL_TOPK_BINS + i], sh_hist[i]);
    }

    // ---------------------------------------------------------------- epilogue
    // All stages are drained (every consumer waited on every full barrier), so the
    // stage ring is reused to combine the token groups of each head.
    named_bar_sync(2, consumer_threads);
    float* ep_o = reinterpret_cast<float*>(stage_base);                    // [slots][HPS*G][D]
    float* ep_ml = ep_o + (size_t)slots * HPS * G * D;                     // [slots][HPS*G][2]
#pragma unroll
    for (int hh = 0; hh < HPS; ++hh)
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int e = (slot * HPS + hh) * G + g;
            float4* dst = reinterpret_cast<float4*>(ep_o + (size_t)e * D + sl * VEC);
#pragma unroll
            for (int i = 0; i < VEC / 4; ++i)
                dst[i] = make_float4(of[hh][g][4 * i], of[hh][g][4 * i + 1], of[hh][g][4 * i + 2], of[hh][g][4 * i + 3]);
            if (sl == 0) {
                ep_ml[2 * e] = mrun[hh][g];
                ep_ml[2 * e + 1] = lrun[hh][g];
            }
        }
    named_bar_sync(2, consumer_threads);
    // outputs of the CTA: HC*G q heads x D
    const int nout = HC * G * D;
    for (int idx = ctid; idx < nout; idx += consumer_threads) {
        const int d = idx % D;
        const int hg = idx / D;             // local (kv head, g)
        const int hl = hg / G, g = hg % G;
        // the slots that hold head hl: TG == 1 → slot hl/HPS, sub-head hl%HPS; else slots hl + j*HC
        float M = -INFINITY;
        for (int j = 0; j < TG; ++j) {
            const int e = (TG == 1) ? ((hl / HPS) * HPS + hl % HPS) * G + g : ((hl + j * HC) * HPS) * G + g;
            M = fmaxf(M, ep_ml[2 * e]);
        }
        float acc = 0.f, L = 0.f;
        for (int j = 0; j < TG; ++j) {
            const int e = (TG == 1) ? ((hl / HPS) * HPS + hl % HPS) * G + g : ((hl + j * HC) * HPS) * G + g;
            const float m = ep_ml[2 * e];
            const float w = (m == -INFINITY) ? 0.f : fast_exp2(m - M);
            acc = fmaf(w, ep_o[(size_t)e * D + d], acc);
            L = fmaf(w, ep_ml[2 * e + 1], L);
        }
        cta_o[idx] = acc;
        if (d == 0) {
            cta_ml[2 * hg] = M;
            cta_ml[2 * hg + 1] = L;
        }
    }
    if (ctid == 0) TIDAL_STAMP(8);
    }   // consumers
    store_attention_result<T>(p, cta_o, cta_ml, reinterpret_cast<float*>(smem + p.recv_off), HC, G, D, qh0, b, chunk);
}

// Merge the split-KV partials of one (sequence, q head): grid (Hq, B), 1024 threads as
// kMergeGroups groups of D/4 lanes.  A lane owns four consecutive output elements (float4 loads);
// the groups stride over the chunks, so with up to a few hundred chunks every load of the kernel
// is in flight at once.  Weights, denominator and the cross-group sum use fixed orders.
constexpr int kMergeThreads = 1024;
template <typename T>
__global__ void __launch_bounds__(kMergeThreads) merge_chunks_kernel(const float* __restrict__ part_o,
                                                                     const float* __restrict__ part_ml, int nchunks, int Hq,
                                                                     int D, T* __restrict__ o, float* __restrict__ shard_m,
                                                                     float* __restrict__ shard_l, float* __restrict__ shard_o) {
    extern __shared__ __align__(16) float msm[];     // [nchunks] weights, then [groups][D] partial sums
    __shared__ float s_red[32];
    __shared__ float s_M, s_L;
    pdl_wait();
    pdl_launch_dependents();
    const int hq = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int lanes = D / 4, groups = kMergeThreads / lanes;
    const int lane4 = tid % lanes, grp = tid / lanes;
    const int wlane = tid & 31, warp = tid >> 5;
    float* wgt = msm;
    float* red = msm + ((nchunks + 3) & ~3);
    const size_t ph = (size_t)b * Hq + hq;
    const float* ml = part_ml + ph * nchunks * 2;
    // running maximum over the chunks
    float m_mine = -INFINITY, l_mine = 0.f;
    float2 mlv = make_float2(-INFINITY, 0.f);
    if (tid < nchunks) mlv = *reinterpret_cast<const float2*>(ml + 2 * tid);
    m_mine = mlv.x;
    for (int c = tid + kMergeThreads; c < nchunks; c += kMergeThreads) m_mine = fmaxf(m_mine, ml[2 * c]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m_mine = fmaxf(m_mine, __shfl_xor_sync(0xffffffffu, m_mine, off));
    if (wlane == 0) s_red[warp] = m_mine;
    __syncthreads();
    if (warp == 0) {
        float v = s_red[wlane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
        if (wlane == 0) s_M = v;
    }
    __syncthreads();
    const float M = s_M;
    // weights and denominator
    for (int c = tid; c < nchunks; c += kMergeThreads) {
        const float m = (c == tid) ? mlv.x : ml[2 * c];
        const float l = (c == tid) ? mlv.y : ml[2 * c + 1];
        const float w = (m == -INFINITY) ? 0.f : fast_exp2(m - M);
        wgt[c] = w;
        l_mine = fmaf(w, l, l_mine);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l_mine += __shfl_xor_sync(0xffffffffu, l_mine, off);
    __syncthreads();                 // s_red reuse
    if (wlane == 0) s_red[warp] = l_mine;
    __syncthreads();
    if (warp == 0) {
        float v = s_red[wlane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (wlane == 0) s_L = v;
    }
    // weighted sum of the partial outputs
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* po = part_o + ph * nchunks * D + 4 * lane4;
    if (grp < groups) {
#pragma unroll 8
        for (int c = grp; c < nchunks; c += groups) {
            const float4 v = *reinterpret_cast<const float4*>(po + (size_t)c * D);
            const float w = wgt[c];
            acc.x = fmaf(w, v.x, acc.x);
            acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z);
            acc.w = fmaf(w, v.w, acc.w);
        }
        *reinterpret_cast<float4*>(red + (size_t)grp * D + 4 * lane4) = acc;
    }
    __syncthreads();
    if (tid < D) {
        float tot = 0.f;
        for (int g2 = 0; g2 < groups; ++g2) tot += red[g2 * D + tid];
        const float L = s_L;
        if (o) o[ph * D + tid] = from_f32<T>(L > 0.f ? tot / L : 0.f);
        if (shard_o) {
            shard_o[ph * D + tid] = tot;
            if (tid == 0) {
                shard_m[ph] = M;
                shard_l[ph] = L;
            }
        }
    }
}

// Merge `shards` sets of un-normalised partials laid out [shards][B*Hq(*D)].
template <typename T>
__global__ void merge_shards_kernel(const float* __restrict__ m, const float* __restrict__ l,
                                    const float* __restrict__ o, int shards, int rows, int D, T* __restrict__ out,
                                    int64_t stride_ml, int64_t stride_o) {
    const int r = blockIdx.x, d = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    float M = -INFINITY;
    for (int s = 0; s < shards; ++s) M = fmaxf(M, m[(size_t)s * stride_ml + r]);
    float acc = 0.f, L = 0.f;
    for (int s = 0; s < shards; ++s) {
        const float ms = m[(size_t)s * stride_ml + r];
        const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
        acc = fmaf(w, o[(size_t)s * stride_o + (size_t)r * D + d], acc);
        L = fmaf(w, l[(size_t)s * stride_ml + r], L);
    }
    out[(size_t)r * D + d] = from_f32<T>(L > 0.f ? acc / L : 0.f);
}

// ------------------------------------------------------------------ planning
struct AttnPlan {
    int HC, HPS, TG, CW, T, S, nchunks, nslices;
    size_t smem;
};

constexpr size_t kSmemBudget = 227 * 1024 - 512 - sizeof(uint32_t) * 2 * kAddrBlock;   // per CTA (227 KB is the hardware limit)

// Pick the slot geometry for HC heads per CTA; false if HC cannot be mapped.
static bool plan_slots(int HC, int lpr, bool allow_hps2, int max_cw, int tps, int* CW, int* HPS, int* TG) {
    const int spw = 32 / lpr;
    // more consumer warps hide the shuffle and shared-memory latency of the dot products better
    // than more heads per slot (measured: 16 warps x 1 head beats 8 warps x 2 heads by 16 %)
    const int order[3] = {16, 8, 4};
    for (int cw : order) {
        if (cw > max_cw) continue;
        const int slots = cw * spw;
        if (slots % HC == 0 && (slots / HC) * tps > kAddrBlock) continue;    // a stage must fit a block of looked-up rows
        if (slots % HC == 0) {
            *CW = cw; *HPS = 1; *TG = slots / HC;
            return true;
        }
        if (allow_hps2 && HC == slots * 2) {
            *CW = cw; *HPS = 2; *TG = 1;
            return true;
        }
    }
    return false;
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_plan_chunks(int batch, int head_slices, int tokens, int min_tokens_per_chunk, int sm_count) {
    if (batch <= 0 || head_slices <= 0 || tokens < 0) return TIDAL_ERR_ARG;
    if (sm_count <= 0) sm_count = 148;
    if (min_tokens_per_chunk < 1) min_tokens_per_chunk = 1;
    const int rows = batch * head_slices;
    // one wave of CTAs over the SMs: the shared-memory ring allows one CTA per SM
    int n = sm_count / rows;
    if (n < 1) n = 1;
    const int by_work = (tokens + min_tokens_per_chunk - 1) / min_tokens_per_chunk;
    if (n > by_work) n = by_work < 1 ? 1 : by_work;
    if (n > kMaxChunks) n = kMaxChunks;
    return n;
}

namespace tidal {

// query != nullptr: nothing is launched; *query receives how many clusters of this launch's geometry can be
// resident on the device at once (cudaOccupancyMaxActiveClusters)
template <typename T, int D, int G, int HPS, int MPW>
static int launch_attn_pw(const AttnParams& p, const AttnPlan& plan, cudaStream_t st, int* query) {
    auto kern = decode_attn_kernel<T, D, G, HPS, MPW>;
    dim3 grid(plan.nchunks, plan.nslices, p.B);
    dim3 block((plan.CW + p.PW) * 32);
    if (query) return max_resident_clusters(kern, grid, block, plan.smem, p.cluster, query);
    TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem));
    if (p.cluster > 8) TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    TIDAL_CUDA_OK(launch_pdl(kern, grid, block, plan.smem, st, (unsigned)(p.cluster > 1 ? p.cluster : 1), p));
    count_launch();
    return TIDAL_OK;
}

template <typename T, int D, int G, int HPS>
static int launch_attn(const AttnParams& p, const AttnPlan& plan, cudaStream_t st, int* query) {
    return p.PW == 1 ? launch_attn_pw<T, D, G, HPS, 1>(p, plan, st, query)
                     : launch_attn_pw<T, D, G, HPS, kMaxProducerWarps>(p, plan, st, query);
}

template <typename T, int D>
static int dispatch_g(const AttnParams& p, const AttnPlan& plan, int G, cudaStream_t st, int* query) {
    if (plan.HPS == 2) {
        if (G == 1) return launch_attn<T, D, 1, 2>(p, plan, st, query);
        set_error("two KV heads per slot is only built for MHA (group size 1), got %d", G);
        return TIDAL_ERR_ARG;
    }
    switch (G) {
        case 1: return launch_attn<T, D, 1, 1>(p, plan, st, query);
        case 2: return launch_attn<T, D, 2, 1>(p, plan, st, query);
        case 4: return launch_attn<T, D, 4, 1>(p, plan, st, query);
        case 8: return launch_attn<T, D, 8, 1>(p, plan, st, query);
        default:
            set_error("unsupported GQA group size %d (built: 1, 2, 4, 8)", G);
            return TIDAL_ERR_ARG;
    }
}

template <typename T>
static int dispatch_d(const AttnParams& p, const AttnPlan& plan, int D, int G, cudaStream_t st, int* query) {
    switch (D) {
        case 64: return dispatch_g<T, 64>(p, plan, G, st, query);
        case 128: return dispatch_g<T, 128>(p, plan, G, st, query);
        default:
            set_error("unsupported head_dim %d (built: 64, 128)", D);
            return TIDAL_ERR_ARG;
    }
}

template <typename T>
static int launch_merge(const AttnParams& p, int D, cudaStream_t st) {
    const int groups = kMergeThreads / (D / 4);
    const size_t smem = sizeof(float) * ((size_t)((p.nchunks + 3) & ~3) + (size_t)groups * D);
    TIDAL_CUDA_OK(launch_pdl(merge_chunks_kernel<T>, dim3(p.Hq, p.B), dim3(kMergeThreads), smem, st, 1,
                             (const float*)p.part_o, (const float*)p.part_ml, (int)p.nchunks, (int)p.Hq, D, (T*)p.o, p.shard_m,
                             p.shard_l, p.shard_o));
    count_launch();
    return TIDAL_OK;
}

}  // namespace tidal

extern "C" int tidal_decode_attention(const tidal_attn_args* a, void* d_ws, size_t ws_bytes, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_q && a->d_kv, TIDAL_ERR_ARG, "q and kv must be given");
    TIDAL_REQUIRE(((uintptr_t)a->d_q & 15) == 0 && ((uintptr_t)a->d_kv & 15) == 0 && ((uintptr_t)a->d_o & 15) == 0,
                  TIDAL_ERR_ARG, "q, o and kv must be 16-byte aligned");
    TIDAL_REQUIRE(a->d_o || a->d_part_o, TIDAL_ERR_ARG, "neither o nor partial outputs given");
    TIDAL_REQUIRE((a->d_part_o != nullptr) == (a->d_part_m != nullptr) && (a->d_part_o != nullptr) == (a->d_part_l != nullptr),
                  TIDAL_ERR_ARG, "part_m, part_l, part_o must be given together");
    TIDAL_REQUIRE(a->batch > 0 && a->num_qo_heads > 0 && a->num_kv_heads > 0, TIDAL_ERR_ARG, "bad batch/heads");
    TIDAL_REQUIRE(a->num_qo_heads % a->num_kv_heads == 0, TIDAL_ERR_ARG,
                  "num_qo_heads %d is not a multiple of num_kv_heads %d", a->num_qo_heads, a->num_kv_heads);
    TIDAL_REQUIRE(a->page_size >= 1 && a->num_pages >= 1, TIDAL_ERR_ARG, "bad page_size/num_pages");
    TIDAL_REQUIRE(a->seq_len >= 0, TIDAL_ERR_ARG, "negative seq_len");
    TIDAL_REQUIRE(a->num_pages * 2 * a->page_size < ((int64_t)1 << 32), TIDAL_ERR_ARG,
                  "the pool has more than 2^32 token rows (num_pages * 2 * page_size)");
    TIDAL_REQUIRE(a->dtype >= 0 && a->dtype <= 2, TIDAL_ERR_ARG, "unknown dtype %d", a->dtype);
    const int G = a->num_qo_heads / a->num_kv_heads;
    const int D = a->head_dim;
    const int es = a->dtype == TIDAL_DTYPE_F32 ? 4 : 2;
    TIDAL_REQUIRE(D == 64 || D == 128, TIDAL_ERR_ARG, "unsupported head_dim %d (built: 64, 128)", D);
    const int lpr = D * es / 16;
    const bool sel = a->d_sel_idx != nullptr;
    if (sel) {
        TIDAL_REQUIRE(a->sel_rows == 1 || a->sel_rows == a->num_qo_heads, TIDAL_ERR_ARG,
                      "sel_rows must be 1 or num_qo_heads, got %d", a->sel_rows);
        TIDAL_REQUIRE(a->sel_count >= 0 && a->sel_stride >= a->sel_count, TIDAL_ERR_ARG, "bad sel_count/sel_stride");
        TIDAL_REQUIRE(!a->sel_physical || a->page_size == 1, TIDAL_ERR_ARG, "physical page lists need page_size 1");
        TIDAL_REQUIRE(a->d_scores == nullptr || a->score_rows == a->sel_rows || a->sel_rows == 1, TIDAL_ERR_ARG,
                      "head-summed logits over per-head lists are undefined");
    } else {
        TIDAL_REQUIRE(a->extra_page < 0, TIDAL_ERR_ARG, "extra_page needs a selection list");
        if (!a->d_page_table) {
            // identity mapping: sequence b occupies pages [b * stride, b * stride + pages of seq_len)
            const int64_t need = (int64_t)(a->batch - 1) * a->page_table_stride + (a->seq_len + a->page_size - 1) / a->page_size;
            TIDAL_REQUIRE(a->page_table_stride >= 0 && need <= a->num_pages, TIDAL_ERR_ARG,
                          "identity page mapping needs %lld pages, the pool has %lld", (long long)need, (long long)a->num_pages);
        }
    }
    if (a->d_scores) {
        TIDAL_REQUIRE(a->score_rows == 1 || a->score_rows == a->num_qo_heads, TIDAL_ERR_ARG,
                      "score_rows must be 1 or num_qo_heads, got %d", a->score_rows);
        TIDAL_REQUIRE(a->score_stride >= (sel ? a->sel_count + (a->extra_page >= 0 ? 1 : 0) : a->seq_len), TIDAL_ERR_ARG,
                      "score_stride shorter than the token list");
    } else {
        TIDAL_REQUIRE(a->d_hist == nullptr, TIDAL_ERR_ARG, "a histogram needs d_scores");
    }
    const WsLayout* L = find_ws(d_ws);
    TIDAL_REQUIRE(L != nullptr, TIDAL_ERR_WORKSPACE, "workspace %p was not initialised with tidal_ws_init", d_ws);
    TIDAL_REQUIRE(ws_bytes >= L->total, TIDAL_ERR_WORKSPACE, "workspace is %zu bytes, layout needs %zu", ws_bytes, L->total);

    AttnPlan plan;
    const bool per_head = sel && a->sel_rows != 1 && a->num_qo_heads > 1;
    const bool sum_heads = a->d_scores && a->score_rows == 1;
    int kernel_G = per_head ? 1 : G;
    const int ntok = sel ? a->sel_count + (a->extra_page >= 0 ? 1 : 0) : a->seq_len;

    // Tensor cores where the query group makes q.K^T a tile contraction: 16-bit storage and
    // 2..16 query heads per KV head.  use_tensor_cores: 0 = this rule, 1 = whenever the
    // kernel can run (G = 1 included), -1 = never.
    const bool want_mma = es == 2 && kernel_G <= 16 && a->use_tensor_cores >= 0 && (kernel_G >= 2 || a->use_tensor_cores > 0);
    const int max_cw = kernel_G >= 4 ? 8 : 16;   // the CUDA-core kernel's launch bound
    bool use_mma = false;
    // Geometry for `hc` KV heads per CTA on the chosen kernel; false if that kernel cannot take it.
    auto set_heads = [&](int hc, bool mma) -> bool {
        if (hc < 1 || (!per_head && a->num_kv_heads % hc != 0)) return false;
        if (mma) {
            if (!(hc == 1 || hc == 2 || hc == 4 || hc == 8)) return false;
            plan.CW = kMmaWarps; plan.HPS = 1; plan.TG = kMmaWarps / hc;
            plan.T = kMmaTile * plan.TG;
        } else {
            if (!plan_slots(hc, lpr, kernel_G == 1, max_cw, attn_tps(kernel_G), &plan.CW, &plan.HPS, &plan.TG)) return false;
            plan.T = plan.TG * attn_tps(kernel_G);
        }
        plan.HC = hc;
        plan.nslices = per_head ? a->num_qo_heads : a->num_kv_heads / hc;
        return true;
    };
    int hc0;                                        // preferred KV heads per CTA
    if (per_head) hc0 = 1;
    else if (sum_heads) hc0 = a->num_kv_heads;      // the head sum of the logits is formed inside one CTA
    else if (a->heads_per_cta > 0) hc0 = a->heads_per_cta;
    else hc0 = 0;
    if (want_mma) {
        if (hc0) use_mma = set_heads(hc0, true);
        else
            for (int c : {8, 4, 2, 1})
                if ((use_mma = set_heads(c, true))) break;
    }
    TIDAL_REQUIRE(use_mma || a->use_tensor_cores <= 0, TIDAL_ERR_ARG,
                  "tensor-core attention needs f16/bf16, at most 16 query heads per KV head and 1, 2, 4 or 8 KV heads per CTA");
    if (!use_mma) {
        int hc = hc0 ? hc0 : a->num_kv_heads;
        // rows of 4 KB stream a little faster than rows of 8 KB (measured 88.7 vs 92.8 us at 32 x 128 fp16)
        // — but a gathered list wants the longest rows it can get (fewer copies per byte: 172 vs 218 us for 1 GiB)
        if (!hc0 && !sel && a->num_kv_heads % 2 == 0 && a->num_kv_heads * D * es >= 8192) hc = a->num_kv_heads / 2;
        TIDAL_REQUIRE(per_head || a->num_kv_heads % hc == 0, TIDAL_ERR_ARG, "heads_per_cta %d does not divide num_kv_heads %d", hc,
                      a->num_kv_heads);
        if (!set_heads(hc, false)) {
            // fall back to one KV head per CTA unless the head sum must stay in one CTA
            TIDAL_REQUIRE(!sum_heads, TIDAL_ERR_ARG, "head-summed logits need num_kv_heads in {1,2,4,...,%d} for this head_dim/dtype, got %d",
                          16 * (32 / lpr) * (kernel_G == 1 ? 2 : 1), a->num_kv_heads);
            set_heads(1, false);
        }
    }
    // Short token lists (sparse layers): the whole list is covered by ONE cluster of up to 8 CTAs per
    // (sequence, head slice), which merges through distributed shared memory and writes the result
    // itself — no partials in global memory, no merge launch.  Heads are split over more CTAs until
    // about half the SMs are busy.
    int cluster = 1;
    const size_t list_bytes = (size_t)ntok * 2 * a->num_kv_heads * D * es;
    if (sel && a->num_chunks == 0 && ntok >= 1 && list_bytes <= ((size_t)8 << 20)) {
        // ... unless the CTA takes all KV heads of a token in one copy (tensor-core kernel, page_size 1):
        // splitting the heads would double the copies per byte, which costs more than idle SMs
        // (measured 7.0 vs 8.5 us at 4 sequences x 8 KV heads x 128 tokens).
        const bool one_copy = use_mma && a->page_size == 1 && plan.HC == a->num_kv_heads;
        if (!hc0 && !one_copy) {
            int hc = plan.HC;
            while (hc > 1 && a->batch * plan.nslices * 8 < 64 && set_heads(hc / 2, use_mma)) hc = plan.HC;
        }
        const int per_cta = (int)((64 * 1024) / (2 * (size_t)plan.HC * D * es)) > 0 ? (int)((64 * 1024) / (2 * (size_t)plan.HC * D * es)) : 1;
        cluster = 8;
        while (cluster > 1 && ntok < cluster * per_cta / 2) cluster >>= 1;     // at least half a stage-load per CTA
    }
    const int row_bytes = plan.HC * D * es;
    // a chunk should move at least ~64 KB so that its pipeline fills
    int min_tok = (64 * 1024) / (2 * row_bytes);
    if (min_tok < 1) min_tok = 1;
    const int slots = plan.CW * (32 / lpr);
    const int copy_bytes = ((a->page_size == 1 && plan.HC == a->num_kv_heads && !per_head) ? 2 : 1) * row_bytes;
    cudaStream_t st = (cudaStream_t)stream;
    AttnParams p;
    // Everything that depends on the cluster size; returns a negative code on a bad geometry.
    auto build = [&](int cl, int ns) -> int {
        if (cl > 1) plan.nchunks = cl * ns;
        else plan.nchunks = a->num_chunks > 0 ? a->num_chunks
                                              : tidal_plan_chunks(a->batch, plan.nslices, ntok, min_tok, sm_count_cached());
        TIDAL_REQUIRE(plan.nchunks >= 1 && plan.nchunks <= kMaxChunks, TIDAL_ERR_ARG, "num_chunks %d out of range [1,%d]",
                      plan.nchunks, kMaxChunks);
        // a cluster CTA also holds a receive block for the merge, behind everything else
        const size_t recv_bytes = cl > 1 ? cluster_recv_bytes(plan.HC, kernel_G, D, cl) : 0;
        auto smem_base = [&](int S) {
            return round16(use_mma ? attn_mma_smem_bytes(S, plan.HC, kernel_G, D, sum_heads)
                                   : attn_smem_bytes(S, plan.T, row_bytes, plan.HC, plan.CW, slots, plan.HPS, kernel_G, D, sum_heads));
        };
        auto smem_of = [&](int S) { return smem_base(S) + recv_bytes; };
        int S = 8;
        while (S > 1 && smem_of(S) > kSmemBudget) --S;
        // no more stages than the longest chunk can use (short lists: less shared memory to set up)
        const int iters = ((ntok + plan.nchunks - 1) / plan.nchunks + plan.T - 1) / plan.T;
        if (S > iters) S = iters < 1 ? 1 : iters;
        plan.S = S;
        plan.smem = smem_of(S);
        TIDAL_REQUIRE(plan.smem + sizeof(uint32_t) * 2 * kAddrBlock <= 227 * 1024, TIDAL_ERR_ARG, "shared memory %zu exceeds 227 KB (row %d bytes)", plan.smem, row_bytes);

        p.q = a->d_q; p.o = a->d_o; p.kv = (const char*)a->d_kv;
        p.page_table = a->d_page_table; p.pt_stride = a->page_table_stride;
        p.seq_lens = a->d_seq_lens; p.seq_len = a->seq_len;
        p.sel_idx = a->d_sel_idx; p.sel_counts = a->d_sel_counts;
        p.sel_rows = sel ? a->sel_rows : 1; p.sel_count = a->sel_count; p.sel_physical = a->sel_physical;
        p.extra_page = sel ? a->extra_page : -1; p.sel_stride = a->sel_stride;
        p.scores = a->d_scores; p.score_rows = a->score_rows; p.score_stride = a->score_stride;
        p.hist = a->d_hist; p.force_last = a->force_last;
        p.part_o = (float*)((char*)d_ws + L->part_o_off);
        p.part_ml = (float*)((char*)d_ws + L->part_ml_off);
        p.shard_m = a->d_part_m; p.shard_l = a->d_part_l; p.shard_o = a->d_part_o;
        p.status = (uint32_t*)((char*)d_ws + L->status_off);
        p.B = a->batch; p.Hq = a->num_qo_heads; p.Hkv = a->num_kv_heads; p.page_size = a->page_size;
        p.num_pages = a->num_pages;
        p.sm_scale = a->sm_scale > 0.f ? a->sm_scale : 1.0f / sqrtf((float)D);
        p.nchunks = plan.nchunks; p.HC = plan.HC; p.greal = G; p.per_head = per_head ? 1 : 0;
        p.T = plan.T; p.S = plan.S; p.TG = plan.TG; p.CW = plan.CW; p.cluster = cl;
        p.nsuper = cl > 1 ? ns : 1;
        p.xc_count = (uint32_t*)((char*)d_ws + L->xc_off);
        p.recv_off = (uint32_t)smem_base(plan.S);
        p.kv_fused = (a->page_size == 1 && plan.HC == a->num_kv_heads && !per_head) ? 1 : 0;
        // One warp gets a bulk copy accepted every ~70 cycles, so short rows want more producer warps.
        // On the CUDA-core kernel that is a second instance of the kernel: with rows of 1 KB and more the
        // single-producer instance is kept, because a step that alternates between two instances pays more
        // in cold instruction fetches than the extra producers gain (measured: 119.8 vs 121.5 us per step of
        // a selection and a sparse layer at 32 x 128 heads).
        if (use_mma) p.PW = copy_bytes <= 2048 ? kMmaMaxProducers : 1;
        else p.PW = copy_bytes <= 512 ? kMaxProducerWarps : 1;
        return TIDAL_OK;
    };
    // query != nullptr: do not launch, report how many clusters of this geometry the device holds at once
    auto run = [&](int* query) -> int {
        if (use_mma) return launch_attn_mma(p, D, a->dtype, dim3(plan.nchunks, plan.nslices, p.B), plan.smem, st, query);
        switch (a->dtype) {
            case TIDAL_DTYPE_F16: return dispatch_d<__half>(p, plan, D, kernel_G, st, query);
            case TIDAL_DTYPE_BF16: return dispatch_d<__nv_bfloat16>(p, plan, D, kernel_G, st, query);
            default: return dispatch_d<float>(p, plan, D, kernel_G, st, query);
        }
    };
    int rc;
    // Long lists on a cluster of 8 leave each CTA more than an SM takes in quickly (~40 B/cycle): with 16 CTAs
    // per cluster (the non-portable size) twice as many SMs pull data — if the device can hold all clusters at
    // once (a cluster sits inside one GPC), otherwise they would run one after the other.
    const size_t cta_bytes_at_8 = (size_t)ntok * 2 * plan.HC * D * es / 8;      // what one CTA of an 8-cluster streams
    if (cluster == 8 && cta_bytes_at_8 > ((size_t)192 << 10) && 16 * a->batch * plan.nslices <= sm_count_cached()) {
        if ((rc = build(16, 1)) != TIDAL_OK) return rc;
        int resident = 0;
        if ((rc = run(&resident)) != TIDAL_OK) return rc;
        if (resident >= a->batch * plan.nslices) cluster = 16;
    }
    // Otherwise several clusters per list (two of 8, else four of 4), as long as all of them are resident at once:
    // each cluster merges inside itself as before and leaves its share in the workspace, the last to arrive finishes.
    int nsuper = 1;
    // Not with per-row counts in device memory: the lists may be much shorter than their width (a rank's share of a
    // sharded selection), and the second merge would cost more than it gains (7.9 -> 11.1 us at an eighth of cfg5).
    if (cluster == 8 && cta_bytes_at_8 > ((size_t)192 << 10) && a->d_sel_counts == nullptr) {
        const int tries[2][2] = {{8, 2}, {4, 4}};
        for (int t = 0; t < 2 && nsuper == 1; ++t) {
            const int cl = tries[t][0], ns = tries[t][1];
            if (cl * ns * a->batch * plan.nslices > sm_count_cached()) continue;
            if ((rc = build(cl, ns)) != TIDAL_OK) return rc;
            int resident = 0;
            if ((rc = run(&resident)) != TIDAL_OK) return rc;
            if (resident >= ns * a->batch * plan.nslices) {
                cluster = cl;
                nsuper = ns;
            }
        }
    }
    if ((rc = build(cluster, nsuper)) != TIDAL_OK) return rc;
    const int part_chunks = cluster > 1 ? nsuper : plan.nchunks;      // partials that go through the workspace
    const size_t part_need = sizeof(float) * (size_t)a->batch * a->num_qo_heads * part_chunks * D;
    const size_t ml_need = sizeof(float) * (size_t)a->batch * a->num_qo_heads * part_chunks * 2;
    TIDAL_REQUIRE(part_chunks == 1 ||
                      (L->part_o_off + part_need <= L->part_ml_off && L->part_ml_off + ml_need <= L->hist_off),
                  TIDAL_ERR_WORKSPACE, "workspace was sized for a smaller batch/heads/head_dim than this call");

    // TIDAL_DEBUG_PLAN=1 in the environment: one line per call on stderr with the planner's choices
    static const bool debug_plan = std::getenv("TIDAL_DEBUG_PLAN") != nullptr;
    if (debug_plan)
        fprintf(stderr, "tidal plan: %s ntok %d B %d Hq %d Hkv %d | HC %d slices %d chunks %d cluster %d x %d T %d S %d CW %d PW %d smem %zu fused %d\n",
                use_mma ? "mma" : "cuda-core", ntok, a->batch, a->num_qo_heads, a->num_kv_heads, plan.HC, plan.nslices, plan.nchunks,
                cluster, nsuper, plan.T, plan.S, plan.CW, p.PW, plan.smem, p.kv_fused);
    rc = run(nullptr);
    if (rc != TIDAL_OK) return rc;
    if (plan.nchunks > 1 && cluster == 1) {
        switch (a->dtype) {
            case TIDAL_DTYPE_F16: rc = launch_merge<__half>(p, D, st); break;
            case TIDAL_DTYPE_BF16: rc = launch_merge<__nv_bfloat16>(p, D, st); break;
            default: rc = launch_merge<float>(p, D, st); break;
        }
    }
    return rc;
}

extern "C" int tidal_merge_partials_strided(const float* d_m, const float* d_l, const float* d_o, int64_t shard_stride,
                                            int shards, int batch, int num_qo_heads, int head_dim, void* d_out, int dtype,
                                            void* stream) {
    TIDAL_REQUIRE(d_m && d_l && d_o && d_out, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(shards >= 1 && batch >= 1 && num_qo_heads >= 1, TIDAL_ERR_ARG, "bad shards/batch/heads");
    TIDAL_REQUIRE(head_dim >= 1 && head_dim <= 1024, TIDAL_ERR_ARG, "bad head_dim %d", head_dim);
    const int rows = batch * num_qo_heads;
    const int64_t sml = shard_stride > 0 ? shard_stride : rows;
    const int64_t so = shard_stride > 0 ? shard_stride : (int64_t)rows * head_dim;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    switch (dtype) {
        case TIDAL_DTYPE_F16: e = launch_pdl(merge_shards_kernel<__half>, dim3(rows), dim3(head_dim), 0, st, 1, d_m, d_l, d_o, shards, rows, head_dim, (__half*)d_out, sml, so); break;
        case TIDAL_DTYPE_BF16: e = launch_pdl(merge_shards_kernel<__nv_bfloat16>, dim3(rows), dim3(head_dim), 0, st, 1, d_m, d_l, d_o, shards, rows, head_dim, (__nv_bfloat16*)d_out, sml, so); break;
        case TIDAL_DTYPE_F32: e = launch_pdl(merge_shards_kernel<float>, dim3(rows), dim3(head_dim), 0, st, 1, d_m, d_l, d_o, shards, rows, head_dim, (float*)d_out, sml, so); break;
        default: set_error("unknown dtype %d", dtype); return TIDAL_ERR_ARG;
    }
    TIDAL_CUDA_OK(e);
    count_launch();
    return TIDAL_OK;
}

extern "C" int tidal_merge_partials(const float* d_m, const float* d_l, const float* d_o, int shards, int batch,
                                    int num_qo_heads, int head_dim, void* d_out, int dtype, void* stream) {
    return tidal_merge_partials_strided(d_m, d_l, d_o, 0, shards, batch, num_qo_heads, head_dim, d_out, dtype, stream);
}

TIDAL_TRACE_READER(tidal_trace_read_cc)
