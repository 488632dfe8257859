// Tensor-core variant of the decode-attention kernel for grouped-query heads
// (16-bit K/V, up to 16 query heads per KV head).
//
// With G query heads sharing one KV head, q·K^T for a tile of tokens is a real
// [G x D] x [D x tokens] contraction: the G query rows are the M dimension of
// mma.sync.m16n8k16 (padded to 16), the tokens the N dimension.  The CUDA-core
// kernel spends G FMAs per loaded K/V element and becomes issue-bound from G = 4
// on (measured: 30 % of HBM peak at G = 4); here one warp per KV head issues about
// 11 instructions per token and the kernel stays memory-bound.  tcgen05/TMEM is
// not used: its smallest tile has 64 rows per CTA, G rows cannot fill it, and rows
// of different sequences cannot share a K tile.
//
// Data movement is the same as in the CUDA-core kernel (producer warp, per-token
// cp.async.bulk of the K row and the V row into an mbarrier-tracked ring), except
// that token rows are laid down with a 16-byte pad so that ldmatrix reads of eight
// consecutive tokens fall into distinct bank groups.
//
//   S = Q K^T   A = Q fragments (registers), B = K rows via ldmatrix
//   online softmax on the accumulator fragments (rows = query heads)
//   O += P V    A = P repacked from the S fragments, B = V rows via ldmatrix.trans
#include "attn_params.cuh"

namespace tidal {

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <typename T>
struct Mma16;
template <>
struct Mma16<__half> {
    __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <>
struct Mma16<__nv_bfloat16> {
    __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

__host__ __device__ inline int mma_pitch(int HC, int D) { return HC * D * 2 + 16; }

size_t attn_mma_smem_bytes(int S, int HC, int G, int D, bool sum_heads) {
    const int T = kMmaTile * (kMmaWarps / HC);
    const size_t stage = (size_t)S * 2 * T * mma_pitch(HC, D);
    const size_t ep = (size_t)kMmaWarps * 16 * (D + 2) * sizeof(float) + cta_result_bytes(HC, G, D);
    const size_t main_bytes = round16(stage > ep ? stage : ep);
    const size_t sc = sum_heads ? score_smem_bytes(T, HC) + sizeof(uint32_t) * TIDAL_TOPK_BINS : 0;
    return main_bytes + sc + (2 * S + 4) * sizeof(uint64_t) + 64;
}

template <typename T, int D>
__global__ void __launch_bounds__((kMmaWarps + 1 + kMmaMaxProducers) * 32) decode_attn_mma_kernel(const __grid_constant__ AttnParams p) {
    constexpr int KS = D / 16;    // k-steps of Q K^T
    constexpr int NT = D / 8;     // n-tiles of P V
    using M = Mma16<T>;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t src_row[2 * kAddrBlock];  // pool rows of the producers' current and next block of list entries
    const int HC = p.HC, S = p.S, TG = kMmaWarps / HC, TT = kMmaTile * TG;
    const int row_bytes = HC * D * 2;
    // token rows carry a 16-byte pad; K rows then V rows, or token-major K|V when both arrive in one copy
    const int pitch = p.kv_fused ? 2 * row_bytes + 16 : mma_pitch(HC, D);
    const int v_base = p.kv_fused ? row_bytes : TT * pitch;
    const size_t stage_stride = (size_t)2 * TT * mma_pitch(HC, D);
    const size_t stage_bytes = (size_t)S * stage_stride;
    const int G = p.per_head ? 1 : p.greal;
    const size_t ep_bytes = (size_t)kMmaWarps * 16 * (D + 2) * sizeof(float);
    const size_t main_bytes = round16(stage_bytes > ep_bytes + cta_result_bytes(HC, G, D) ? stage_bytes
                                                                                           : ep_bytes + cta_result_bytes(HC, G, D));
    float* cta_o = reinterpret_cast<float*>(smem + ep_bytes);                          // [HC*G][D], then [HC*G][2]
    float* cta_ml = cta_o + (size_t)HC * G * D;
    const bool want_scores = p.scores != nullptr;
    const bool sum_heads = want_scores && p.score_rows == 1;
    unsigned char* stage_base = smem;
    float* sc_smem = reinterpret_cast<float*>(smem + main_bytes);                      // [2][R*TT][HC]
    const size_t sc_bytes = sum_heads ? score_smem_bytes(TT, HC) + sizeof(uint32_t) * TIDAL_TOPK_BINS : 0;
    uint32_t* sh_hist = reinterpret_cast<uint32_t*>(smem + main_bytes + score_smem_bytes(TT, HC));   // CTA-local digit counts
    const int R = score_block_stages(TT, HC);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + main_bytes + sc_bytes);
    uint64_t* empty_bar = full_bar + S;
    uint64_t* sc_full = empty_bar + S;        // [2] consumers -> reducer: a super-block of logits is parked
    uint64_t* sc_empty = sc_full + 2;         // [2] reducer -> consumers: the buffer may be overwritten
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sc_empty + 2);

    const int chunk = blockIdx.x, slice = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        TIDAL_STAMP(0);
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kMmaWarps);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sc_full[i], kMmaWarps);
            mbar_init(&sc_empty[i], 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Rows of a stage that no copy fills (a short last stage) still enter the P V product
    // with weight zero; zero * stale NaN would poison the accumulator, so the ring starts
    // out as zeros (later contents are real K/V rows, finite whenever the cache is).
    for (size_t i = (size_t)threadIdx.x * 16; i < stage_bytes; i += (size_t)blockDim.x * 16)
        *reinterpret_cast<uint4*>(stage_base + i) = make_uint4(0, 0, 0, 0);
    if (sum_heads && p.hist)
        for (int i = threadIdx.x; i < TIDAL_TOPK_BINS; i += blockDim.x) sh_hist[i] = 0;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // the prologue above touched no global memory; from here on this kernel is ordered
    // after the earlier kernels of the stream (see common.cuh)
    // a cluster's CTAs write into each other's shared memory at the end: all of them must be running by then.
    // Arrive now, wait only before the first such store (store_attention_result).
    if (p.cluster > 1) cluster_arrive_relaxed();
    if (threadIdx.x == 0) TIDAL_STAMP(1);
    pdl_wait();
    if (threadIdx.x == 0) TIDAL_STAMP(2);
    pdl_launch_dependents();
    // ---- token list of this CTA (same rules as the CUDA-core kernel)
    const int sel_row = p.sel_idx ? (p.sel_rows == 1 ? 0 : slice) : 0;
    int list_len;
    if (p.sel_idx) {
        list_len = p.sel_counts ? p.sel_counts[(size_t)b * p.sel_rows + sel_row] : p.sel_count;
        list_len = max(0, min(list_len, p.sel_count));
    } else {
        list_len = p.seq_lens ? p.seq_lens[b] : p.seq_len;
        list_len = max(0, min(list_len, p.seq_len));
    }
    const int seq_len_b = p.seq_lens ? min(p.seq_lens[b], p.seq_len) : p.seq_len;
    const int ntok_all = list_len + (p.extra_page >= 0 ? 1 : 0);
    const int last_index = (p.sel_idx ? ntok_all : seq_len_b) - 1;
    const int ctok = (ntok_all + p.nchunks - 1) / p.nchunks;
    const int tok0 = chunk * ctok;
    const int ntok = max(0, min(ntok_all, tok0 + ctok) - tok0);
    const int n_iters = (ntok + TT - 1) / TT;
    const int kvh0 = p.per_head ? slice / p.greal : slice * HC;
    const int qh0 = p.per_head ? slice : kvh0 * G;

    const TokenList tl{b, sel_row, list_len, seq_len_b, tok0, ntok};
    fill_first_rows(p, tl, src_row);
    __syncthreads();
    if (threadIdx.x == 0) TIDAL_STAMP(3);

    if (warp < p.PW) {
        // ============================================================== producers
        produce_stages<kMmaMaxProducers>(p, tl, src_row, warp, lane, S, TT, n_iters, (uint32_t)row_bytes, (uint32_t)pitch, (uint32_t)v_base, stage_stride,
                       (size_t)kvh0 * D * 2, (size_t)p.Hkv * D * 2, stage_base, full_bar, empty_bar, abort_flag);
    } else if (warp == p.PW) {
        // ================================================================== reducer
        // Sums the logits of each token over the CTA's heads (fixed order), stores them, counts their
        // first radix digit — one super-block of R stages at a time, while the consumers stream on.
        if (sum_heads) {
            const int n_sb = (n_iters + R - 1) / R;
            for (int sb = 0; sb < n_sb; ++sb) {
                const int buf = sb & 1;
                mbar_wait_bounded(&sc_full[buf], (sb >> 1) & 1, abort_flag, p.status);
                const float* blk = sc_smem + (size_t)buf * R * TT * HC;
                const int first = sb * R * TT;                       // token index (within the chunk) of row 0
                const int rows = min(R * TT, ntok - first);
                for (int r = lane; r < rows; r += 32) {
                    float a = 0.f;
                    for (int h = 0; h < HC; ++h) a += blk[r * HC + h];
                    const int pos = tok0 + first + r;
                    p.scores[(size_t)b * p.score_stride + pos] = a;
                    if (p.hist) {
                        uint32_t bin = ordered_key(a) >> kDigit0Shift;
                        if (p.force_last && pos == last_index) bin = TIDAL_TOPK_BINS - 1;
                        atomicAdd(&sh_hist[bin], 1u);               // flushed to the row's global histogram once, below
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sc_empty[buf]);
            }
        }
    } else {
    // ================================================================= consumers
    const int cw = warp - p.PW - 1;
    const int head_local = cw % HC, tg = cw / HC;
    const int consumer_threads = kMmaWarps * 32;
    const int ctid = threadIdx.x - 32 * (p.PW + 1);
    const int r0 = lane >> 2;            // fragment row (query head within the group); the second row is r0 + 8
    const int cq = (lane & 3) * 2;       // fragment column pair

    // Q fragments: rows = query heads of this KV head (zero beyond G)
    uint32_t qa[KS][4];
    {
        const T* qb = reinterpret_cast<const T*>(p.q) + ((size_t)b * p.Hq + qh0 + (size_t)head_local * G) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = r0 + (i & 1) * 8;
                const int col = ks * 16 + cq + (i >> 1) * 8;
                qa[ks][i] = (row < G) ? *reinterpret_cast<const uint32_t*>(qb + (size_t)row * D + col) : 0u;
            }
        }
    }
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[nt][i] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const float scale_log2 = p.sm_scale * kLog2e;
    const uint32_t head_off = (uint32_t)head_local * D * 2;

    for (int it = 0; it < n_iters; ++it) {
        const int s = it % S;
        mbar_wait_bounded(&full_bar[s], (it / S) & 1, abort_flag, p.status);
        if (ctid == 0 && it == 0) TIDAL_STAMP(6);
        if (sum_heads && (it % R) == 0 && it >= 2 * R)               // the reducer is done with this buffer's previous use
            mbar_wait_bounded(&sc_empty[(it / R) & 1], ((it / R) / 2 - 1) & 1, abort_flag, p.status);
        const int valid = min(TT, ntok - it * TT);
        const int tbase = tg * kMmaTile;
        const int mine = min(kMmaTile, valid - tbase);          // valid tokens of this warp's tile (may be <= 0)
        const uint32_t kst = smem_u32(stage_base + (size_t)s * stage_stride);
        const uint32_t vst = kst + (uint32_t)v_base;
        float* sc = sc_smem + ((size_t)((it / R) & 1) * R + (it % R)) * TT * HC;   // this stage's rows of the super-block
        if (mine > 0) {
            // ---- S = Q K^T for 16 tokens: two n-tiles of 8
            float sf[2][4];
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) {
#pragma unroll
                for (int i = 0; i < 4; ++i) sf[n2][i] = 0.f;
                const uint32_t rowaddr = kst + (uint32_t)((tbase + n2 * 8 + (lane & 7)) * pitch) + head_off + (uint32_t)((lane >> 3) * 16);
#pragma unroll
                for (int kp = 0; kp < KS / 2; ++kp) {
                    uint32_t bk[4];
                    ldsm_x4(bk, rowaddr + kp * 64);
                    M::mma(sf[n2], qa[2 * kp], bk[0], bk[1]);
                    M::mma(sf[n2], qa[2 * kp + 1], bk[2], bk[3]);
                }
            }
            // ---- logits out
            if (want_scores) {
                if (sum_heads) {
                    // sum over the group's query heads: rows live in lanes with equal (lane & 3)
                    float v[4];
#pragma unroll
                    for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            v[n2 * 2 + e] = ((r0 < G) ? sf[n2][e] : 0.f) + ((r0 + 8 < G) ? sf[n2][2 + e] : 0.f);
#pragma unroll
                    for (int off = 4; off < 32; off <<= 1)
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
                    if (lane < 4) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int tt = (i >> 1) * 8 + cq + (i & 1);
                            if (tt < mine) sc[(tbase + tt) * HC + head_local] = v[i] * p.sm_scale;
                        }
                    }
                } else {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int row = r0 + half * 8;
                        if (row < G) {
                            const int hq = qh0 + head_local * G + row;
                            const size_t srow = ((size_t)b * p.score_rows + hq);
#pragma unroll
                            for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int tt = n2 * 8 + cq + e;
                                    if (tt < mine) {
                                        const int pos = tok0 + it * TT + tbase + tt;
                                        const float sraw = sf[n2][half * 2 + e] * p.sm_scale;
                                        p.scores[srow * p.score_stride + pos] = sraw;
                                        if (p.hist) {
                                            uint32_t bin = ordered_key(sraw) >> kDigit0Shift;
                                            if (p.force_last && pos == last_index) bin = TIDAL_TOPK_BINS - 1;
                                            atomicAdd(&p.hist[srow * TIDAL_TOPK_BINS + bin], 1u);
                                        }
                                    }
                                }
                        }
                    }
                }
            }
            // ---- online softmax per row
            uint32_t pa[4];
            float alpha[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float x[4];
                float mx = -INFINITY;
#pragma unroll
                for (int n2 = 0; n2 < 2; ++n2)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tt = n2 * 8 + cq + e;
                        const float xv = (tt < mine) ? sf[n2][half * 2 + e] * scale_log2 : -INFINITY;
                        x[n2 * 2 + e] = xv;
                        mx = fmaxf(mx, xv);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float mnew = fmaxf(mrow[half], mx);
                const float msafe = (mnew == -INFINITY) ? 0.f : mnew;
                alpha[half] = fast_exp2(mrow[half] - msafe);
                float ps = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    x[i] = fast_exp2(x[i] - msafe);
                    ps += x[i];
                }
                mrow[half] = mnew;
                lrow[half] = fmaf(lrow[half], alpha[half], ps);      // per-thread part; the quad is summed at the end
                pa[half] = M::pack(x[0], x[1]);                      // tokens cq, cq+1
                pa[2 + half] = M::pack(x[2], x[3]);                  // tokens 8+cq, 8+cq+1
            }
            // ---- rescale the accumulator only when some row's maximum moved
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    o[nt][0] *= alpha[0];
                    o[nt][1] *= alpha[0];
                    o[nt][2] *= alpha[1];
                    o[nt][3] *= alpha[1];
                }
            }
            // ---- O += P V
            const uint32_t vrow = vst + (uint32_t)((tbase + ((lane >> 3) & 1) * 8 + (lane & 7)) * pitch) + head_off + (uint32_t)((lane >> 4) * 16);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t bv[4];
                ldsm_x4_trans(bv, vrow + np * 32);
                M::mma(o[2 * np], pa, bv[0], bv[1]);
                M::mma(o[2 * np + 1], pa, bv[2], bv[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);          // the stage is free: the logits wait in their own buffer
        if (sum_heads && ((it % R) == R - 1 || it == n_iters - 1)) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&sc_full[(it / R) & 1]);     // this warp's logits of the super-block are parked
        }
    }

    // ---------------------------------------------------------------- epilogue
    if (ctid == 0) TIDAL_STAMP(7);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        lrow[half] += __shfl_xor_sync(0xffffffffu, lrow[half], 1);
        lrow[half] += __shfl_xor_sync(0xffffffffu, lrow[half], 2);
    }
    named_bar_sync(2, consumer_threads);                 // every consumer is done with the stage ring
    if (TG == 1) {
        // one warp per KV head: its rows are the CTA's result as they are
        const int hg0 = head_local * G;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = r0 + half * 8;
            if (row < G) {
                float* dst = cta_o + (size_t)(hg0 + row) * D + cq;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
                if ((lane & 3) == 0) {
                    cta_ml[2 * (hg0 + row)] = mrow[half];
                    cta_ml[2 * (hg0 + row) + 1] = lrow[half];
                }
            }
        }
    } else {
        // TG warps hold parts of each head: park the fragments, then one warp per (head, query) row merges them
        float* ep_o = reinterpret_cast<float*>(stage_base);                 // [warps][16][D]
        float* ep_ml = ep_o + (size_t)kMmaWarps * 16 * D;                   // [warps][16][2]
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            *reinterpret_cast<float2*>(ep_o + ((size_t)cw * 16 + r0) * D + nt * 8 + cq) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(ep_o + ((size_t)cw * 16 + r0 + 8) * D + nt * 8 + cq) = make_float2(o[nt][2], o[nt][3]);
        }
        if ((lane & 3) == 0) {
            ep_ml[((size_t)cw * 16 + r0) * 2] = mrow[0];
            ep_ml[((size_t)cw * 16 + r0) * 2 + 1] = lrow[0];
            ep_ml[((size_t)cw * 16 + r0 + 8) * 2] = mrow[1];
            ep_ml[((size_t)cw * 16 + r0 + 8) * 2 + 1] = lrow[1];
        }
        named_bar_sync(2, consumer_threads);
        for (int hg = cw; hg < HC * G; hg += kMmaWarps) {
            const int hl = hg / G, g = hg - hl * G;
            float Mx = -INFINITY;
            for (int j = 0; j < TG; ++j) Mx = fmaxf(Mx, ep_ml[((size_t)(hl + j * HC) * 16 + g) * 2]);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const int d = lane * 4;
            for (int j = 0; j < TG; ++j) {
                const size_t e = (size_t)(hl + j * HC) * 16 + g;
                const float m = ep_ml[e * 2];
                const float w = (m == -INFINITY) ? 0.f : fast_exp2(m - Mx);
                L = fmaf(w, ep_ml[e * 2 + 1], L);
                if (d < D) {
                    const float4 v = *reinterpret_cast<const float4*>(ep_o + e * D + d);
                    acc.x = fmaf(w, v.x, acc.x);
                    acc.y = fmaf(w, v.y, acc.y);
                    acc.z = fmaf(w, v.z, acc.z);
                    acc.w = fmaf(w, v.w, acc.w);
                }
            }
            if (d < D) *reinterpret_cast<float4*>(cta_o + (size_t)hg * D + d) = acc;
            if (lane == 0) {
                cta_ml[2 * hg] = Mx;
                cta_ml[2 * hg + 1] = L;
            }
        }
    }
    if (ctid == 0) TIDAL_STAMP(8);
    }   // consumers
    if (sum_heads && p.hist) {
        // every warp is done with its role: flush the CTA's digit counts with all threads
        __syncthreads();
        for (int i = threadIdx.x; i < TIDAL_TOPK_BINS; i += blockDim.x)
            if (sh_hist[i]) atomicAdd(&p.hist[(size_t)b * TIDAL_TOPK_BINS + i], sh_hist[i]);
    }
    store_attention_result<T>(p, cta_o, cta_ml, reinterpret_cast<float*>(smem + p.recv_off), HC, G, D, qh0, b, chunk);
}

template <typename T, int D>
static int launch_one(const AttnParams& p, dim3 grid, size_t smem, cudaStream_t st, int* query) {
    auto kern = decode_attn_mma_kernel<T, D>;
    const dim3 block((kMmaWarps + 1 + p.PW) * 32);
    if (query) return max_resident_clusters(kern, grid, block, smem, p.cluster, query);
    TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (p.cluster > 8) TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    TIDAL_CUDA_OK(launch_pdl(kern, grid, block, smem, st, (unsigned)(p.cluster > 1 ? p.cluster : 1), p));
    count_launch();
    return TIDAL_OK;
}

int launch_attn_mma(const AttnParams& p, int D, int dtype, dim3 grid, size_t smem, cudaStream_t st, int* query) {
    if (dtype == TIDAL_DTYPE_F16) {
        if (D == 128) return launch_one<__half, 128>(p, grid, smem, st, query);
        if (D == 64) return launch_one<__half, 64>(p, grid, smem, st, query);
    } else if (dtype == TIDAL_DTYPE_BF16) {
        if (D == 128) return launch_one<__nv_bfloat16, 128>(p, grid, smem, st, query);
        if (D == 64) return launch_one<__nv_bfloat16, 64>(p, grid, smem, st, query);
    }
    set_error("tensor-core attention is built for f16/bf16 and head_dim 64/128 (got dtype %d, head_dim %d)", dtype, D);
    return TIDAL_ERR_ARG;
}

}  // namespace tidal

TIDAL_TRACE_READER(tidal_trace_read_mma)
