// RoPE on q and the new k, fused with the write of k,v into their KV-pool slots.
// One CTA per new token; threads cover (head, 16-byte vector) pairs of q, k and v.
// Rotate-half convention: out[i] = x[i]*cos - x[i+D/2]*sin for i < D/2 and
// out[i] = x[i]*cos + x[i-D/2]*sin for i >= D/2, angle = pos/scale * theta^(-2(i mod D/2)/D).
#include "common.cuh"

namespace tidal {

struct RopeParams {
    void* q;
    const void* q_src;   // rows of q are read from here (q itself when rotating in place)
    void* k;
    const void* v;
    char* kv;
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* pos0_dev;
    int32_t pos0;
    int32_t kv_pos_base;   // position held by the pool's first slot of every sequence (a shard of the context)
    const float* inv_freq;
    float theta, scale;
    int32_t rope_mode, rotate_k_in_place;
    int32_t B, tokens_per_seq, Hq, Hkv, page_size;
    int64_t num_pages;
    uint32_t* status;
};

// cs[i] = (cos, sin) of the token's angle for frequency index i < D/2, already rounded to T in mode 1.
template <typename T, int D>
__device__ __forceinline__ void rotate_vec(const T* row, int d0, const float2* cs, int rope_mode, float* out) {
    using V = Vec16<T>;
    constexpr int VEC = V::N;
    constexpr int HALF = D / 2;
    float x[VEC], y[VEC];
    V::to_float(*reinterpret_cast<const uint4*>(row + d0), x);
    const int d1 = d0 < HALF ? d0 + HALF : d0 - HALF;
    V::to_float(*reinterpret_cast<const uint4*>(row + d1), y);
    const float sign = d0 < HALF ? -1.f : 1.f;
    const int f0 = d0 % HALF;                    // a 16-byte vector never straddles the two halves
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const float c = cs[f0 + i].x, s = cs[f0 + i].y;
        if (rope_mode == 1) {
            // reference-model order: each product rounded to T, then the sum
            out[i] = V::round(__fadd_rn(V::round(__fmul_rn(x[i], c)), V::round(__fmul_rn(sign * y[i], s))));
        } else {
            out[i] = x[i] * c + sign * y[i] * s;
        }
    }
}

template <typename T, int D>
__global__ void rope_append_kernel(const RopeParams p) {
    using V = Vec16<T>;
    constexpr int VEC = V::N;
    constexpr int VPR = D / VEC;  // vectors per row
    __shared__ float2 cs[D / 2];
    pdl_wait();
    pdl_launch_dependents();
    const int tok = blockIdx.x;
    const int b = tok / p.tokens_per_seq;
    const int tpos = (p.pos0_dev ? p.pos0_dev[b] : p.pos0) + tok % p.tokens_per_seq;
    // The angle depends on the position and the frequency index only: D/2 threads evaluate the
    // transcendental functions once, all heads then rotate from the table.
    if (p.rope_mode != 0 && threadIdx.x < D / 2) {
        const int fi = threadIdx.x;
        const float inv = p.inv_freq ? p.inv_freq[fi] : 1.0f / powf(p.theta, (float)(2 * fi) / (float)D);
        const float ang = ((float)tpos / p.scale) * inv;
        float c = cosf(ang), s = sinf(ang);
        if (p.rope_mode == 1) {       // the reference model rounds cos and sin to the storage type first
            c = V::round(c);
            s = V::round(s);
        }
        cs[fi] = make_float2(c, s);
    }
    __syncthreads();

    char* kdst = nullptr;
    size_t plane = 0;
    if (p.kv) {
        const int spos = tpos - p.kv_pos_base;           // slot index within the sequence's part of the pool
        const int pg = spos / p.page_size;
        const int entry = spos - pg * p.page_size;
        int64_t page = -1;
        if (spos >= 0) page = p.page_table ? p.page_table[(size_t)b * p.pt_stride + pg] : (int64_t)b * p.pt_stride + pg;
        if (page < 0 || page >= p.num_pages) {
            if (threadIdx.x == 0 && p.status) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
        } else {
            plane = (size_t)p.page_size * p.Hkv * D * sizeof(T);
            kdst = p.kv + (size_t)page * 2 * plane + (size_t)entry * p.Hkv * D * sizeof(T);
        }
    }
    const int nq = p.q ? p.Hq * VPR : 0;
    const int nk = p.Hkv * VPR;
    // Phase 1: compute into registers (reads of both halves), then write — a row is
    // rotated in place, so all reads of the CTA must precede its writes.
    // Each thread handles at most kMaxItems vectors.
    constexpr int kMaxItems = 4;
    float res[kMaxItems][VEC];
#pragma unroll
    for (int cnt = 0; cnt < kMaxItems; ++cnt) {
        const int idx = threadIdx.x + cnt * blockDim.x;
        if (idx >= nq + nk) break;
        const bool is_q = idx < nq;
        const int j = is_q ? idx : idx - nq;
        const int h = j / VPR, d0 = (j % VPR) * VEC;
        const T* row = is_q ? reinterpret_cast<const T*>(p.q_src) + ((size_t)tok * p.Hq + h) * D
                            : reinterpret_cast<const T*>(p.k) + ((size_t)tok * p.Hkv + h) * D;
        if (p.rope_mode != 0) {
            rotate_vec<T, D>(row, d0, cs, p.rope_mode, res[cnt]);
        } else {
            V::to_float(*reinterpret_cast<const uint4*>(row + d0), res[cnt]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kMaxItems; ++c) {
        const int idx = threadIdx.x + c * blockDim.x;
        if (idx >= nq + nk) break;
        const bool is_q = idx < nq;
        const int j = is_q ? idx : idx - nq;
        const int h = j / VPR, d0 = (j % VPR) * VEC;
        const uint4 packed = V::from_float(res[c]);
        if (is_q) {
            if (p.rope_mode != 0 || p.q_src != p.q)
                *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.q) + ((size_t)tok * p.Hq + h) * D + d0) = packed;
        } else {
            if (p.rope_mode != 0 && p.rotate_k_in_place)
                *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.k) + ((size_t)tok * p.Hkv + h) * D + d0) = packed;
            if (kdst) *reinterpret_cast<uint4*>(kdst + ((size_t)h * D + d0) * sizeof(T)) = packed;
        }
    }
    if (kdst && p.v) {
        const uint4* vsrc = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.v) + (size_t)tok * p.Hkv * D);
        uint4* vdst = reinterpret_cast<uint4*>(kdst + plane);
        for (int idx = threadIdx.x; idx < nk; idx += blockDim.x) vdst[idx] = vsrc[idx];
    }
}

template <typename T>
static int launch_rope(const RopeParams& p, int D, int n_tokens, int threads, cudaStream_t st) {
    cudaError_t e;
    if (D == 64) e = launch_pdl(rope_append_kernel<T, 64>, dim3(n_tokens), dim3(threads), 0, st, 1, p);
    else if (D == 128) e = launch_pdl(rope_append_kernel<T, 128>, dim3(n_tokens), dim3(threads), 0, st, 1, p);
    else {
        set_error("unsupported head_dim %d (built: 64, 128)", D);
        return TIDAL_ERR_ARG;
    }
    TIDAL_CUDA_OK(e);
    count_launch();
    return TIDAL_OK;
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_rope_append(const tidal_rope_append_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_k != nullptr, TIDAL_ERR_ARG, "k must be given");
    TIDAL_REQUIRE(a->batch >= 1 && a->tokens_per_seq >= 1, TIDAL_ERR_ARG, "bad batch/tokens_per_seq");
    TIDAL_REQUIRE(a->num_kv_heads >= 1 && a->num_qo_heads >= 0, TIDAL_ERR_ARG, "bad head counts");
    TIDAL_REQUIRE(a->rope_mode >= 0 && a->rope_mode <= 2, TIDAL_ERR_ARG, "rope_mode must be 0, 1 or 2");
    TIDAL_REQUIRE(a->dtype >= 0 && a->dtype <= 2, TIDAL_ERR_ARG, "unknown dtype %d", a->dtype);
    TIDAL_REQUIRE(a->d_kv == nullptr || (a->page_size >= 1 && a->num_pages >= 1), TIDAL_ERR_ARG, "bad page_size/num_pages");
    TIDAL_REQUIRE(a->d_kv == nullptr || a->d_v != nullptr, TIDAL_ERR_ARG, "appending needs v");
    TIDAL_REQUIRE(a->rope_mode == 0 || a->rope_scale > 0.f, TIDAL_ERR_ARG, "rope_scale must be positive");
    TIDAL_REQUIRE(a->rope_mode == 0 || a->d_inv_freq || a->rope_theta > 0.f, TIDAL_ERR_ARG, "rope_theta must be positive");
    TIDAL_REQUIRE((((uintptr_t)a->d_q | (uintptr_t)a->d_k | (uintptr_t)a->d_v | (uintptr_t)a->d_kv | (uintptr_t)a->d_q_src) & 15) == 0,
                  TIDAL_ERR_ARG, "q, q_src, k, v and kv must be 16-byte aligned");
    TIDAL_REQUIRE(a->d_q_src == nullptr || a->d_q != nullptr, TIDAL_ERR_ARG, "q_src needs q as its destination");
    const int es = a->dtype == TIDAL_DTYPE_F32 ? 4 : 2;
    const int vec = 16 / es;
    const int vpr = a->head_dim / vec;
    const int items = ((a->d_q ? a->num_qo_heads : 0) + a->num_kv_heads) * vpr;
    int threads = (items + 3) / 4;                 // at most 4 vectors per thread
    threads = (threads + 31) / 32 * 32;
    if (threads < 64) threads = 64;
    TIDAL_REQUIRE(threads <= 1024, TIDAL_ERR_ARG, "too many heads for one CTA per token (%d vectors)", items);

    RopeParams p;
    p.q = a->d_q; p.q_src = a->d_q_src ? a->d_q_src : a->d_q; p.k = a->d_k; p.v = a->d_v; p.kv = (char*)a->d_kv;
    p.page_table = a->d_page_table; p.pt_stride = a->page_table_stride;
    p.pos0_dev = a->d_pos0; p.pos0 = a->pos0; p.kv_pos_base = a->kv_pos_base; p.inv_freq = a->d_inv_freq;
    p.theta = a->rope_theta; p.scale = a->rope_scale;
    p.rope_mode = a->rope_mode; p.rotate_k_in_place = a->rotate_k_in_place;
    p.B = a->batch; p.tokens_per_seq = a->tokens_per_seq; p.Hq = a->num_qo_heads; p.Hkv = a->num_kv_heads;
    p.page_size = a->page_size; p.num_pages = a->num_pages; p.status = a->d_status;
    const int n_tokens = a->batch * a->tokens_per_seq;
    cudaStream_t st = (cudaStream_t)stream;
    switch (a->dtype) {
        case TIDAL_DTYPE_F16: return launch_rope<__half>(p, a->head_dim, n_tokens, threads, st);
        case TIDAL_DTYPE_BF16: return launch_rope<__nv_bfloat16>(p, a->head_dim, n_tokens, threads, st);
        default: return launch_rope<float>(p, a->head_dim, n_tokens, threads, st);
    }
}
