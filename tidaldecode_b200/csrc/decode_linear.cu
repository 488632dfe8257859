// Decode-step linear layers: y[M][N] = x[M][K] W[N][K]^T for a handful of rows of activations
// (M <= 8: one token per sequence).  The weights are read once, so the op is a stream of W through
// HBM; everything next to it in a transformer layer is folded into the same launch:
//   * RMSNorm of x on the way into shared memory (every CTA needs all of x anyway),
//   * residual add on the way out,
//   * SiLU(gate) * up when W stacks the gate and up projections.
// Two kernels.  16-bit weights go through mma.sync.m16n8k16 with a tile of 16 rows of W as the A
// operand and the (up to 8) activation rows as the 8 columns of B, the tiles staged in shared memory
// by bulk copies (see below).  Everything else (fp32, odd shapes) takes the CUDA-core kernel: one warp
// owns two rows of W at a time, lanes stride over K in 16-byte vectors, a butterfly reduces the 2 M sums.
#include "common.cuh"

namespace tidal {

constexpr int kLinThreads = 512;
constexpr int kLinWarps = kLinThreads / 32;
constexpr int kLinUnroll = 4;

struct LinearParams {
    const void* x;
    const void* w;
    void* y;
    const void* residual;
    const void* norm_w;
    float eps;
    int round_before_weight;
    int N, K, epilogue;
    int items;            // row pairs
    int64_t up_off;       // elements from the first row of a pair to the second
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <typename T, int M>
__global__ void __launch_bounds__(kLinThreads, M <= 2 ? 2 : 1) decode_linear_kernel(const __grid_constant__ LinearParams p) {
    using V = Vec16<T>;
    constexpr int VEC = V::N;
    extern __shared__ __align__(128) unsigned char lin_smem[];
    T* xs = reinterpret_cast<T*>(lin_smem);                  // [M][K], normalised if asked for
    __shared__ float s_part[M][kLinWarps];
    __shared__ float s_scale[M];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = p.K;
    const int nvec = K / VEC;                                // vectors per row
    const T* W = reinterpret_cast<const T*>(p.w);
    const int item0 = blockIdx.x * kLinWarps + warp;
    const int item_step = gridDim.x * kLinWarps;

    // ---- weights of this warp's first pair towards L2 while the predecessor still runs
    if (item0 < p.items) {
        const int r = p.epilogue == TIDAL_LINEAR_SILU_MUL ? item0 : 2 * item0;
        const char* a = reinterpret_cast<const char*>(W + (size_t)r * K);
        const char* b = (p.epilogue == TIDAL_LINEAR_SILU_MUL || r + 1 < p.N) ? reinterpret_cast<const char*>(W + (size_t)r * K + p.up_off) : a;
        const int lines = (int)((size_t)K * sizeof(T) / 128);
        for (int l = lane; l < lines; l += 32) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a + (size_t)l * 128));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(b + (size_t)l * 128));
        }
    }
    pdl_wait();
    pdl_launch_dependents();

    // ---- activations into shared memory, RMS-normalised on the way if a norm weight is given
    {
        const uint4* xg = reinterpret_cast<const uint4*>(p.x);
        uint4* xv = reinterpret_cast<uint4*>(xs);
        if (p.norm_w) {
            float ss[M];
#pragma unroll
            for (int m = 0; m < M; ++m) ss[m] = 0.f;
            for (int i = threadIdx.x; i < nvec; i += kLinThreads) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float f[VEC];
                    V::to_float(xg[(size_t)m * nvec + i], f);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) ss[m] = fmaf(f[e], f[e], ss[m]);
                }
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], off);
                if (lane == 0) s_part[m][warp] = ss[m];
            }
            __syncthreads();
            if (threadIdx.x < M) {
                float tot = 0.f;
                for (int i = 0; i < kLinWarps; ++i) tot += s_part[threadIdx.x][i];
                s_scale[threadIdx.x] = rsqrtf(tot / (float)K + p.eps);
            }
            __syncthreads();
            const uint4* wn = reinterpret_cast<const uint4*>(p.norm_w);
            for (int i = threadIdx.x; i < nvec; i += kLinThreads) {
                float g[VEC];
                V::to_float(wn[i], g);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float f[VEC], o[VEC];
                    V::to_float(xg[(size_t)m * nvec + i], f);
                    const float sc = s_scale[m];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        const float n = f[e] * sc;
                        o[e] = p.round_before_weight ? __fmul_rn(V::round(n), g[e]) : n * g[e];
                    }
                    xv[(size_t)m * nvec + i] = V::from_float(o);      // rounded to T, as a separate norm kernel would store it
                }
            }
        } else {
            for (int i = threadIdx.x; i < M * nvec; i += kLinThreads) xv[i] = xg[i];
        }
    }
    __syncthreads();

    // ---- the stream
    const uint4* xv = reinterpret_cast<const uint4*>(xs);
    for (int item = item0; item < p.items; item += item_step) {
        const int r0 = p.epilogue == TIDAL_LINEAR_SILU_MUL ? item : 2 * item;
        const uint4* wa = reinterpret_cast<const uint4*>(W + (size_t)r0 * K);
        // an odd N leaves the last pair one row short: read the first row twice
        const bool pair = p.epilogue == TIDAL_LINEAR_SILU_MUL || r0 + 1 < p.N;
        const uint4* wb = pair ? reinterpret_cast<const uint4*>(W + (size_t)r0 * K + p.up_off) : wa;
        float acc0[M], acc1[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc0[m] = acc1[m] = 0.f;
        for (int i0 = lane; i0 < nvec; i0 += 32 * kLinUnroll) {
            uint4 a[kLinUnroll], b[kLinUnroll];
#pragma unroll
            for (int u = 0; u < kLinUnroll; ++u) {
                const int i = i0 + u * 32;
                if (i < nvec) {
                    a[u] = ldg_stream(wa + i);
                    b[u] = ldg_stream(wb + i);
                }
            }
#pragma unroll
            for (int u = 0; u < kLinUnroll; ++u) {
                const int i = i0 + u * 32;
                if (i < nvec) {
                    float fa[VEC], fb[VEC];
                    V::to_float(a[u], fa);
                    V::to_float(b[u], fb);
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        float fx[VEC];
                        V::to_float(xv[(size_t)m * nvec + i], fx);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            acc0[m] = fmaf(fa[e], fx[e], acc0[m]);
                            acc1[m] = fmaf(fb[e], fx[e], acc1[m]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                acc0[m] += __shfl_xor_sync(0xffffffffu, acc0[m], off);
                acc1[m] += __shfl_xor_sync(0xffffffffu, acc1[m], off);
            }
        }
        // lane m finishes batch row m
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (lane == m) {
                T* y = reinterpret_cast<T*>(p.y);
                if (p.epilogue == TIDAL_LINEAR_SILU_MUL) {
                    // torch: silu on the rounded gate (fp32 inside, rounded), times the rounded up value, rounded
                    const float g = V::round(acc0[m]), u = V::round(acc1[m]);
                    const float s = V::round(g / (1.f + __expf(-g)));
                    y[(size_t)m * (p.N / 2) + r0] = from_f32<T>(s * u);
                } else {
                    float o0 = acc0[m], o1 = acc1[m];
                    if (p.residual) {
                        const T* res = reinterpret_cast<const T*>(p.residual);
                        o0 = V::round(o0) + to_f32(res[(size_t)m * p.N + r0]);
                        if (r0 + 1 < p.N) o1 = V::round(o1) + to_f32(res[(size_t)m * p.N + r0 + 1]);
                    }
                    y[(size_t)m * p.N + r0] = from_f32<T>(o0);
                    if (r0 + 1 < p.N) y[(size_t)m * p.N + r0 + 1] = from_f32<T>(o1);
                }
            }
        }
    }
}

// ------------------------------------------------------------------ tensor-core kernel
// Same data path as the attention kernels: a producer warp brings tiles of 16 rows of W into a ring of
// shared-memory stages with one bulk copy per row (2-4 KB each, so DRAM sees long bursts and the SM
// keeps up to ~190 KB in flight whatever the register budget), 8 consumer warps read them with
// ldmatrix and multiply by the activation rows kept in shared memory.  The warps of a CTA split the
// K range of a stage between them and add their partial tiles up through shared memory once per
// tile (pair), while the producer is already filling stages of the next one.  The first stages are
// requested before the kernel is ordered after its predecessor: weights do not depend on anything.
constexpr int kLinConsumers = 8;
constexpr int kLinProducers = 2;      // a warp gets a bulk copy accepted every ~70 cycles: two of them for 16 rows of 2 KB
constexpr int kLinMmaThreads = (kLinConsumers + kLinProducers) * 32;

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_a(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Where the q, k and v rows of a fused q|k|v projection go: q (rotated) to q_out, k (rotated) and v into
// the slot of the sequence's newest token in the paged KV pool — what tidal_rope_append does in a
// launch of its own.
struct QkvEpilogue {
    void* q_out;                 // [M][Hq][D]
    char* kv;
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* pos_dev;
    int32_t pos;
    const float* inv_freq;
    float theta, scale;
    int32_t rope_mode, Hq, Hkv, D, page_size;
    int64_t num_pages;
};

struct LinearMmaGeom {
    // unit u covers tile t0 = (u / upg) * tpg + u % upg and, with tpu == 2, tile t0 + tile1_off
    int M, tiles, units, tpu, upg, tpg, tile1_off;
    int KC;        // elements of K per stage
    int S;         // stages
    uint32_t* status;
    int static_weights;   // the weights were not written by the stream's preceding kernel: fetch them before stream order
    int stream_x;         // the activations travel with the weights, M more rows per stage (no norm; for x too large to keep resident)
    QkvEpilogue qkv;      // TIDAL_LINEAR_QKV_ROPE only
};

__host__ __device__ inline size_t lin_x_bytes(int M, int K) { return ((size_t)M * (K * 2 + 16) + 127) & ~(size_t)127; }
__host__ __device__ inline size_t lin_stage_bytes(int KC, int rows) { return (size_t)rows * (KC * 2 + 16); }

template <typename T>
__global__ void __launch_bounds__(kLinMmaThreads) decode_linear_mma_kernel(const __grid_constant__ LinearParams p,
                                                                           const __grid_constant__ LinearMmaGeom gm) {
    using V = Vec16<T>;
    extern __shared__ __align__(128) unsigned char lin_smem[];
    const int K = p.K, M = gm.M, KC = gm.KC, S = gm.S;
    const int xpitch = K * 2 + 16;                            // bytes; the 8 x 4 lanes of a B fragment then hit 32 distinct banks
    const int pitch = KC * 2 + 16;                            // bytes between the 16 rows of a stage
    const int srows = gm.stream_x ? 16 + M : 16;              // rows of a stage: the tile, then (streamed) the x rows
    const size_t sbytes = lin_stage_bytes(KC, srows);
    unsigned char* xs = lin_smem;                             // [M] rows of x, normalised if asked for (resident mode)
    unsigned char* stages = lin_smem + (gm.stream_x ? 0 : lin_x_bytes(M, K));     // [S][srows][pitch]
    float* red = reinterpret_cast<float*>(stages + (size_t)S * sbytes);             // [2][8 warps][2 tiles][128]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(red + 2 * kLinConsumers * 256);
    uint64_t* empty_bar = full_bar + S;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + S);
    __shared__ float s_part[8][kLinConsumers];
    __shared__ float s_scale[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* W = reinterpret_cast<const T*>(p.w);
    const int nkc = (K + KC - 1) / KC;                        // stages per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kLinConsumers);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp >= kLinConsumers) {
        // ============================================================== producers
        const int pw = warp - kLinConsumers;                  // rows 8 pw .. 8 pw + 7 of every tile
        // with static weights and resident x never ordered after the predecessor: it reads nothing but weights
        if (!gm.static_weights || gm.stream_x) pdl_wait();
        int it = 0;
        for (int u = blockIdx.x; u < gm.units; u += gridDim.x) {
            for (int t = 0; t < gm.tpu; ++t) {
                const int tile = (u / gm.upg) * gm.tpg + u % gm.upg + (t ? gm.tile1_off : 0);
                if (tile >= gm.tiles) break;
                const int trow = pw * 8 + (lane & 7);
                const int row = min(tile * 16 + trow, p.N - 1);             // a short last tile reads the last row again
                const char* src = reinterpret_cast<const char*>(W + (size_t)row * K);
                for (int kc = 0; kc < nkc; ++kc, ++it) {
                    const int s = it % S;
                    if (it >= S && !mbar_wait_bounded(&empty_bar[s], ((it / S) - 1) & 1, abort_flag, gm.status)) break;
                    const uint32_t len = (uint32_t)min(KC, K - kc * KC) * 2u;
                    if (pw == 0 && lane == 0) mbar_arrive_expect_tx(&full_bar[s], (uint32_t)srows * len);   // (the other warp's copies may land first)
                    __syncwarp();
                    if (lane < 8)
                        bulk_g2s(stages + (size_t)s * sbytes + (size_t)trow * pitch, src + (size_t)kc * KC * 2, len, &full_bar[s]);
                    else if (gm.stream_x && pw == 0 && lane < 8 + M)
                        bulk_g2s(stages + (size_t)s * sbytes + (size_t)(16 + lane - 8) * pitch,
                                 reinterpret_cast<const char*>(p.x) + ((size_t)(lane - 8) * K + (size_t)kc * KC) * 2, len, &full_bar[s]);
                }
            }
        }
        // nothing of this CTA may still be in flight when it retires: after a wait that ran out, outlast the copies
        if (*abort_flag)
            for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    } else {
        // ============================================================== consumers
        pdl_wait();
        pdl_launch_dependents();
        const int ctid = threadIdx.x;                         // consumers are warps 0..7
        constexpr int CT = kLinConsumers * 32;
        // ---- activations into shared memory, RMS-normalised on the way if a norm weight is given
        if (!gm.stream_x) {
            const int nvec = K / 8;
            const uint4* xg = reinterpret_cast<const uint4*>(p.x);
            if (p.norm_w) {
                for (int m = 0; m < M; ++m) {
                    float ss = 0.f;
                    for (int i = ctid; i < nvec; i += CT) {
                        float f[8];
                        V::to_float(xg[(size_t)m * nvec + i], f);
#pragma unroll
                        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
                    }
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                    if (lane == 0) s_part[m][warp] = ss;
                }
                named_bar_sync(1, CT);
                if (ctid < M) {
                    float tot = 0.f;
                    for (int i = 0; i < kLinConsumers; ++i) tot += s_part[ctid][i];
                    s_scale[ctid] = rsqrtf(tot / (float)K + p.eps);
                }
                named_bar_sync(1, CT);
                const uint4* wn = reinterpret_cast<const uint4*>(p.norm_w);
                for (int i = ctid; i < nvec; i += CT) {
                    float gw[8];
                    V::to_float(wn[i], gw);
                    for (int m = 0; m < M; ++m) {
                        float f[8], o[8];
                        V::to_float(xg[(size_t)m * nvec + i], f);
                        const float sc = s_scale[m];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float n = f[e] * sc;
                            o[e] = p.round_before_weight ? __fmul_rn(V::round(n), gw[e]) : n * gw[e];
                        }
                        *reinterpret_cast<uint4*>(xs + (size_t)m * xpitch + (size_t)i * 16) = V::from_float(o);
                    }
                }
            } else {
                for (int i = ctid; i < M * nvec; i += CT) {
                    const int m = i / nvec, j = i - m * nvec;
                    *reinterpret_cast<uint4*>(xs + (size_t)m * xpitch + (size_t)j * 16) = xg[i];
                }
            }
        }
        named_bar_sync(1, CT);

        const int g = lane >> 2, c = lane & 3;
        const bool has_x = g < M;
        // B fragment: x[g][k0 + 2c, +1] and [k0 + 8 + 2c, +1], from the resident rows or from the stage
        const unsigned char* xrow = xs + (size_t)g * xpitch + c * 4;
        const size_t xstage = (size_t)(16 + g) * pitch + c * 4;
        const int kslice = KC / kLinConsumers;                           // K elements of a stage per warp (a multiple of 16)
        const uint32_t a_lane = (uint32_t)((lane & 15) * pitch + (lane >> 4) * 16);
        int it = 0, round = 0;
        for (int u = blockIdx.x; u < gm.units; u += gridDim.x, ++round) {
            const int t0 = (u / gm.upg) * gm.tpg + u % gm.upg, t1 = t0 + gm.tile1_off;
            const int ntile = (gm.tpu == 2 && t1 < gm.tiles) ? 2 : 1;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 1
            for (int t = 0; t < ntile; ++t) {
                float cur[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                for (int kc = 0; kc < nkc; ++kc, ++it) {
                    const int s = it % S;
                    mbar_wait_bounded(&full_bar[s], (it / S) & 1, abort_flag, gm.status);
                    const int len = min(KC, K - kc * KC);                // elements of this stage
                    const int k_lo = warp * kslice, k_hi = min(len, k_lo + kslice);
                    const uint32_t st = smem_u32(stages + (size_t)s * sbytes) + a_lane;
                    const unsigned char* xk = gm.stream_x ? stages + (size_t)s * sbytes + xstage : xrow + (size_t)kc * KC * 2;
#pragma unroll 4
                    for (int k0 = k_lo; k0 < k_hi; k0 += 16) {
                        uint32_t a[4];
                        ldsm_a(a, st + (uint32_t)k0 * 2);
                        uint32_t b0 = 0, b1 = 0;
                        if (has_x) {
                            b0 = *reinterpret_cast<const uint32_t*>(xk + (size_t)k0 * 2);
                            b1 = *reinterpret_cast<const uint32_t*>(xk + (size_t)k0 * 2 + 16);
                        }
                        mma16816<T>(cur, a, b0, b1);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty_bar[s]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (t == 0) acc[0][i] = cur[i];
                    else acc[1][i] = cur[i];
                }
            }
            // ---- add the 8 warps' partial tiles up (double-buffered: one barrier per round)
            float* rbuf = red + (size_t)(round & 1) * kLinConsumers * 256;
            float4* myred = reinterpret_cast<float4*>(rbuf) + (size_t)warp * 64 + lane;
            myred[0] = make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]);
            myred[32] = make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]);
            named_bar_sync(1, CT);
            if (ctid < 128) {
                // element e of tile 0 and of tile 1: fragment of lane el, register i
                const int e = ctid, el = e >> 2, i = e & 3;
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int w = 0; w < kLinConsumers; ++w) {
                    s0 += rbuf[(size_t)w * 256 + e];
                    s1 += rbuf[(size_t)w * 256 + 128 + e];
                }
                const int rr = (el >> 2) + (i >= 2 ? 8 : 0);              // row within the tile
                const int m = (el & 3) * 2 + (i & 1);                     // batch row
                if (m < M) {
                    T* y = reinterpret_cast<T*>(p.y);
                    const int ra = t0 * 16 + rr;
                    if (p.epilogue == TIDAL_LINEAR_QKV_ROPE) {
                        // s0, s1: elements i and i + D/2 of head h of sequence m's q|k|v row
                        const QkvEpilogue& e = gm.qkv;
                        const int tph = e.D / 16;                            // tiles per head
                        const int h = t0 / tph, i0 = (t0 - h * tph) * 16 + rr;
                        const int pos = e.pos_dev ? e.pos_dev[m] : e.pos;
                        float x0 = V::round(s0), x1 = V::round(s1);          // what a separate projection would have stored
                        if (h < e.Hq + e.Hkv && e.rope_mode != 0) {
                            const float inv = e.inv_freq ? e.inv_freq[i0] : 1.0f / powf(e.theta, (float)(2 * i0) / (float)e.D);
                            const float ang = ((float)pos / e.scale) * inv;
                            float cs = cosf(ang), sn = sinf(ang);
                            float r0, r1;
                            if (e.rope_mode == 1) {    // the reference model's order: cos, sin and each product rounded to T
                                cs = V::round(cs);
                                sn = V::round(sn);
                                r0 = V::round(__fadd_rn(V::round(__fmul_rn(x0, cs)), V::round(__fmul_rn(-x1, sn))));
                                r1 = V::round(__fadd_rn(V::round(__fmul_rn(x1, cs)), V::round(__fmul_rn(x0, sn))));
                            } else {
                                r0 = x0 * cs - x1 * sn;
                                r1 = x1 * cs + x0 * sn;
                            }
                            x0 = r0;
                            x1 = r1;
                        }
                        if (h < e.Hq) {
                            T* q = reinterpret_cast<T*>(e.q_out) + ((size_t)m * e.Hq + h) * e.D + i0;
                            q[0] = from_f32<T>(x0);
                            q[e.D / 2] = from_f32<T>(x1);
                        } else {
                            const int pg = pos / e.page_size, entry = pos - pg * e.page_size;
                            const int64_t page = e.page_table ? e.page_table[(size_t)m * e.pt_stride + pg] : (int64_t)m * e.pt_stride + pg;
                            if (pos < 0 || page < 0 || page >= e.num_pages) {
                                if (gm.status) atomicOr(gm.status, TIDAL_DEV_BAD_INDEX);
                            } else {
                                const size_t plane = (size_t)e.page_size * e.Hkv * e.D;           // elements of a page's K (or V) plane
                                const bool is_v = h >= e.Hq + e.Hkv;
                                const int hk = h - e.Hq - (is_v ? e.Hkv : 0);
                                T* dst = reinterpret_cast<T*>(e.kv) + (size_t)page * 2 * plane + (is_v ? plane : 0) +
                                         ((size_t)entry * e.Hkv + hk) * e.D + i0;
                                dst[0] = from_f32<T>(x0);
                                dst[e.D / 2] = from_f32<T>(x1);
                            }
                        }
                    } else if (p.epilogue == TIDAL_LINEAR_SILU_MUL) {
                        const float gt = V::round(s0), up = V::round(s1);
                        const float sg = V::round(gt / (1.f + __expf(-gt)));
                        y[(size_t)m * (p.N / 2) + ra] = from_f32<T>(sg * up);
                    } else {
                        const T* res = reinterpret_cast<const T*>(p.residual);
                        if (ra < p.N) y[(size_t)m * p.N + ra] = from_f32<T>(res ? V::round(s0) + to_f32(res[(size_t)m * p.N + ra]) : s0);
                        const int rb = t1 * 16 + rr;
                        if (ntile == 2 && rb < p.N) y[(size_t)m * p.N + rb] = from_f32<T>(res ? V::round(s1) + to_f32(res[(size_t)m * p.N + rb]) : s1);
                    }
                }
            }
        }
    }
}

// false: the shapes do not fit (the caller takes the CUDA-core kernel).  One CTA per SM with all of its
// shared memory: stages as long as they come (4 KB per row) and at least three of them.  (Half-SM CTAs,
// two per SM or one next to the next launch's, measured no better: the kernel streams at the copy rate
// either way and pays ~5 us per launch for ramp-up and tail.)
static bool plan_linear_mma(const LinearParams& p, int M, LinearMmaGeom* gm, size_t* smem, int* per_sm) {
    const size_t other = (size_t)2 * kLinConsumers * 256 * sizeof(float) + 2 * 8 * sizeof(uint64_t) + 64;
    const size_t budget = 225 * 1024;
    *per_sm = 1;
    auto try_plan = [&](int KC, bool stream) {
        if (KC > p.K && KC > 128) return false;               // no stage longer than a row (but at least 128: 16 per warp)
        const size_t fixed = other + (stream ? 0 : lin_x_bytes(M, p.K));
        const size_t stage = lin_stage_bytes(KC, stream ? 16 + M : 16);
        if (fixed + 3 * stage > budget) return false;
        const int S = (int)((budget - fixed) / stage);
        gm->KC = KC; gm->S = S > 8 ? 8 : S; gm->stream_x = stream ? 1 : 0;
        *smem = fixed + (size_t)gm->S * stage;
        return true;
    };
    // x resident in shared memory (needed for the fused norm; lets the producers run ahead of stream order) with
    // rows of at least 2 KB per copy; else x travelling with the weights; else resident with shorter stages
    for (int KC : {2048, 1024})
        if (try_plan(KC, false)) return true;
    if (!p.norm_w)
        for (int KC : {2048, 1024})
            if (try_plan(KC, true)) return true;
    for (int KC : {512, 256, 128})
        if (try_plan(KC, false)) return true;
    return false;
}

template <typename T>
static int launch_linear_mma(const LinearParams& p, LinearMmaGeom gm, size_t smem, int per_sm, cudaStream_t st) {
    auto kern = decode_linear_mma_kernel<T>;
    const int sms = sm_count_cached();
    if (p.epilogue == TIDAL_LINEAR_SILU_MUL) {
        const int F = p.N / 2;
        gm.tiles = p.N / 16; gm.units = F / 16; gm.tpu = 2; gm.upg = gm.units; gm.tpg = gm.units; gm.tile1_off = F / 16;
    } else if (p.epilogue == TIDAL_LINEAR_QKV_ROPE) {
        const int D = gm.qkv.D;                     // pairs of tiles half a head apart
        gm.tiles = p.N / 16; gm.units = p.N / 32; gm.tpu = 2; gm.upg = D / 32; gm.tpg = D / 16; gm.tile1_off = D / 32;
    } else {
        gm.tiles = (p.N + 15) / 16;
        gm.tpu = gm.tiles >= 8 * sms ? 2 : 1;       // small matrices: one tile per round, so that every CTA gets some
        gm.units = (gm.tiles + gm.tpu - 1) / gm.tpu; gm.upg = 1; gm.tpg = gm.tpu; gm.tile1_off = 1;
    }
    TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = gm.units < sms * per_sm ? gm.units : sms * per_sm;
    TIDAL_CUDA_OK(launch_pdl(kern, dim3(grid), dim3(kLinMmaThreads), smem, st, 1, p, gm));
    count_launch();
    return TIDAL_OK;
}

template <typename T, int M>
static int launch_linear(const LinearParams& p, cudaStream_t st) {
    auto kern = decode_linear_kernel<T, M>;
    const size_t smem = (size_t)M * p.K * sizeof(T);
    TIDAL_REQUIRE(smem <= 200 * 1024, TIDAL_ERR_ARG, "activations of %d x %d do not fit shared memory", M, p.K);
    TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int sms = sm_count_cached();
    const int per_sm = (M <= 2 && smem <= 100 * 1024) ? 2 : 1;
    int grid = (p.items + kLinWarps - 1) / kLinWarps;
    if (grid > sms * per_sm) grid = sms * per_sm;
    TIDAL_CUDA_OK(launch_pdl(kern, dim3(grid), dim3(kLinThreads), smem, st, 1, p));
    count_launch();
    return TIDAL_OK;
}

template <typename T>
static int dispatch_m(const LinearParams& p, int M, cudaStream_t st) {
    switch (M) {
        case 1: return launch_linear<T, 1>(p, st);
        case 2: return launch_linear<T, 2>(p, st);
        case 3: return launch_linear<T, 3>(p, st);
        case 4: return launch_linear<T, 4>(p, st);
        case 5: return launch_linear<T, 5>(p, st);
        case 6: return launch_linear<T, 6>(p, st);
        case 7: return launch_linear<T, 7>(p, st);
        case 8: return launch_linear<T, 8>(p, st);
        default: set_error("decode linear takes 1..8 rows of activations, got %d", M); return TIDAL_ERR_ARG;
    }
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_decode_linear(const tidal_linear_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_x && a->d_w && a->d_y, TIDAL_ERR_ARG, "x, w and y must be given");
    TIDAL_REQUIRE(a->M >= 1 && a->M <= 8, TIDAL_ERR_ARG, "M %d out of range [1,8]", a->M);
    TIDAL_REQUIRE(a->dtype >= 0 && a->dtype <= 2, TIDAL_ERR_ARG, "unknown dtype %d", a->dtype);
    const int vec = a->dtype == TIDAL_DTYPE_F32 ? 4 : 8;
    TIDAL_REQUIRE(a->K >= vec && a->K % vec == 0, TIDAL_ERR_ARG, "K %d must be a multiple of %d", a->K, vec);
    TIDAL_REQUIRE(a->N >= 1, TIDAL_ERR_ARG, "bad N %d", a->N);
    TIDAL_REQUIRE(a->epilogue == TIDAL_LINEAR_PLAIN || a->epilogue == TIDAL_LINEAR_SILU_MUL, TIDAL_ERR_ARG, "unknown epilogue %d",
                  a->epilogue);
    TIDAL_REQUIRE(a->epilogue != TIDAL_LINEAR_SILU_MUL || (a->N % 2 == 0 && !a->d_residual), TIDAL_ERR_ARG,
                  "the gated form needs an even N and takes no residual");
    TIDAL_REQUIRE((((uintptr_t)a->d_x | (uintptr_t)a->d_w | (uintptr_t)a->d_norm_weight) & 15) == 0, TIDAL_ERR_ARG,
                  "x, w and the norm weight must be 16-byte aligned");
    LinearParams p;
    p.x = a->d_x; p.w = a->d_w; p.y = a->d_y; p.residual = a->d_residual; p.norm_w = a->d_norm_weight;
    p.eps = a->norm_eps; p.round_before_weight = a->norm_round_before_weight;
    p.N = a->N; p.K = a->K; p.epilogue = a->epilogue;
    if (a->epilogue == TIDAL_LINEAR_SILU_MUL) {
        p.items = a->N / 2;
        p.up_off = (int64_t)(a->N / 2) * a->K;
    } else {
        p.items = (a->N + 1) / 2;
        p.up_off = a->K;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // tensor cores: 16-bit weights, whole 16-element k steps, 16-byte row starts, whole gate/up tiles
    const bool mma_ok = a->dtype != TIDAL_DTYPE_F32 && a->K % 16 == 0 && a->K >= 128 && a->N >= 16 &&
                        (a->epilogue != TIDAL_LINEAR_SILU_MUL || (a->N / 2) % 16 == 0);
    if (mma_ok) {
        LinearMmaGeom gm;
        size_t smem = 0;
        gm.M = a->M; gm.status = (uint32_t*)a->d_status; gm.static_weights = a->static_weights;
        int per_sm = 1;
        if (plan_linear_mma(p, a->M, &gm, &smem, &per_sm)) {
            if (a->dtype == TIDAL_DTYPE_F16) return launch_linear_mma<__half>(p, gm, smem, per_sm, st);
            return launch_linear_mma<__nv_bfloat16>(p, gm, smem, per_sm, st);
        }
    }
    switch (a->dtype) {
        case TIDAL_DTYPE_F16: return dispatch_m<__half>(p, a->M, st);
        case TIDAL_DTYPE_BF16: return dispatch_m<__nv_bfloat16>(p, a->M, st);
        default: return dispatch_m<float>(p, a->M, st);
    }
}

extern "C" int tidal_decode_qkv(const tidal_linear_args* a, const tidal_rope_append_args* r, void* stream) {
    TIDAL_REQUIRE(a != nullptr && r != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_x && a->d_w, TIDAL_ERR_ARG, "x and w must be given");
    TIDAL_REQUIRE(r->d_q && r->d_kv, TIDAL_ERR_ARG, "the q output and the KV pool must be given");
    TIDAL_REQUIRE(a->M >= 1 && a->M <= 8 && r->batch == a->M && r->tokens_per_seq == 1, TIDAL_ERR_ARG,
                  "one new token for each of 1..8 sequences (M %d, batch %d, tokens_per_seq %d)", a->M, r->batch, r->tokens_per_seq);
    TIDAL_REQUIRE((a->dtype == TIDAL_DTYPE_F16 || a->dtype == TIDAL_DTYPE_BF16) && r->dtype == a->dtype, TIDAL_ERR_ARG,
                  "the fused q|k|v projection is built for f16/bf16");
    TIDAL_REQUIRE(r->head_dim == 64 || r->head_dim == 128, TIDAL_ERR_ARG, "unsupported head_dim %d (built: 64, 128)", r->head_dim);
    TIDAL_REQUIRE(r->num_qo_heads >= 1 && r->num_kv_heads >= 1 && a->N == (r->num_qo_heads + 2 * r->num_kv_heads) * r->head_dim,
                  TIDAL_ERR_ARG, "W must have (Hq + 2 Hkv) * D = %d rows, got %d", (r->num_qo_heads + 2 * r->num_kv_heads) * r->head_dim, a->N);
    TIDAL_REQUIRE(a->K % 16 == 0 && a->K >= 128, TIDAL_ERR_ARG, "K %d must be a multiple of 16, at least 128", a->K);
    TIDAL_REQUIRE(r->rope_mode >= 0 && r->rope_mode <= 2, TIDAL_ERR_ARG, "rope_mode must be 0, 1 or 2");
    TIDAL_REQUIRE(r->kv_pos_base == 0 && r->d_q_src == nullptr, TIDAL_ERR_ARG,
                  "tidal_decode_qkv writes whole-sequence pools and produces q itself: kv_pos_base must be 0, d_q_src NULL");
    TIDAL_REQUIRE(r->rope_mode == 0 || r->rope_scale > 0.f, TIDAL_ERR_ARG, "rope_scale must be positive");
    TIDAL_REQUIRE(r->rope_mode == 0 || r->d_inv_freq || r->rope_theta > 0.f, TIDAL_ERR_ARG, "rope_theta must be positive");
    TIDAL_REQUIRE(r->page_size >= 1 && r->num_pages >= 1, TIDAL_ERR_ARG, "bad page_size/num_pages");
    TIDAL_REQUIRE((((uintptr_t)a->d_x | (uintptr_t)a->d_w | (uintptr_t)a->d_norm_weight) & 15) == 0, TIDAL_ERR_ARG,
                  "x, w and the norm weight must be 16-byte aligned");
    LinearParams p;
    p.x = a->d_x; p.w = a->d_w; p.y = nullptr; p.residual = nullptr; p.norm_w = a->d_norm_weight;
    p.eps = a->norm_eps; p.round_before_weight = a->norm_round_before_weight;
    p.N = a->N; p.K = a->K; p.epilogue = TIDAL_LINEAR_QKV_ROPE;
    p.items = 0; p.up_off = 0;
    LinearMmaGeom gm;
    gm.M = a->M; gm.status = r->d_status ? (uint32_t*)r->d_status : (uint32_t*)a->d_status; gm.static_weights = a->static_weights;
    QkvEpilogue& e = gm.qkv;
    e.q_out = r->d_q; e.kv = (char*)r->d_kv; e.page_table = r->d_page_table; e.pt_stride = r->page_table_stride;
    e.pos_dev = r->d_pos0; e.pos = r->pos0; e.inv_freq = r->d_inv_freq; e.theta = r->rope_theta; e.scale = r->rope_scale;
    e.rope_mode = r->rope_mode; e.Hq = r->num_qo_heads; e.Hkv = r->num_kv_heads; e.D = r->head_dim; e.page_size = r->page_size;
    e.num_pages = r->num_pages;
    size_t smem = 0;
    int per_sm = 1;
    TIDAL_REQUIRE(plan_linear_mma(p, a->M, &gm, &smem, &per_sm), TIDAL_ERR_ARG, "activations of %d x %d do not fit shared memory", a->M, a->K);
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == TIDAL_DTYPE_F16) return launch_linear_mma<__half>(p, gm, smem, per_sm, st);
    return launch_linear_mma<__nv_bfloat16>(p, gm, smem, per_sm, st);
}
