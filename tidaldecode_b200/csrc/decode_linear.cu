// Decode-step linear layers: y[M][N] = x[M][K] W[N][K]^T for a handful of rows of activations
// (M <= 8: one token per sequence).  The weights are read once, so the op is a stream of W through
// HBM; everything next to it in a transformer layer is folded into the same launch:
//   * RMSNorm of x on the way into shared memory (every CTA needs all of x anyway),
//   * residual add on the way out,
//   * SiLU(gate) * up when W stacks the gate and up projections.
// One warp owns two rows of W at a time (for the gated form: gate row r and up row r + N/2), lanes
// stride over K in 16-byte vectors with four vectors per row in flight, accumulate in fp32, and a
// butterfly reduces the 2 M sums.  Before the kernel is ordered after its predecessor it already
// asks L2 for its first rows: the weights do not depend on anything.
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
    extern __shared__ __align__(16) unsigned char lin_smem[];
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
    switch (a->dtype) {
        case TIDAL_DTYPE_F16: return dispatch_m<__half>(p, a->M, st);
        case TIDAL_DTYPE_BF16: return dispatch_m<__nv_bfloat16>(p, a->M, st);
        default: return dispatch_m<float>(p, a->M, st);
    }
}
