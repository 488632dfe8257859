// RMSNorm over the last dimension: y = x * rsqrt(mean(x^2) + eps) * w, statistics in fp32.
// One CTA per row, 16-byte vector loads, the row is kept in registers between the two passes.
#include "common.cuh"

namespace tidal {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;     // vectors per thread: rows up to 256 * 8 * 8 = 16384 16-bit elements

template <typename T>
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                                                int hidden, float eps, int round_before_weight) {
    using V = Vec16<T>;
    constexpr int VEC = V::N;
    __shared__ float s_part[kNormThreads / 32];
    __shared__ float s_scale;
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    const int nvec = hidden / VEC;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
    float v[kNormMaxVec][VEC];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kNormMaxVec; ++u) {
        const int i = threadIdx.x + u * kNormThreads;
        if (i < nvec) {
            V::to_float(xr[i], v[u]);
#pragma unroll
            for (int e = 0; e < VEC; ++e) ss = fmaf(v[u][e], v[u][e], ss);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < kNormThreads / 32; ++i) tot += s_part[i];
        s_scale = rsqrtf(tot / (float)hidden + eps);
    }
    __syncthreads();
    const float scale = s_scale;
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(y + row * hidden);
#pragma unroll
    for (int u = 0; u < kNormMaxVec; ++u) {
        const int i = threadIdx.x + u * kNormThreads;
        if (i < nvec) {
            float wf[VEC], out[VEC];
            V::to_float(wr[i], wf);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float n = v[u][e] * scale;
                // the reference's PyTorch model rounds the normalised value to the storage type before the
                // weight (llama_tidaldecoding.py:122-127); its kernel multiplies in fp32 (rms_norm.cu:139-154)
                out[e] = round_before_weight ? __fmul_rn(V::round(n), wf[e]) : n * wf[e];
            }
            yr[i] = V::from_float(out);
        }
    }
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_rms_norm(const void* d_x, const void* d_weight, void* d_y, int64_t rows, int hidden, float eps, int dtype,
                              int round_before_weight, void* stream) {
    TIDAL_REQUIRE(d_x && d_weight && d_y, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(rows >= 1 && rows <= 0x7fffffff, TIDAL_ERR_ARG, "bad row count %lld", (long long)rows);
    TIDAL_REQUIRE((((uintptr_t)d_x | (uintptr_t)d_weight | (uintptr_t)d_y) & 15) == 0, TIDAL_ERR_ARG, "pointers must be 16-byte aligned");
    const int vec = dtype == TIDAL_DTYPE_F32 ? 4 : 8;
    TIDAL_REQUIRE(hidden >= vec && hidden % vec == 0, TIDAL_ERR_ARG, "hidden %d must be a multiple of %d", hidden, vec);   // rms_norm.cu: hid % 8
    TIDAL_REQUIRE(hidden / vec <= kNormThreads * kNormMaxVec, TIDAL_ERR_ARG, "hidden %d exceeds the built maximum %d", hidden,
                  vec * kNormThreads * kNormMaxVec);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    switch (dtype) {
        case TIDAL_DTYPE_F16: e = launch_pdl(rms_norm_kernel<__half>, dim3((unsigned)rows), dim3(kNormThreads), 0, st, 1, (const __half*)d_x, (const __half*)d_weight, (__half*)d_y, hidden, eps, round_before_weight); break;
        case TIDAL_DTYPE_BF16: e = launch_pdl(rms_norm_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(kNormThreads), 0, st, 1, (const __nv_bfloat16*)d_x, (const __nv_bfloat16*)d_weight, (__nv_bfloat16*)d_y, hidden, eps, round_before_weight); break;
        case TIDAL_DTYPE_F32: e = launch_pdl(rms_norm_kernel<float>, dim3((unsigned)rows), dim3(kNormThreads), 0, st, 1, (const float*)d_x, (const float*)d_weight, (float*)d_y, hidden, eps, round_before_weight); break;
        default: set_error("unknown dtype %d", dtype); return TIDAL_ERR_ARG;
    }
    TIDAL_CUDA_OK(e);
    count_launch();
    return TIDAL_OK;
}
