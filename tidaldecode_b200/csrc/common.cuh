// Shared device/host helpers of the tidal_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <utility>

#include "../../include/tidal_b200.h"

namespace tidal {

// ---------------------------------------------------------------- host errors
void set_error(const char* fmt, ...);

#define TIDAL_REQUIRE(cond, code, ...)      \
    do {                                    \
        if (!(cond)) {                      \
            ::tidal::set_error(__VA_ARGS__); \
            return (code);                  \
        }                                   \
    } while (0)

#define TIDAL_CUDA_OK(expr)                                                        \
    do {                                                                           \
        cudaError_t e__ = (expr);                                                  \
        if (e__ != cudaSuccess) {                                                  \
            ::tidal::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));   \
            return TIDAL_ERR_CUDA;                                                 \
        }                                                                          \
    } while (0)

// ------------------------------------------------------------------ workspace
// One caller-owned buffer, carved at fixed offsets so that every entry point
// finds the same regions.  All counters are zero at rest.
struct WsLayout {
    size_t status_off;     // uint32[64]: [0] = OR of TIDAL_DEV_* bits
    size_t part_o_off;     // float [max_batch*Hq][kMaxChunks][D]
    size_t part_ml_off;    // float [max_batch*Hq][kMaxChunks][2]
    size_t hist_off;       // uint32 [max_rows][TIDAL_TOPK_BINS]   (top-k's own, when the caller gives none)
    size_t row_state_off;  // uint32 [max_rows][8]   per-row top-k state
    size_t xc_off;         // uint32 [max_batch*Hq][16]  arrival counters of clusters that share one token list
    size_t cand_off;       // uint64 [max_rows][cand_cap]
    size_t sel_off;        // uint64 [max_rows][kMaxK]  keys certainly selected, before ordering
    size_t total;
    int64_t cand_cap;
};

constexpr int kMaxChunks = 1024;    // upper bound of the KV split per (sequence, head slice)
constexpr int kMaxK = 16384;        // largest k tidal_topk accepts
constexpr int64_t kCandCapMax = 1 << 20;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline WsLayout ws_layout(int max_batch, int num_qo_heads, int head_dim, int max_rows, int64_t max_n) {
    WsLayout L;
    size_t off = 0;
    L.status_off = off;
    off += 256;
    L.part_o_off = off;
    off = align_up(off + sizeof(float) * (size_t)max_batch * num_qo_heads * kMaxChunks * head_dim, 256);
    L.part_ml_off = off;
    off = align_up(off + sizeof(float) * (size_t)max_batch * num_qo_heads * kMaxChunks * 2, 256);
    L.hist_off = off;
    off = align_up(off + sizeof(uint32_t) * (size_t)max_rows * TIDAL_TOPK_BINS, 256);
    L.row_state_off = off;
    off = align_up(off + sizeof(uint32_t) * (size_t)max_rows * 8, 256);
    L.xc_off = off;
    off = align_up(off + sizeof(uint32_t) * (size_t)max_batch * num_qo_heads * 16, 256);
    L.cand_cap = max_n < kCandCapMax ? max_n : kCandCapMax;
    if (L.cand_cap < 1) L.cand_cap = 1;
    L.cand_off = off;
    off = align_up(off + sizeof(uint64_t) * (size_t)max_rows * L.cand_cap, 256);
    L.sel_off = off;
    off = align_up(off + sizeof(uint64_t) * (size_t)max_rows * kMaxK, 256);
    L.total = off;
    return L;
}

// Kernel launches issued by this library since load (host-side counter).
void count_launch(int n = 1);

// Geometry a workspace was initialised for, looked up by its device address
// (host-side table filled by tidal_ws_init; nullptr when unknown).
const WsLayout* find_ws(const void* d_ws);

// ------------------------------------------------------------------- dtypes
template <typename T>
struct Vec16;  // 16-byte vector of T converted to float[N]

template <>
struct Vec16<__half> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void to_float(const uint4& v, float* f) {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    __device__ static __forceinline__ uint4 from_float(const float* f) {
        uint4 v;
        __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        return v;
    }
    __device__ static __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};

template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void to_float(const uint4& v, float* f) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static __forceinline__ uint4 from_float(const float* f) {
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        return v;
    }
    __device__ static __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};

template <>
struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void to_float(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    __device__ static __forceinline__ uint4 from_float(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    __device__ static __forceinline__ float round(float x) { return x; }
};

__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(float x) { return x; }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }

// --------------------------------------------------- order-preserving keys
// fp32 → uint32 whose unsigned order equals the float order (−NaN lowest,
// +NaN highest).  The first radix digit of the top-k is the top 12 bits.
__host__ __device__ __forceinline__ uint32_t ordered_key(float x) {
#ifdef __CUDA_ARCH__
    uint32_t b = __float_as_uint(x);
#else
    union { float f; uint32_t u; } c; c.f = x; uint32_t b = c.u;
#endif
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
    uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}
constexpr int kDigit0Shift = 20;  // 32 - log2(TIDAL_TOPK_BINS)

// ----------------------------------------------------- mbarrier / bulk copy
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait with an iteration limit.  On expiry: raises *abort_flag (shared memory, so
// every later wait of the CTA returns at once), ORs TIDAL_DEV_WAIT_TIMEOUT into
// *status and returns false.  The caller keeps its control flow and produces
// garbage, which the status word marks as such.
constexpr uint32_t kWaitSpinLimit = 1u << 21;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  uint32_t* status) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < kWaitSpinLimit; ++i) {
        if (*abort_flag) return false;
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 16) __nanosleep(i > 1024 ? 256 : 32);
    }
    *abort_flag = 1;
    if (status) atomicOr(status, TIDAL_DEV_WAIT_TIMEOUT);
    return false;
}

// One-dimensional bulk copy global → shared through the TMA unit; completion is
// signalled on `bar` as `bytes` transaction bytes.  dst, src 16-byte aligned,
// bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Split cluster barrier: every thread of every CTA of the cluster arrives once and waits once per phase.
// The arrive at the top of a kernel only says "this CTA is running" (no memory to publish: relaxed); the
// matching wait sits right before the first store into another CTA's shared memory, so the prologue and
// the whole streaming loop run without waiting for the slowest CTA of the cluster to start.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


// ------------------------------------------- programmatic dependent launch
// Every kernel of the library is launched with the programmatic-stream-serialization
// attribute and begins with pdl_wait(): memory effects are ordered exactly as in plain
// stream order, but the next kernel's launch latency and prologue overlap the tail of
// the previous one.  pdl_launch_dependents() lets the successor be scheduled early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cluster_x,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    int n = 0;
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
    if (cluster_x > 1) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = cluster_x;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// How many clusters of `cluster_x` CTAs of this launch geometry the current device can hold at the same time
// (a cluster lives inside one GPC).  Asked once per (kernel, geometry, device) and remembered: planners use it
// to decide whether a non-portable cluster size would run all its clusters side by side.
template <typename... KArgs>
inline int max_resident_clusters(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x, int* out) {
    struct Entry { const void* fn; size_t smem; unsigned threads; int cluster, dev, result; };
    static Entry cache[32];
    static int n_cached = 0;
    static std::mutex mu;
    int dev = 0;
    TIDAL_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < n_cached; ++i) {
        const Entry& e = cache[i];
        if (e.fn == (const void*)kern && e.smem == smem && e.threads == block.x && e.cluster == cluster_x && e.dev == dev) {
            *out = e.result;
            return TIDAL_OK;
        }
    }
    TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (cluster_x > 8) TIDAL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)cluster_x;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();          // not launchable in this shape: report none, the caller keeps the portable size
        n = 0;
    }
    if (n_cached < 32) cache[n_cached++] = Entry{(const void*)kern, smem, block.x, cluster_x, dev, n};
    *out = n;
    return TIDAL_OK;
}

// SM count of the current device (148 if it cannot be read); looked up once.
inline int sm_count_cached() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// Timeline stamps for debugging (compiled only with -DTIDAL_TRACE; nothing in a normal build).
// Each translation unit that stamps has its own array [kTraceCtas][kTraceSlots][2] of
// (%globaltimer ns, clock64) and exports a reader through TIDAL_TRACE_READER(name).
#ifdef TIDAL_TRACE
constexpr int kTraceSlots = 16, kTraceCtas = 2048;
static __device__ unsigned long long g_trace[kTraceCtas * kTraceSlots * 2];
__device__ __forceinline__ void trace_stamp(int slot) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < kTraceCtas) {
        g_trace[(cta * kTraceSlots + slot) * 2] = t;
        g_trace[(cta * kTraceSlots + slot) * 2 + 1] = (unsigned long long)clock64();
    }
}
#define TIDAL_STAMP(slot) ::tidal::trace_stamp(slot)
#define TIDAL_TRACE_READER(name)                                                                              \
    extern "C" int name(unsigned long long* host, int clear) {                                                 \
        cudaError_t e = cudaMemcpyFromSymbol(host, ::tidal::g_trace, sizeof(::tidal::g_trace));                \
        if (e == cudaSuccess && clear) {                                                                       \
            void* d = nullptr;                                                                                 \
            e = cudaGetSymbolAddress(&d, ::tidal::g_trace);                                                    \
            if (e == cudaSuccess) e = cudaMemset(d, 0, sizeof(::tidal::g_trace));                              \
        }                                                                                                      \
        return e == cudaSuccess ? 0 : -3;                                                                      \
    }
#else
#define TIDAL_STAMP(slot) ((void)0)
#define TIDAL_TRACE_READER(name)
#endif

constexpr float kLog2e = 1.4426950408889634f;

}  // namespace tidal
