// Quest's page-criticality estimate and the per-page key bounds it reads (the legacy operators on the
// reference's surface that TidalDecode's own layers do not call): for every KV page the element-wise
// maximum and minimum of its keys are kept in a second paged pool of the same layout as the KV pool
// ("metadata": plane 0 = maxima, plane 1 = minima, one ENTRY per KV page), and the estimate of a page for a
// query head is the upper bound  sum_d max(q_d * max_d, q_d * min_d)  of q.k over the keys of the page
// (kernels/include/decode/decode_attn.cuh:141-172, 249-405; kernels/include/decode/decode_page.cuh:417-441).
//
// Both kernels stream contiguous rows (a page's rows of one plane are H*D elements apart) with 128-bit
// loads; they are bandwidth-bound and tiny next to the attention itself.
#include "common.cuh"

namespace tidal {

struct PageMetaParams {
    const char* kv;               // KV pool [pages][2][page_size][H][D]
    char* meta;                   // metadata pool [meta_pages][2][meta_page_size][H][D]
    const int32_t* kv_table;      // [batch][kv_stride] or nullptr (identity: page b * kv_stride + j)
    const int32_t* meta_table;    // [batch][meta_stride] or nullptr (identity)
    int64_t kv_stride, meta_stride;
    int32_t batch, H, page_size, meta_page_size;
    int64_t num_pages, num_meta_pages;
    int32_t first_page, n_pages;  // logical KV pages [first_page, first_page + n_pages) of every sequence are rebuilt
    int32_t seq_len;              // tokens per sequence: the last page may be partly filled
    uint32_t* status;
};

// One (sequence, logical page, head, 16-byte vector) per thread: bounds over the page's valid keys.
template <typename T, int D>
__global__ void page_meta_kernel(const PageMetaParams p) {
    using V = Vec16<T>;
    constexpr int VEC = V::N, VPR = D / VEC;
    pdl_wait();
    pdl_launch_dependents();
    const int64_t units = (int64_t)p.batch * p.n_pages * p.H * VPR;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(u % VPR);
        const int h = (int)((u / VPR) % p.H);
        const int pg = p.first_page + (int)((u / ((int64_t)VPR * p.H)) % p.n_pages);
        const int b = (int)(u / ((int64_t)VPR * p.H * p.n_pages));
        const int valid = min(p.page_size, p.seq_len - pg * p.page_size);      // keys of this page that exist
        if (valid <= 0) continue;
        const int64_t page = p.kv_table ? p.kv_table[(size_t)b * p.kv_stride + pg] : (int64_t)b * p.kv_stride + pg;
        const int mpg = pg / p.meta_page_size, ment = pg - mpg * p.meta_page_size;
        const int64_t mpage = p.meta_table ? p.meta_table[(size_t)b * p.meta_stride + mpg] : (int64_t)b * p.meta_stride + mpg;
        if (page < 0 || page >= p.num_pages || mpage < 0 || mpage >= p.num_meta_pages) {
            if (p.status) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
            continue;
        }
        const size_t row = (size_t)p.H * D * sizeof(T);
        const char* k = p.kv + (size_t)page * 2 * p.page_size * row + (size_t)h * D * sizeof(T) + (size_t)v * 16;
        float mx[VEC], mn[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            mx[i] = -INFINITY;
            mn[i] = INFINITY;
        }
        for (int e = 0; e < valid; ++e) {
            float x[VEC];
            V::to_float(*reinterpret_cast<const uint4*>(k + (size_t)e * row), x);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                mx[i] = fmaxf(mx[i], x[i]);
                mn[i] = fminf(mn[i], x[i]);
            }
        }
        char* m = p.meta + (size_t)mpage * 2 * p.meta_page_size * row + (size_t)ment * row + (size_t)h * D * sizeof(T) + (size_t)v * 16;
        *reinterpret_cast<uint4*>(m) = V::from_float(mx);                                   // plane 0: maxima
        *reinterpret_cast<uint4*>(m + (size_t)p.meta_page_size * row) = V::from_float(mn);   // plane 1: minima
    }
}

struct EstimateParams {
    const void* q;                // [batch][Hq][D]
    const char* meta;
    const int32_t* meta_table;
    int64_t meta_stride;
    void* out;                    // [batch][Hq][out_stride] of out_dtype
    int64_t out_stride;
    int32_t batch, Hq, H, meta_page_size, n_entries, out_dtype;
    int64_t num_meta_pages;
    uint32_t* status;
};

// A group of D*sizeof(T)/16 lanes per (entry, KV head): the group loads the head's maxima and minima once and
// forms the bound for each of the G query heads that share the KV head (q in shared memory as fp32).
template <typename T, int D>
__global__ void __launch_bounds__(256) estimate_kernel(const EstimateParams p) {
    using V = Vec16<T>;
    constexpr int VEC = V::N, LPR = D / VEC;          // lanes per row
    extern __shared__ float qs[];                     // [Hq][D]
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.y;
    const int G = p.Hq / p.H;
    for (int i = threadIdx.x; i < p.Hq * D; i += blockDim.x)
        qs[i] = to_f32(reinterpret_cast<const T*>(p.q)[(size_t)b * p.Hq * D + i]);
    __syncthreads();
    const int lane = threadIdx.x % LPR;
    const unsigned gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << ((threadIdx.x & 31) / LPR * LPR));
    const int groups = blockDim.x / LPR;
    const int64_t units = (int64_t)p.n_entries * p.H;
    const size_t row = (size_t)p.H * D * sizeof(T);
    for (int64_t u = (int64_t)blockIdx.x * groups + threadIdx.x / LPR; u < units; u += (int64_t)gridDim.x * groups) {
        const int h = (int)(u % p.H);
        const int e = (int)(u / p.H);
        const int mpg = e / p.meta_page_size, ment = e - mpg * p.meta_page_size;
        const int64_t mpage = p.meta_table ? p.meta_table[(size_t)b * p.meta_stride + mpg] : (int64_t)b * p.meta_stride + mpg;
        const bool ok = mpage >= 0 && mpage < p.num_meta_pages;
        float mx[VEC], mn[VEC];
        if (ok) {
            const char* m = p.meta + (size_t)mpage * 2 * p.meta_page_size * row + (size_t)ment * row + (size_t)h * D * sizeof(T) + (size_t)lane * 16;
            V::to_float(*reinterpret_cast<const uint4*>(m), mx);
            V::to_float(*reinterpret_cast<const uint4*>(m + (size_t)p.meta_page_size * row), mn);
        } else {
            if (lane == 0 && p.status) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
#pragma unroll
            for (int i = 0; i < VEC; ++i) mx[i] = mn[i] = 0.f;
        }
        for (int g = 0; g < G; ++g) {
            const int hq = h * G + g;
            const float* qh = qs + (size_t)hq * D + lane * VEC;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc += fmaxf(qh[i] * mx[i], qh[i] * mn[i]);
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(gmask, acc, o);
            if (lane == 0) {
                const size_t at = ((size_t)b * p.Hq + hq) * p.out_stride + e;
                if (p.out_dtype == TIDAL_DTYPE_F16) reinterpret_cast<__half*>(p.out)[at] = __float2half_rn(acc);
                else if (p.out_dtype == TIDAL_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(acc);
                else reinterpret_cast<float*>(p.out)[at] = acc;
            }
        }
    }
}

template <typename T>
static int launch_meta(const PageMetaParams& p, int D, cudaStream_t st) {
    const int vpr = D * (int)sizeof(T) / 16;
    const int64_t units = (int64_t)p.batch * p.n_pages * p.H * vpr;
    int64_t blocks = (units + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    cudaError_t e;
    if (D == 64) e = launch_pdl(page_meta_kernel<T, 64>, dim3((unsigned)blocks), dim3(256), 0, st, 1, p);
    else e = launch_pdl(page_meta_kernel<T, 128>, dim3((unsigned)blocks), dim3(256), 0, st, 1, p);
    TIDAL_CUDA_OK(e);
    count_launch();
    return TIDAL_OK;
}

template <typename T>
static int launch_estimate(const EstimateParams& p, int D, cudaStream_t st) {
    const int lpr = D * (int)sizeof(T) / 16;
    const int groups = 256 / lpr;
    const int64_t units = (int64_t)p.n_entries * p.H;
    int64_t blocks = (units + groups - 1) / groups;
    const int64_t cap = (148 * 8 + p.batch - 1) / p.batch;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const size_t smem = sizeof(float) * (size_t)p.Hq * D;
    cudaError_t e;
    if (D == 64) {
        TIDAL_CUDA_OK(cudaFuncSetAttribute(estimate_kernel<T, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        e = launch_pdl(estimate_kernel<T, 64>, dim3((unsigned)blocks, (unsigned)p.batch), dim3(256), smem, st, 1, p);
    } else {
        TIDAL_CUDA_OK(cudaFuncSetAttribute(estimate_kernel<T, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        e = launch_pdl(estimate_kernel<T, 128>, dim3((unsigned)blocks, (unsigned)p.batch), dim3(256), smem, st, 1, p);
    }
    TIDAL_CUDA_OK(e);
    count_launch();
    return TIDAL_OK;
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_update_page_meta(const tidal_page_meta_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_kv && a->d_meta, TIDAL_ERR_ARG, "the KV pool and the metadata pool must be given");
    TIDAL_REQUIRE((((uintptr_t)a->d_kv | (uintptr_t)a->d_meta) & 15) == 0, TIDAL_ERR_ARG, "pools must be 16-byte aligned");
    TIDAL_REQUIRE(a->batch >= 1 && a->num_kv_heads >= 1, TIDAL_ERR_ARG, "bad batch/heads");
    TIDAL_REQUIRE(a->head_dim == 64 || a->head_dim == 128, TIDAL_ERR_ARG, "unsupported head_dim %d (built: 64, 128)", a->head_dim);
    TIDAL_REQUIRE(a->page_size >= 1 && a->meta_page_size >= 1 && a->num_pages >= 1 && a->num_meta_pages >= 1, TIDAL_ERR_ARG,
                  "bad page sizes / pool sizes");
    TIDAL_REQUIRE(a->dtype >= 0 && a->dtype <= 2, TIDAL_ERR_ARG, "unknown dtype %d", a->dtype);
    TIDAL_REQUIRE(a->seq_len >= 1 && a->first_pos >= 0 && a->first_pos < a->seq_len, TIDAL_ERR_ARG,
                  "need 0 <= first_pos (%d) < seq_len (%d)", a->first_pos, a->seq_len);
    PageMetaParams p;
    p.kv = (const char*)a->d_kv; p.meta = (char*)a->d_meta;
    p.kv_table = a->d_page_table; p.meta_table = a->d_meta_table;
    p.kv_stride = a->page_table_stride; p.meta_stride = a->meta_table_stride;
    p.batch = a->batch; p.H = a->num_kv_heads; p.page_size = a->page_size; p.meta_page_size = a->meta_page_size;
    p.num_pages = a->num_pages; p.num_meta_pages = a->num_meta_pages;
    p.first_page = a->first_pos / a->page_size;
    p.n_pages = (a->seq_len - 1) / a->page_size - p.first_page + 1;
    p.seq_len = a->seq_len;
    p.status = a->d_status;
    cudaStream_t st = (cudaStream_t)stream;
    switch (a->dtype) {
        case TIDAL_DTYPE_F16: return launch_meta<__half>(p, a->head_dim, st);
        case TIDAL_DTYPE_BF16: return launch_meta<__nv_bfloat16>(p, a->head_dim, st);
        default: return launch_meta<float>(p, a->head_dim, st);
    }
}

extern "C" int tidal_estimate(const tidal_estimate_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_q && a->d_meta && a->d_out, TIDAL_ERR_ARG, "q, the metadata pool and the output must be given");
    TIDAL_REQUIRE((((uintptr_t)a->d_q | (uintptr_t)a->d_meta) & 15) == 0, TIDAL_ERR_ARG, "q and the pool must be 16-byte aligned");
    TIDAL_REQUIRE(a->batch >= 1 && a->num_qo_heads >= 1 && a->num_kv_heads >= 1 && a->num_qo_heads % a->num_kv_heads == 0,
                  TIDAL_ERR_ARG, "num_qo_heads %d is not a multiple of num_kv_heads %d", a->num_qo_heads, a->num_kv_heads);
    TIDAL_REQUIRE(a->head_dim == 64 || a->head_dim == 128, TIDAL_ERR_ARG, "unsupported head_dim %d (built: 64, 128)", a->head_dim);
    TIDAL_REQUIRE(a->meta_page_size >= 1 && a->num_meta_pages >= 1, TIDAL_ERR_ARG, "bad metadata page size / pool size");
    TIDAL_REQUIRE(a->dtype >= 0 && a->dtype <= 2 && a->out_dtype >= 0 && a->out_dtype <= 2, TIDAL_ERR_ARG, "unknown dtype");
    TIDAL_REQUIRE(a->n_entries >= 0 && a->out_stride >= a->n_entries, TIDAL_ERR_ARG, "out_stride shorter than n_entries");
    TIDAL_REQUIRE((size_t)a->num_qo_heads * a->head_dim * sizeof(float) <= 200 * 1024, TIDAL_ERR_ARG, "too many query heads");
    if (a->n_entries == 0) return TIDAL_OK;
    EstimateParams p;
    p.q = a->d_q; p.meta = (const char*)a->d_meta; p.meta_table = a->d_meta_table; p.meta_stride = a->meta_table_stride;
    p.out = a->d_out; p.out_stride = a->out_stride;
    p.batch = a->batch; p.Hq = a->num_qo_heads; p.H = a->num_kv_heads; p.meta_page_size = a->meta_page_size;
    p.n_entries = a->n_entries; p.out_dtype = a->out_dtype; p.num_meta_pages = a->num_meta_pages; p.status = a->d_status;
    cudaStream_t st = (cudaStream_t)stream;
    switch (a->dtype) {
        case TIDAL_DTYPE_F16: return launch_estimate<__half>(p, a->head_dim, st);
        case TIDAL_DTYPE_BF16: return launch_estimate<__nv_bfloat16>(p, a->head_dim, st);
        default: return launch_estimate<float>(p, a->head_dim, st);
    }
}
