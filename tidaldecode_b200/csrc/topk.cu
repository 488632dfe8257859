// Row-wise top-k of fp32 scores by radix selection.
//
// Keys are 64-bit and distinct: (order-preserving image of the score) << 32 |
// (0xFFFFFFFF - position), so the result is one well-defined set — equal scores
// resolve towards the lower position — and every rank that sees the same scores
// selects the same tokens.
//
//   digit 0   histogram of the top 12 key bits of the row.  The attention kernel
//             can count the logits while it writes them; otherwise it is built here.
//   split     the threshold bin b* is read off the histogram; keys in higher bins
//             are certainly selected (`sel`), keys in b* are candidates (`cand`).
//   resolve   8-bit radix passes over the remaining 52 bits of the candidates,
//             stopping as soon as a digit's population equals what is still needed.
//   emit      winners ordered by position, ownership filter, outputs, counters
//             back to zero.
//
// Usual case (k <= kClusterMaxK, rows up to kClusterMaxN): ONE launch, one
// thread-block cluster of up to 8 CTAs per row.  Every CTA scans a slice of the
// row and pushes what it finds into the shared memory of the cluster's first CTA
// through distributed shared memory; after one cluster barrier that CTA resolves,
// orders and emits without touching global memory again.  Larger problems split
// the histogram and the scan over many independent CTAs per row with lists in
// global memory (block-then-global) and finish with one CTA per row.
#include <cstdlib>
#include <mutex>

#include "topk_common.cuh"

namespace tidal {

__global__ void __launch_bounds__(kTopkThreads) topk_hist_kernel(const TopkParams p) {
    __shared__ uint32_t h[kBins];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.y;
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const float* s = p.scores + (size_t)row * p.row_stride;
    const int64_t per = (p.n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per, hi = min(p.n, lo + per);
#pragma unroll 4
    for (int64_t j = lo + threadIdx.x; j < hi; j += blockDim.x)
        atomicAdd(&h[key_bin(make_key(s[j], (uint32_t)j, p.n, p.force_last))], 1u);
    __syncthreads();
    for (int i = threadIdx.x; i < kBins; i += blockDim.x)
        if (h[i]) atomicAdd(&p.hist[(size_t)row * kBins + i], h[i]);
}

// Scan positions [lo, hi) of a row and append to `sel` / `cand`; counters may
// live in shared or global memory.
__device__ __forceinline__ void split_range(const TopkParams& p, int row, int64_t lo, int64_t hi, int bstar,
                                            uint32_t* sel_cnt, uint32_t* cand_cnt) {
    const float* s = p.scores + (size_t)row * p.row_stride;
    uint64_t* sel = p.sel + (size_t)row * kMaxK;
    uint64_t* cand = p.cand + (size_t)row * p.cand_cap;
#pragma unroll 4
    for (int64_t j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        const uint64_t key = make_key(s[j], (uint32_t)j, p.n, p.force_last);
        const int bin = key_bin(key);
        if (bin > bstar) {
            const uint32_t at = append_slot(sel_cnt);
            if (at < (uint32_t)kMaxK) sel[at] = key;
        } else if (bin == bstar) {
            const uint32_t at = append_slot(cand_cnt);
            if ((int64_t)at < p.cand_cap) cand[at] = key;
        }
    }
}

__global__ void __launch_bounds__(kTopkThreads) topk_partition_kernel(const TopkParams p) {
    __shared__ uint32_t h[kBins];
    __shared__ uint32_t ws[32];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.y;
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) h[i] = p.hist[(size_t)row * kBins + i];
    __syncthreads();
    int bstar;
    uint32_t above;
    find_threshold_bin(h, ws, (uint32_t)p.k, &bstar, &above);
    uint32_t* st = p.row_state + (size_t)row * 8;
    const int64_t per = (p.n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per;
    split_range(p, row, lo, min(p.n, lo + per), bstar, &st[0], &st[1]);
}

// Iterate the candidates of a row: the compacted list, or — if it overflowed —
// the score row itself filtered by the threshold bin.
template <typename F>
__device__ __forceinline__ void for_each_candidate(const TopkParams& p, int row, int bstar, uint32_t ncand, bool overflow, F f) {
    if (!overflow) {
        const uint64_t* cand = p.cand + (size_t)row * p.cand_cap;
        for (uint32_t j = threadIdx.x; j < ncand; j += blockDim.x) f(cand[j]);
    } else {
        const float* s = p.scores + (size_t)row * p.row_stride;
        for (int64_t j = threadIdx.x; j < p.n; j += blockDim.x) {
            const uint64_t key = make_key(s[j], (uint32_t)j, p.n, p.force_last);
            if (key_bin(key) == bstar) f(key);
        }
    }
}

// FUSED: the CTA also builds the histogram (unless one is supplied) and splits the row.
// select_all: k >= n, every position is emitted in order.
template <bool FUSED>
__global__ void __launch_bounds__(kTopkThreads) topk_finish_kernel(const TopkParams p, int select_all) {
    // `h` (threshold search, then the per-pass digit histograms) is dead before the
    // winners are collected, so both live in one 32 KB array.
    __shared__ uint64_t winners[kSortMax];
    uint32_t* h = reinterpret_cast<uint32_t*>(winners);
    static_assert(sizeof(uint64_t) * kSortMax >= sizeof(uint32_t) * kBins, "winners must cover the histogram");
    __shared__ uint32_t ws[32];
    __shared__ uint32_t s_cnt, s_digit, s_need, s_done, s_nsel, s_ncand;
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int t = threadIdx.x;
    uint32_t* st = FUSED ? nullptr : p.row_state + (size_t)row * 8;     // the fused form keeps its counters in shared memory
    const float* srow = p.scores + (size_t)row * p.row_stride;
    const uint32_t k = (uint32_t)p.k;
    int32_t* out_idx = p.out_idx + (size_t)row * p.out_stride;
    float* out_val = p.out_val ? p.out_val + (size_t)row * p.out_stride : nullptr;
    const bool own = p.own_hi > p.own_lo;

    auto emit_value = [&](uint32_t pos) -> int32_t {
        return p.in_idx ? p.in_idx[(size_t)row * p.in_idx_stride + pos] : (int32_t)pos + p.idx_offset;
    };
    // Order-preserving emission of `count` items; item j is described by get(j, &pos, &score)
    // returning false for padding.
    auto emit_ordered = [&](uint32_t count, auto get) {
        uint32_t before = 0;
        for (uint32_t base = 0; base < count; base += kTopkThreads) {
            const uint32_t j = base + t;
            int32_t v = 0;
            float sc = 0.f;
            bool keep = false;
            uint32_t pos = 0;
            if (j < count && get(j, &pos, &sc)) {
                v = emit_value(pos);
                keep = !own || (v >= p.own_lo && v < p.own_hi);
            }
            const uint32_t incl = block_scan_incl(keep ? 1u : 0u, ws);
            if (keep) {
                const uint32_t at = before + incl - 1;
                out_idx[at] = own ? v - p.own_lo : v;
                if (out_val) out_val[at] = sc;
            }
            if (t == kTopkThreads - 1) s_cnt = before + incl;
            __syncthreads();
            before = s_cnt;
            __syncthreads();
        }
        if (t == 0 && p.out_count) p.out_count[row] = (int32_t)before;
    };

    if (select_all) {
        emit_ordered(k, [&](uint32_t j, uint32_t* pos, float* sc) { *pos = j; *sc = srow[j]; return true; });
        // a histogram the attention kernel filled for this row is not needed: clear it
        if (p.hist)
            for (int i = t; i < kBins; i += kTopkThreads) p.hist[(size_t)row * kBins + i] = 0;
        return;
    }

    // ---- digit-0 histogram into shared memory
    if (p.hist) {
        for (int i = t; i < kBins; i += kTopkThreads) h[i] = p.hist[(size_t)row * kBins + i];
    } else {
        for (int i = t; i < kBins; i += kTopkThreads) h[i] = 0;
        __syncthreads();
#pragma unroll 4
        for (int64_t j = t; j < p.n; j += kTopkThreads)
            atomicAdd(&h[key_bin(make_key(srow[j], (uint32_t)j, p.n, p.force_last))], 1u);
    }
    __syncthreads();
    int bstar;
    uint32_t above;
    find_threshold_bin(h, ws, k, &bstar, &above);

    // ---- split (fused) or pick up the counts the partition kernel left
    if (FUSED) {
        if (t == 0) { s_nsel = 0; s_ncand = 0; }
        __syncthreads();
        split_range(p, row, 0, p.n, bstar, &s_nsel, &s_ncand);
        __syncthreads();
    } else {
        if (t == 0) { s_nsel = st[0]; s_ncand = st[1]; }
        __syncthreads();
    }
    const uint32_t nsel = min(s_nsel, (uint32_t)kMaxK);
    const uint32_t ncand_total = s_ncand;
    const bool overflow = (int64_t)ncand_total > p.cand_cap;
    uint32_t need = k - above;                 // how many candidates win (>= 1)
    if (s_nsel != above && t == 0) atomicOr(p.status, TIDAL_DEV_TOPK_OVERFLOW);

    // ---- radix passes over key bits 51..0 among the candidates
    uint64_t prefix = (uint64_t)bstar << 52;   // known high bits
    uint64_t known_mask = 0xFFFull << 52;
    bool done = (need == ncand_total);         // all candidates win
    for (int shift = 44; !done && shift >= -4; shift -= 8) {
        const int sh = shift < 0 ? 0 : shift;
        const int nb = shift < 0 ? 16 : 256;
        const uint32_t dmask = (uint32_t)nb - 1u;
        if (t < 256) h[t] = 0;
        __syncthreads();
        for_each_candidate(p, row, bstar, ncand_total, overflow, [&](uint64_t key) {
            if ((key & known_mask) == prefix) count_digit(h, (uint32_t)(key >> sh) & dmask);
        });
        __syncthreads();
        if (t < 32) warp_find_digit(h, nb, need, &s_digit, &s_need, &s_done);
        __syncthreads();
        prefix |= (uint64_t)s_digit << sh;
        known_mask |= (uint64_t)dmask << sh;
        need = s_need;
        done = s_done != 0;
        __syncthreads();
    }
    const uint64_t thr = prefix;               // winners among candidates: key >= thr

    // ---- collect the k winners
    if (t == 0) s_cnt = 0;
    __syncthreads();
    const uint64_t* sel = p.sel + (size_t)row * kMaxK;
    if (k <= (uint32_t)kSortMax) {
        // as (position << 32 | score bits), so that an ascending order is the position order
        auto push = [&](uint64_t key) {
            const uint32_t pos = key_pos(key);
            winners[atomicAdd(&s_cnt, 1u) % kSortMax] = ((uint64_t)pos << 32) | (uint64_t)__float_as_uint(srow[pos]);
        };
        for (uint32_t j = t; j < nsel; j += kTopkThreads) push(sel[j]);
        for_each_candidate(p, row, bstar, ncand_total, overflow, [&](uint64_t key) {
            if (key >= thr) push(key);
        });
        __syncthreads();
        const uint32_t got = min(s_cnt, k);
        if (s_cnt != k && t == 0) atomicOr(p.status, TIDAL_DEV_TOPK_OVERFLOW);
        if (k <= (uint32_t)kRankSortMax) {
            // rank by counting: thread j finds how many winners precede its own
            uint64_t mine = ~0ull;
            uint32_t rank = 0;
            if ((uint32_t)t < got) {
                mine = winners[t];
                for (uint32_t i = 0; i < got; ++i) rank += (winners[i] < mine) ? 1u : 0u;
            }
            __syncthreads();
            if ((uint32_t)t < got) winners[rank] = mine;
            __syncthreads();
        } else {
            uint32_t np2 = 1;
            while (np2 < k) np2 <<= 1;
            for (uint32_t j = got + t; j < np2; j += kTopkThreads) winners[j] = ~0ull;
            __syncthreads();
            for (uint32_t size = 2; size <= np2; size <<= 1) {
                for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
                    for (uint32_t j = t; j < np2 / 2; j += kTopkThreads) {
                        const uint32_t lo = 2 * j - (j & (stride - 1));
                        const uint32_t hi = lo + stride;
                        const bool asc = ((lo & size) == 0);
                        const uint64_t a = winners[lo], b = winners[hi];
                        if ((a > b) == asc) { winners[lo] = b; winners[hi] = a; }
                    }
                    __syncthreads();
                }
            }
        }
        emit_ordered(got, [&](uint32_t j, uint32_t* pos, float* sc) {
            const uint64_t w = winners[j];
            *pos = (uint32_t)(w >> 32);
            *sc = __uint_as_float((uint32_t)(w & 0xFFFFFFFFull));
            return true;
        });
    } else {
        // large k: unordered emission straight to the output
        auto put = [&](uint64_t key) {
            const uint32_t pos = key_pos(key);
            const int32_t v = emit_value(pos);
            if (own && !(v >= p.own_lo && v < p.own_hi)) return;
            const uint32_t at = atomicAdd(&s_cnt, 1u);
            if (at < k) {
                out_idx[at] = own ? v - p.own_lo : v;
                if (out_val) out_val[at] = srow[pos];
            }
        };
        for (uint32_t j = t; j < nsel; j += kTopkThreads) put(sel[j]);
        for_each_candidate(p, row, bstar, ncand_total, overflow, [&](uint64_t key) {
            if (key >= thr) put(key);
        });
        __syncthreads();
        if (t == 0 && p.out_count) p.out_count[row] = (int32_t)min(s_cnt, k);
    }

    // ---- leave the global counters zero at rest
    if (p.hist)
        for (int i = t; i < kBins; i += kTopkThreads) p.hist[(size_t)row * kBins + i] = 0;
    if (!FUSED && t < 8) st[t] = 0;
}


// The one-launch path: one cluster of up to 8 CTAs per row (topk_cluster_row, topk_common.cuh).
__global__ void __launch_bounds__(kTopkThreads) topk_cluster_kernel(const TopkParams p) {
    extern __shared__ __align__(16) unsigned char csm[];
    pdl_wait();
    pdl_launch_dependents();
    topk_cluster_row(p, (int)(blockIdx.x / cg::this_cluster().num_blocks()), csm);
}

// Largest cluster the one-launch path uses per row (8).  TIDAL_TOPK_MAX_CLUSTER=1|2|4|8 in the environment
// lowers it — a tuning knob for measurements, read once.
static int topk_max_cluster() {
    static int v = 0;
    if (v == 0) {
        v = 8;
        if (const char* e = std::getenv("TIDAL_TOPK_MAX_CLUSTER")) {
            const int x = std::atoi(e);
            if (x == 1 || x == 2 || x == 4 || x == 8) v = x;
        }
    }
    return v;
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_topk(const tidal_topk_args* a, void* d_ws, size_t ws_bytes, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_scores && a->d_out_idx, TIDAL_ERR_ARG, "scores and out_idx must be given");
    TIDAL_REQUIRE(a->rows >= 1 && a->n >= 1 && a->k >= 1, TIDAL_ERR_ARG, "rows, n and k must be positive (rows %d n %lld k %d)",
                  a->rows, (long long)a->n, a->k);
    TIDAL_REQUIRE(a->n <= 0x7FFFFFFFll, TIDAL_ERR_ARG, "row length %lld does not fit int32 positions", (long long)a->n);
    TIDAL_REQUIRE(a->seg_len > 0 || a->row_stride >= a->n, TIDAL_ERR_ARG, "row_stride shorter than n");
    TIDAL_REQUIRE(a->seg_len > 0 || a->d_in_idx == nullptr || a->in_idx_stride == 0 || a->in_idx_stride >= a->n, TIDAL_ERR_ARG,
                  "in_idx_stride must be 0 (shared row) or at least n");
    const int k = (int64_t)a->k < a->n ? a->k : (int)a->n;
    TIDAL_REQUIRE(k <= kMaxK || (int64_t)a->k >= a->n, TIDAL_ERR_ARG, "k %d exceeds the built maximum %d", k, kMaxK);
    TIDAL_REQUIRE(a->out_stride >= k, TIDAL_ERR_ARG, "out_stride %lld shorter than min(k, n) = %d", (long long)a->out_stride, k);
    const WsLayout* L = find_ws(d_ws);
    TIDAL_REQUIRE(L != nullptr, TIDAL_ERR_WORKSPACE, "workspace %p was not initialised with tidal_ws_init", d_ws);
    TIDAL_REQUIRE(ws_bytes >= L->total, TIDAL_ERR_WORKSPACE, "workspace is %zu bytes, layout needs %zu", ws_bytes, L->total);
    const size_t rows_cap = (L->row_state_off - L->hist_off) / (sizeof(uint32_t) * kBins);
    TIDAL_REQUIRE((size_t)a->rows <= rows_cap, TIDAL_ERR_WORKSPACE, "workspace was sized for %zu rows, call has %d", rows_cap, a->rows);

    TopkParams p;
    p.scores = a->d_scores; p.in_idx = a->d_in_idx; p.in_idx_stride = a->in_idx_stride; p.rows = a->rows; p.n = a->n; p.row_stride = a->row_stride;
    p.k = k; p.out_idx = a->d_out_idx; p.out_val = a->d_out_val; p.out_stride = a->out_stride;
    p.idx_offset = a->idx_offset; p.force_last = a->force_last; p.own_lo = a->own_lo; p.own_hi = a->own_hi;
    p.out_count = a->d_out_count;
    p.hist = a->d_hist;
    p.row_state = (uint32_t*)((char*)d_ws + L->row_state_off);
    p.cand = (uint64_t*)((char*)d_ws + L->cand_off);
    p.sel = (uint64_t*)((char*)d_ws + L->sel_off);
    p.cand_cap = L->cand_cap;
    p.status = (uint32_t*)((char*)d_ws + L->status_off);
    p.seg_len = a->seg_len; p.seg_stride = a->seg_stride; p.row_len = a->d_row_len;
    TIDAL_REQUIRE(a->seg_len >= 0, TIDAL_ERR_ARG, "negative seg_len");
    TIDAL_REQUIRE(a->d_row_len == nullptr || ((int64_t)a->k < a->n && k <= kClusterMaxK && a->n <= kClusterMaxN), TIDAL_ERR_ARG,
                  "device-side row lengths need k < n (the bound), k <= %d and n <= %lld", kClusterMaxK, (long long)kClusterMaxN);
    TIDAL_REQUIRE(a->seg_len == 0 || ((int64_t)a->k < a->n && k <= kClusterMaxK && a->n <= kClusterMaxN), TIDAL_ERR_ARG,
                  "segmented rows need k < n, k <= %d and n <= %lld", kClusterMaxK, (long long)kClusterMaxN);
    cudaStream_t st = (cudaStream_t)stream;

    if ((int64_t)a->k >= a->n) {
        TIDAL_CUDA_OK(launch_pdl(topk_finish_kernel<true>, dim3(a->rows), dim3(kTopkThreads), 0, st, 1, p, 1));
        count_launch();
        return TIDAL_OK;
    }
    if (k <= kClusterMaxK && a->n <= kClusterMaxN) {
        // one cluster per row; 8 CTAs unless the row is short
        int cs = topk_max_cluster();
        while (cs > 1 && a->n < (int64_t)cs * 2048) cs >>= 1;
        // per launch, like every other kernel here: the attribute belongs to the current device, and a process
        // may drive several
        TIDAL_CUDA_OK(cudaFuncSetAttribute(topk_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kClusterSmem));
        TIDAL_CUDA_OK(launch_pdl(topk_cluster_kernel, dim3((unsigned)(a->rows * cs)), dim3(kTopkThreads), kClusterSmem, st,
                                 (unsigned)cs, p));
        count_launch();
        return TIDAL_OK;
    }
    if (a->n <= kFusedMaxN) {
        TIDAL_CUDA_OK(launch_pdl(topk_finish_kernel<true>, dim3(a->rows), dim3(kTopkThreads), 0, st, 1, p, 0));
        count_launch();
        return TIDAL_OK;
    }
    // long rows: many CTAs per row for the histogram and the split
    if (!p.hist) p.hist = (uint32_t*)((char*)d_ws + L->hist_off);
    int nblk = (int)((a->n + 16383) / 16384);
    const int max_blk = (2 * 148 + a->rows - 1) / a->rows;
    if (nblk > max_blk) nblk = max_blk;
    if (nblk < 1) nblk = 1;
    if (!a->d_hist) {
        TIDAL_CUDA_OK(launch_pdl(topk_hist_kernel, dim3(nblk, a->rows), dim3(kTopkThreads), 0, st, 1, p));
        count_launch();
    }
    TIDAL_CUDA_OK(launch_pdl(topk_partition_kernel, dim3(nblk, a->rows), dim3(kTopkThreads), 0, st, 1, p));
    count_launch();
    TIDAL_CUDA_OK(launch_pdl(topk_finish_kernel<false>, dim3(a->rows), dim3(kTopkThreads), 0, st, 1, p, 0));
    count_launch();
    return TIDAL_OK;
}

// ------------------------------------------------- allocation-free entry point
// tidal_topk_static: the one-CTA-per-row kernel above (topk_finish_kernel<true>) with
// its `sel` / `cand` lists and fault word in a fixed array that is part of the loaded
// library image instead of a caller-supplied workspace.  Every call on a device shares
// the array.
namespace tidal {

constexpr int kStaticRows = 8;                 // rows per call
constexpr int64_t kStaticCand = 16384;         // candidate slots per row (more candidates: the kernel rescans the row)
constexpr int64_t kStaticMaxN = kFusedMaxN;    // longest row
constexpr int kStaticMaxK = kMaxK;

struct StaticTopkScratch {
    uint32_t status[64];                       // [0]: TIDAL_DEV_* bits, sticky
    uint64_t sel[kStaticRows][kMaxK];
    uint64_t cand[kStaticRows][kStaticCand];
};

// ~2 MB per GPU that loads the library, held until the process exits.
static __device__ __align__(256) unsigned char g_static_topk_scratch[sizeof(StaticTopkScratch)];

// In host code the name above is only a handle for the runtime, never a device address:
// the address is looked up once per device and cached here.
static std::mutex g_static_mu;
static StaticTopkScratch* g_static_ptr[64] = {};

static int static_scratch_for_current_device(StaticTopkScratch** out) {
    int dev = -1;
    TIDAL_CUDA_OK(cudaGetDevice(&dev));
    TIDAL_REQUIRE(dev >= 0 && dev < 64, TIDAL_ERR_ARG, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        TIDAL_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_topk_scratch));
        TIDAL_REQUIRE(ptr != nullptr, TIDAL_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_static_ptr[dev] = static_cast<StaticTopkScratch*>(ptr);
    }
    *out = g_static_ptr[dev];
    return TIDAL_OK;
}

}  // namespace tidal

extern "C" int tidal_topk_static(const tidal_topk_args* a, uint32_t* d_status, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_scores && a->d_out_idx, TIDAL_ERR_ARG, "scores and out_idx must be given");
    TIDAL_REQUIRE(a->rows >= 1 && a->n >= 1 && a->k >= 1, TIDAL_ERR_ARG, "rows, n and k must be positive (rows %d n %lld k %d)",
                  a->rows, (long long)a->n, a->k);
    TIDAL_REQUIRE(a->rows <= kStaticRows, TIDAL_ERR_ARG, "tidal_topk_static takes at most %d rows per call, got %d", kStaticRows,
                  a->rows);
    TIDAL_REQUIRE(a->n <= kStaticMaxN, TIDAL_ERR_ARG, "tidal_topk_static takes rows of at most %lld scores, got %lld",
                  (long long)kStaticMaxN, (long long)a->n);
    TIDAL_REQUIRE(a->row_stride >= a->n, TIDAL_ERR_ARG, "row_stride shorter than n");
    TIDAL_REQUIRE(a->d_in_idx == nullptr || a->in_idx_stride == 0 || a->in_idx_stride >= a->n, TIDAL_ERR_ARG,
                  "in_idx_stride must be 0 (shared row) or at least n");
    TIDAL_REQUIRE(a->d_hist == nullptr, TIDAL_ERR_ARG, "tidal_topk_static builds its own histogram: d_hist must be NULL");
    TIDAL_REQUIRE(a->seg_len == 0 && a->seg_stride == 0, TIDAL_ERR_ARG,
                  "tidal_topk_static takes contiguous rows only: seg_len and seg_stride must be 0");
    TIDAL_REQUIRE(a->d_row_len == nullptr, TIDAL_ERR_ARG, "tidal_topk_static takes the row length from n: d_row_len must be NULL");
    const int k = (int64_t)a->k < a->n ? a->k : (int)a->n;
    TIDAL_REQUIRE(k <= kStaticMaxK || (int64_t)a->k >= a->n, TIDAL_ERR_ARG, "tidal_topk_static takes k of at most %d, got %d",
                  kStaticMaxK, k);
    TIDAL_REQUIRE(a->out_stride >= k, TIDAL_ERR_ARG, "out_stride %lld shorter than min(k, n) = %d", (long long)a->out_stride, k);
    StaticTopkScratch* sc = nullptr;
    const int rc = static_scratch_for_current_device(&sc);
    if (rc != TIDAL_OK) return rc;

    TopkParams p;
    p.scores = a->d_scores; p.in_idx = a->d_in_idx; p.in_idx_stride = a->in_idx_stride; p.rows = a->rows; p.n = a->n;
    p.row_stride = a->row_stride; p.k = k; p.out_idx = a->d_out_idx; p.out_val = a->d_out_val; p.out_stride = a->out_stride;
    p.idx_offset = a->idx_offset; p.force_last = a->force_last; p.own_lo = a->own_lo; p.own_hi = a->own_hi;
    p.out_count = a->d_out_count;
    p.hist = nullptr;                       // the kernel counts the first digit in shared memory
    p.row_state = nullptr;                  // its list counters live in shared memory too: nothing to clear between calls
    p.cand = &sc->cand[0][0];
    p.sel = &sc->sel[0][0];
    p.cand_cap = kStaticCand;
    p.status = d_status ? d_status : &sc->status[0];
    p.seg_len = 0; p.seg_stride = 0; p.row_len = nullptr;
    topk_finish_kernel<true><<<a->rows, kTopkThreads, 0, (cudaStream_t)stream>>>(p, (int64_t)a->k >= a->n ? 1 : 0);
    TIDAL_CUDA_OK(cudaGetLastError());
    count_launch();
    return TIDAL_OK;
}

extern "C" int tidal_topk_static_status(int clear, void* stream) {
    StaticTopkScratch* sc = nullptr;
    const int rc = static_scratch_for_current_device(&sc);
    if (rc != TIDAL_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t bits = 0;
    TIDAL_CUDA_OK(cudaMemcpyAsync(&bits, &sc->status[0], sizeof(bits), cudaMemcpyDeviceToHost, st));
    TIDAL_CUDA_OK(cudaStreamSynchronize(st));
    if (clear && bits) TIDAL_CUDA_OK(cudaMemsetAsync(&sc->status[0], 0, sizeof(uint32_t), st));
    return (int)(bits & 0x7fffffffu);
}
