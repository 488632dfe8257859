// Row-wise top-k of fp32 scores by radix selection, block-then-global.
//
// Keys are 64-bit and distinct: (order-preserving image of the score) << 32 |
// (0xFFFFFFFF - position), so the result is one well-defined set — equal scores
// resolve towards the lower position — and every rank that sees the same scores
// selects the same tokens.
//
//   pass 0  histogram of the top 12 key bits over the whole row, many CTAs per
//           row (skipped when the attention kernel already counted the logits
//           while it wrote them);
//   pass 1  every CTA finds the threshold bin from the histogram and scans its
//           slice: keys in higher bins are certainly selected (appended to
//           `sel`), keys in the threshold bin become candidates (`cand`);
//   pass 2  one CTA per row resolves the candidates with 8-bit radix passes over
//           the remaining 52 bits, orders the k winners by position, applies the
//           ownership filter, writes the outputs and re-zeroes the counters.
#include "common.cuh"

namespace tidal {

constexpr int kBins = TIDAL_TOPK_BINS;
constexpr int kTopkThreads = 1024;
constexpr int kSortMax = 4096;   // winners are position-sorted up to this k

struct TopkParams {
    const float* scores;
    const int32_t* in_idx;
    int64_t in_idx_stride;
    int32_t rows;
    int64_t n, row_stride;
    int32_t k;            // already min(k, n)
    int32_t* out_idx;
    float* out_val;
    int64_t out_stride;
    int32_t idx_offset, force_last, own_lo, own_hi;
    int32_t* out_count;
    uint32_t* hist;       // [rows][kBins]
    uint32_t* row_state;  // [rows][8]: 0 sel count, 1 cand count
    uint64_t* cand;       // [rows][cand_cap]
    uint64_t* sel;        // [rows][kMaxK]
    int64_t cand_cap;
    uint32_t* status;
};

__device__ __forceinline__ uint64_t make_key(float s, uint32_t pos, int64_t n, int force_last) {
    uint32_t k32 = ordered_key(s);
    if (force_last && (int64_t)pos == n - 1) k32 = 0xFFFFFFFFu;
    return ((uint64_t)k32 << 32) | (uint64_t)(0xFFFFFFFFu - pos);
}
__device__ __forceinline__ uint32_t key_pos(uint64_t key) { return 0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull); }

__global__ void __launch_bounds__(kTopkThreads) topk_hist_kernel(const TopkParams p) {
    __shared__ uint32_t h[kBins];
    const int row = blockIdx.y;
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const float* s = p.scores + (size_t)row * p.row_stride;
    const int64_t per = (p.n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per, hi = min(p.n, lo + per);
    for (int64_t j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        const uint64_t key = make_key(s[j], (uint32_t)j, p.n, p.force_last);
        atomicAdd(&h[(uint32_t)(key >> 32) >> kDigit0Shift], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins; i += blockDim.x)
        if (h[i]) atomicAdd(&p.hist[(size_t)row * kBins + i], h[i]);
}

// Threshold bin b*: count(bins > b*) < k <= count(bins >= b*).  Every thread of
// the block returns the same (bin, above).  `h` is a shared copy of the row's
// histogram, `scratch` has blockDim.x words.
__device__ void find_threshold_bin(const uint32_t* h, uint32_t* scratch, uint32_t k, int* bin_out, uint32_t* above_out) {
    // each thread owns kBins/blockDim.x consecutive bins, highest bins first
    const int per = kBins / kTopkThreads;     // 4
    const int t = threadIdx.x;
    uint32_t mine = 0;
    const int base = kBins - (t + 1) * per;    // thread 0 owns the top bins
#pragma unroll
    for (int i = 0; i < per; ++i) mine += h[base + i];
    scratch[t] = mine;
    __syncthreads();
    // inclusive scan over threads (Hillis-Steele)
    for (int off = 1; off < kTopkThreads; off <<= 1) {
        uint32_t v = (t >= off) ? scratch[t - off] : 0;
        __syncthreads();
        scratch[t] += v;
        __syncthreads();
    }
    __shared__ int s_bin;
    __shared__ uint32_t s_above;
    if (t == 0) { s_bin = 0; s_above = 0; }
    __syncthreads();
    const uint32_t incl = scratch[t], excl = incl - mine;
    if (excl < k && k <= incl) {
        uint32_t above = excl;
        for (int i = per - 1; i >= 0; --i) {
            const uint32_t c = h[base + i];
            if (above + c >= k) { s_bin = base + i; s_above = above; break; }
            above += c;
        }
    }
    __syncthreads();
    *bin_out = s_bin;
    *above_out = s_above;
    __syncthreads();
}

__global__ void __launch_bounds__(kTopkThreads) topk_partition_kernel(const TopkParams p) {
    __shared__ uint32_t h[kBins];
    __shared__ uint32_t scratch[kTopkThreads];
    const int row = blockIdx.y;
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) h[i] = p.hist[(size_t)row * kBins + i];
    __syncthreads();
    int bstar;
    uint32_t above;
    find_threshold_bin(h, scratch, (uint32_t)p.k, &bstar, &above);
    const float* s = p.scores + (size_t)row * p.row_stride;
    uint32_t* st = p.row_state + (size_t)row * 8;
    uint64_t* sel = p.sel + (size_t)row * kMaxK;
    uint64_t* cand = p.cand + (size_t)row * p.cand_cap;
    const int64_t per = (p.n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per, hi = min(p.n, lo + per);
    for (int64_t j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        const uint64_t key = make_key(s[j], (uint32_t)j, p.n, p.force_last);
        const int bin = (int)((uint32_t)(key >> 32) >> kDigit0Shift);
        if (bin > bstar) {
            const uint32_t at = atomicAdd(&st[0], 1u);
            if (at < (uint32_t)kMaxK) sel[at] = key;
        } else if (bin == bstar) {
            const uint32_t at = atomicAdd(&st[1], 1u);
            if ((int64_t)at < p.cand_cap) cand[at] = key;
        }
    }
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
            if ((int)((uint32_t)(key >> 32) >> kDigit0Shift) == bstar) f(key);
        }
    }
}

__global__ void __launch_bounds__(kTopkThreads) topk_finish_kernel(const TopkParams p, int select_all) {
    // `h` (threshold search, then the 256-bin pass histograms) is dead before the
    // winners are collected, so both live in one 32 KB array.
    __shared__ uint64_t winners[kSortMax];
    uint32_t* h = reinterpret_cast<uint32_t*>(winners);
    static_assert(sizeof(uint64_t) * kSortMax >= sizeof(uint32_t) * kBins, "winners must cover the histogram");
    __shared__ uint32_t scratch[kTopkThreads];
    __shared__ uint32_t s_cnt, s_digit, s_need, s_done;
    const int row = blockIdx.x;
    const int t = threadIdx.x;
    uint32_t* st = p.row_state + (size_t)row * 8;
    const float* srow = p.scores + (size_t)row * p.row_stride;
    const uint32_t k = (uint32_t)p.k;
    const bool sorted = k <= (uint32_t)kSortMax;
    int32_t* out_idx = p.out_idx + (size_t)row * p.out_stride;
    float* out_val = p.out_val ? p.out_val + (size_t)row * p.out_stride : nullptr;
    const bool own = p.own_hi > p.own_lo;

    auto emit_value = [&](uint32_t pos) -> int32_t {
        return p.in_idx ? p.in_idx[(size_t)row * p.in_idx_stride + pos] : (int32_t)pos + p.idx_offset;
    };

    if (select_all) {
        // k >= n: every position is selected, already in ascending order
        if (t == 0) s_cnt = 0;
        __syncthreads();
        for (uint32_t base = 0; base < k; base += blockDim.x) {
            const uint32_t j = base + t;
            int32_t v = 0;
            bool keep = false;
            if (j < k) {
                v = emit_value(j);
                keep = !own || (v >= p.own_lo && v < p.own_hi);
            }
            // order-preserving compaction, one tile of blockDim.x at a time
            scratch[t] = keep ? 1u : 0u;
            __syncthreads();
            for (int off = 1; off < kTopkThreads; off <<= 1) {
                uint32_t x = (t >= off) ? scratch[t - off] : 0;
                __syncthreads();
                scratch[t] += x;
                __syncthreads();
            }
            const uint32_t before = s_cnt;
            if (keep) {
                const uint32_t at = before + scratch[t] - 1;
                out_idx[at] = own ? v - p.own_lo : v;
                if (out_val) out_val[at] = srow[j];
            }
            __syncthreads();
            if (t == kTopkThreads - 1) s_cnt = before + scratch[t];
            __syncthreads();
        }
        if (t == 0 && p.out_count) p.out_count[row] = (int32_t)s_cnt;
        // a histogram the attention kernel filled for this row is not needed: clear it
        for (int i = t; i < kBins; i += blockDim.x) p.hist[(size_t)row * kBins + i] = 0;
        return;
    }

    for (int i = t; i < kBins; i += blockDim.x) h[i] = p.hist[(size_t)row * kBins + i];
    __syncthreads();
    int bstar;
    uint32_t above;
    find_threshold_bin(h, scratch, k, &bstar, &above);
    const uint32_t nsel = min(st[0], (uint32_t)kMaxK);
    const uint32_t ncand_total = st[1];
    const bool overflow = (int64_t)ncand_total > p.cand_cap;
    uint32_t need = k - above;                 // how many candidates win (>= 1)
    if (nsel != above && t == 0) atomicOr(p.status, TIDAL_DEV_TOPK_OVERFLOW);

    // ---- radix passes over key bits 51..0 among the candidates
    uint64_t prefix = (uint64_t)bstar << 52;   // known high bits
    uint64_t known_mask = 0xFFFull << 52;
    bool done = (need == ncand_total);         // all candidates win
    for (int shift = 44; !done && shift >= -4; shift -= 8) {
        const int sh = shift < 0 ? 0 : shift;
        const int bits = shift < 0 ? 4 : 8;
        const uint32_t dmask = (1u << bits) - 1u;
        for (int i = t; i < 256; i += blockDim.x) h[i] = 0;
        __syncthreads();
        for_each_candidate(p, row, bstar, ncand_total, overflow, [&](uint64_t key) {
            if ((key & known_mask) == prefix) atomicAdd(&h[(uint32_t)(key >> sh) & dmask], 1u);
        });
        __syncthreads();
        if (t == 0) {
            uint32_t acc = 0;
            int d = (int)dmask;
            for (; d > 0; --d) {
                if (acc + h[d] >= need) break;
                acc += h[d];
            }
            s_digit = (uint32_t)d;
            s_need = need - acc;
            s_done = (h[d] == need - acc) ? 1u : 0u;
        }
        __syncthreads();
        prefix |= (uint64_t)s_digit << sh;
        known_mask |= (uint64_t)dmask << sh;
        need = s_need;
        done = s_done != 0;
        __syncthreads();
    }
    // winners among candidates: keys >= prefix (unknown low bits zero)
    const uint64_t thr = prefix;

    // ---- collect the k winners
    if (t == 0) s_cnt = 0;
    __syncthreads();
    const uint64_t* sel = p.sel + (size_t)row * kMaxK;
    if (sorted) {
        for (uint32_t j = t; j < nsel; j += blockDim.x) winners[atomicAdd(&s_cnt, 1u) % kSortMax] = sel[j];
        for_each_candidate(p, row, bstar, ncand_total, overflow, [&](uint64_t key) {
            if (key >= thr) winners[atomicAdd(&s_cnt, 1u) % kSortMax] = key;
        });
        __syncthreads();
        const uint32_t got = s_cnt;
        if (got != k && t == 0) atomicOr(p.status, TIDAL_DEV_TOPK_OVERFLOW);
        // re-key by position ascending: (pos << 32) | score bits ; pad with ~0
        uint32_t np2 = 1;
        while (np2 < k) np2 <<= 1;
        __syncthreads();
        for (uint32_t j = t; j < np2; j += blockDim.x) {
            if (j < min(got, k)) {
                const uint32_t pos = key_pos(winners[j]);
                winners[j] = ((uint64_t)pos << 32) | (uint64_t)__float_as_uint(srow[pos]);
            } else {
                winners[j] = ~0ull;
            }
        }
        __syncthreads();
        for (uint32_t size = 2; size <= np2; size <<= 1) {
            for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
                for (uint32_t j = t; j < np2 / 2; j += blockDim.x) {
                    const uint32_t lo = 2 * j - (j & (stride - 1));
                    const uint32_t hi = lo + stride;
                    const bool asc = ((lo & size) == 0);
                    const uint64_t a = winners[lo], b = winners[hi];
                    if ((a > b) == asc) { winners[lo] = b; winners[hi] = a; }
                }
                __syncthreads();
            }
        }
        // emit with the ownership filter, order preserved
        if (t == 0) s_cnt = 0;
        __syncthreads();
        for (uint32_t base = 0; base < k; base += blockDim.x) {
            const uint32_t j = base + t;
            int32_t v = 0;
            bool keep = false;
            uint64_t w = 0;
            if (j < k) {
                w = winners[j];
                if (w != ~0ull) {
                    v = emit_value((uint32_t)(w >> 32));
                    keep = !own || (v >= p.own_lo && v < p.own_hi);
                }
            }
            scratch[t] = keep ? 1u : 0u;
            __syncthreads();
            for (int off = 1; off < kTopkThreads; off <<= 1) {
                uint32_t x = (t >= off) ? scratch[t - off] : 0;
                __syncthreads();
                scratch[t] += x;
                __syncthreads();
            }
            const uint32_t before = s_cnt;
            if (keep) {
                const uint32_t at = before + scratch[t] - 1;
                out_idx[at] = own ? v - p.own_lo : v;
                if (out_val) out_val[at] = __uint_as_float((uint32_t)(w & 0xFFFFFFFFull));
            }
            __syncthreads();
            if (t == kTopkThreads - 1) s_cnt = before + scratch[t];
            __syncthreads();
        }
        if (t == 0 && p.out_count) p.out_count[row] = (int32_t)s_cnt;
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
        for (uint32_t j = t; j < nsel; j += blockDim.x) put(sel[j]);
        for_each_candidate(p, row, bstar, ncand_total, overflow, [&](uint64_t key) {
            if (key >= thr) put(key);
        });
        __syncthreads();
        if (t == 0 && p.out_count) p.out_count[row] = (int32_t)min(s_cnt, k);
    }

    // ---- leave the counters zero at rest
    __syncthreads();
    for (int i = t; i < kBins; i += blockDim.x) p.hist[(size_t)row * kBins + i] = 0;
    if (t < 8) st[t] = 0;
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_topk(const tidal_topk_args* a, void* d_ws, size_t ws_bytes, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_scores && a->d_out_idx, TIDAL_ERR_ARG, "scores and out_idx must be given");
    TIDAL_REQUIRE(a->rows >= 1 && a->n >= 1 && a->k >= 1, TIDAL_ERR_ARG, "rows, n and k must be positive (rows %d n %lld k %d)",
                  a->rows, (long long)a->n, a->k);
    TIDAL_REQUIRE(a->n <= 0x7FFFFFFFll, TIDAL_ERR_ARG, "row length %lld does not fit int32 positions", (long long)a->n);
    TIDAL_REQUIRE(a->row_stride >= a->n, TIDAL_ERR_ARG, "row_stride shorter than n");
    TIDAL_REQUIRE(a->d_in_idx == nullptr || a->in_idx_stride == 0 || a->in_idx_stride >= a->n, TIDAL_ERR_ARG,
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
    p.hist = a->d_hist ? a->d_hist : (uint32_t*)((char*)d_ws + L->hist_off);
    p.row_state = (uint32_t*)((char*)d_ws + L->row_state_off);
    p.cand = (uint64_t*)((char*)d_ws + L->cand_off);
    p.sel = (uint64_t*)((char*)d_ws + L->sel_off);
    p.cand_cap = L->cand_cap;
    p.status = (uint32_t*)((char*)d_ws + L->status_off);
    cudaStream_t st = (cudaStream_t)stream;

    if ((int64_t)a->k >= a->n) {
        topk_finish_kernel<<<a->rows, kTopkThreads, 0, st>>>(p, 1);
        TIDAL_CUDA_OK(cudaGetLastError());
    count_launch();
        return TIDAL_OK;
    }
    int nblk = (int)((a->n + 16383) / 16384);
    const int max_blk = (2 * 148 + a->rows - 1) / a->rows;
    if (nblk > max_blk) nblk = max_blk;
    if (nblk < 1) nblk = 1;
    if (!a->d_hist) {
        topk_hist_kernel<<<dim3(nblk, a->rows), kTopkThreads, 0, st>>>(p);
        TIDAL_CUDA_OK(cudaGetLastError());
    count_launch();
    }
    topk_partition_kernel<<<dim3(nblk, a->rows), kTopkThreads, 0, st>>>(p);
    TIDAL_CUDA_OK(cudaGetLastError());
    count_launch();
    topk_finish_kernel<<<a->rows, kTopkThreads, 0, st>>>(p, 0);
    TIDAL_CUDA_OK(cudaGetLastError());
    count_launch();
    return TIDAL_OK;
}
