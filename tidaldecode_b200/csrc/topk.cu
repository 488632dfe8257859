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
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace tidal {

constexpr int kBins = TIDAL_TOPK_BINS;
constexpr int kTopkThreads = 1024;
constexpr int kSortMax = 4096;        // winners are position-sorted up to this k
constexpr int kRankSortMax = 1024;    // ... by counting up to this k, by a bitonic network above
constexpr int64_t kFusedMaxN = 1 << 18;

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
    uint32_t* hist;       // [rows][kBins] in global memory, or nullptr (fused kernel builds its own)
    uint32_t* row_state;  // [rows][8]: 0 sel count, 1 cand count
    uint64_t* cand;       // [rows][cand_cap]
    uint64_t* sel;        // [rows][kMaxK]
    int64_t cand_cap;
    uint32_t* status;
    int32_t seg_len;      // 0, or rows are made of segments seg_stride elements apart (cluster kernel only)
    int64_t seg_stride;
    const int32_t* row_len;  // nullptr, or per-row lengths on the device (cluster kernel only); n is then their bound
};

// Offset of element j of a row whose contiguous layout would start at row*stride.
__device__ __forceinline__ size_t elem_off(const TopkParams& p, int64_t stride, int row, int64_t j) {
    if (p.seg_len == 0) return (size_t)row * stride + (size_t)j;
    const int64_t sg = j / p.seg_len;
    return (size_t)sg * p.seg_stride + (size_t)row * stride + (size_t)(j - sg * p.seg_len);
}

__device__ __forceinline__ uint64_t make_key(float s, uint32_t pos, int64_t n, int force_last) {
    uint32_t k32 = ordered_key(s);
    if (force_last && (int64_t)pos == n - 1) k32 = 0xFFFFFFFFu;
    return ((uint64_t)k32 << 32) | (uint64_t)(0xFFFFFFFFu - pos);
}
__device__ __forceinline__ uint32_t key_pos(uint64_t key) { return 0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull); }
__device__ __forceinline__ int key_bin(uint64_t key) { return (int)((uint32_t)(key >> 32) >> kDigit0Shift); }

// Inclusive scan over the kTopkThreads threads of the block; `ws` has 32 words.
// Ends with a barrier, so `ws` may be reused at once.
__device__ __forceinline__ uint32_t block_scan_incl(uint32_t v, uint32_t* ws) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += n;
    }
    if (lane == 31) ws[warp] = v;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = ws[lane];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, w, off);
            if (lane >= off) w += n;
        }
        ws[lane] = w;
    }
    __syncthreads();
    if (warp > 0) v += ws[warp - 1];
    __syncthreads();
    return v;
}

// Threshold bin b*: count(bins > b*) < k <= count(bins >= b*).  `h` is a shared
// copy of the row's histogram; every thread returns the same (bin, above).
__device__ void find_threshold_bin(const uint32_t* h, uint32_t* ws, uint32_t k, int* bin_out, uint32_t* above_out) {
    constexpr int per = kBins / kTopkThreads;     // 4 bins per thread, thread 0 owns the top ones
    const int t = threadIdx.x;
    const int base = kBins - (t + 1) * per;
    uint32_t mine = 0;
#pragma unroll
    for (int i = 0; i < per; ++i) mine += h[base + i];
    const uint32_t incl = block_scan_incl(mine, ws), excl = incl - mine;
    __shared__ int s_bin;
    __shared__ uint32_t s_above;
    if (t == 0) { s_bin = 0; s_above = 0; }
    __syncthreads();
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

// One warp finds, in a 256-bin digit histogram, the digit d with
// count(digits > d) < need <= count(digits >= d).  Results through shared words.
__device__ __forceinline__ void warp_find_digit(const uint32_t* h, int nbins, uint32_t need, uint32_t* s_digit,
                                                uint32_t* s_need, uint32_t* s_done) {
    const int lane = threadIdx.x & 31;
    const int per = nbins / 32 > 0 ? nbins / 32 : 1;      // 8 bins per lane (256), or 1 with 16 active lanes (16)
    const bool active = lane * per < nbins;
    const int base = nbins - (lane + 1) * per;            // lane 0 owns the top bins
    uint32_t mine = 0;
    if (active)
        for (int i = 0; i < per; ++i) mine += h[base + i];
    uint32_t incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
    }
    const uint32_t excl = incl - mine;
    if (active && excl < need && need <= incl) {
        uint32_t above = excl;
        for (int i = per - 1; i >= 0; --i) {
            const uint32_t c = h[base + i];
            if (above + c >= need) {
                *s_digit = (uint32_t)(base + i);
                *s_need = need - above;
                *s_done = (c == need - above) ? 1u : 0u;
                break;
            }
            above += c;
        }
    }
}

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
            const uint32_t at = atomicAdd(sel_cnt, 1u);
            if (at < (uint32_t)kMaxK) sel[at] = key;
        } else if (bin == bstar) {
            const uint32_t at = atomicAdd(cand_cnt, 1u);
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
            if ((key & known_mask) == prefix) atomicAdd(&h[(uint32_t)(key >> sh) & dmask], 1u);
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


// ------------------------------------------------------------------ cluster path
constexpr int kClusterMaxK = 2048;            // winners kept in shared memory
constexpr int kClusterCand = 4096;            // candidates kept in shared memory
constexpr int64_t kClusterMaxN = 1 << 21;
constexpr int64_t kClusterSmemCandMaxN = 1 << 16;   // longer rows keep their candidates in the workspace
constexpr size_t kClusterSmem = sizeof(uint32_t) * kBins                       // h
                                + sizeof(uint64_t) * (kClusterMaxK + kClusterCand);  // lists (first CTA) / local histogram

struct ClusterShared {
    uint32_t nsel, ncand, cnt, digit, need, done;
};

template <typename F>
__device__ __forceinline__ void for_each_cluster_candidate(const TopkParams& p, int row, int bstar, const uint64_t* cand,
                                                           uint32_t ncand, bool overflow, F f) {
    if (!overflow) {
        for (uint32_t j = threadIdx.x; j < ncand; j += kTopkThreads) f(cand[j]);
    } else {
        for (int64_t j = threadIdx.x; j < p.n; j += kTopkThreads) {
            const uint64_t key = make_key(p.scores[elem_off(p, p.row_stride, row, j)], (uint32_t)j, p.n, p.force_last);
            if (key_bin(key) == bstar) f(key);
        }
    }
}

__global__ void __launch_bounds__(kTopkThreads) topk_cluster_kernel(const TopkParams p_in) {
    extern __shared__ __align__(16) unsigned char csm[];
    TopkParams p = p_in;
    uint32_t* h = reinterpret_cast<uint32_t*>(csm);                                   // [kBins]
    uint64_t* sel = reinterpret_cast<uint64_t*>(csm + sizeof(uint32_t) * kBins);      // [kClusterMaxK]
    // Candidates of the threshold bin: in shared memory for short rows; long rows can put thousands of
    // keys into one bin (e.g. 1 % of 1 M tokens with high affinity), so theirs go to the workspace.
    const bool cand_global = p.n > kClusterSmemCandMaxN && p.cand != nullptr;
    uint64_t* cand = cand_global ? p.cand + (size_t)blockIdx.x / cg::this_cluster().num_blocks() * p.cand_cap
                                 : sel + kClusterMaxK;                                // [kClusterCand] in shared memory
    const uint32_t cand_capacity = cand_global ? (uint32_t)min(p.cand_cap, (int64_t)0x7fffffff) : (uint32_t)kClusterCand;
    uint32_t* h_local = reinterpret_cast<uint32_t*>(sel);                             // own-slice histogram (no-hist path)
    __shared__ uint32_t ws[32];
    __shared__ ClusterShared sh;
    pdl_wait();
    pdl_launch_dependents();

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned CS = cluster.num_blocks();
    const unsigned rank = cluster.block_rank();
    const int row = blockIdx.x / CS;
    const int t = threadIdx.x;
    if (p.row_len) {
        // the row's length lives on the device (a decode step replayed as a CUDA graph grows it every step)
        const int64_t n_dev = max(0, p.row_len[row]);
        p.n = min(p.n, n_dev);
        p.k = (int32_t)min((int64_t)p.k, p.n);
        if (p.n == 0) {                       // uniform over the cluster: nobody reaches a cluster barrier
            if (rank == 0 && t == 0 && p.out_count) p.out_count[row] = 0;
            return;
        }
    }
    const float* srow = p.seg_len ? nullptr : p.scores + (size_t)row * p.row_stride;   // contiguous rows only
    auto score_at = [&](int64_t j) -> float { return p.scores[elem_off(p, p.row_stride, row, j)]; };
    const uint32_t k = (uint32_t)p.k;
    const int64_t per = ((p.n + CS - 1) / CS + 3) & ~(int64_t)3;      // slice length, a multiple of 4
    const int64_t lo = (int64_t)rank * per, hi = min(p.n, lo + per);

    if (t == 0) { sh.nsel = 0; sh.ncand = 0; sh.cnt = 0; }

    // ---- digit-0 histogram of the whole row into h
    if (p.hist) {
        for (int i = t; i < kBins; i += kTopkThreads) h[i] = p.hist[(size_t)row * kBins + i];
        cluster.sync();            // the first CTA's counters are initialised before anyone pushes to them
    } else {
        for (int i = t; i < kBins; i += kTopkThreads) h_local[i] = 0;
        __syncthreads();
#pragma unroll 4
        for (int64_t j = lo + t; j < hi; j += kTopkThreads)
            atomicAdd(&h_local[key_bin(make_key(score_at(j), (uint32_t)j, p.n, p.force_last))], 1u);
        cluster.sync();
        for (int i = t; i < kBins; i += kTopkThreads) {
            uint32_t a = 0;
            for (unsigned r = 0; r < CS; ++r) a += cluster.map_shared_rank(h_local, r)[i];
            h[i] = a;
        }
        cluster.sync();            // every CTA has read every local histogram: the list area may be written now
    }
    int bstar;
    uint32_t above;
    find_threshold_bin(h, ws, k, &bstar, &above);

    // ---- scan the slice into this CTA's own lists (local shared-memory atomics), then hand them
    //      over to the first CTA in two bulk copies: one remote atomic per CTA instead of one per key
    __shared__ uint32_t my_nsel, my_ncand, base_sel, base_cand;
    uint64_t* my_sel = sel;                      // [kClusterMaxK]   (every CTA has the same layout)
    uint64_t* my_cand = sel + kClusterMaxK;      // [kClusterCand]
    if (t == 0) { my_nsel = 0; my_ncand = 0; }
    __syncthreads();
    {
        auto push = [&](float v, int64_t j) {
            const uint64_t key = make_key(v, (uint32_t)j, p.n, p.force_last);
            const int bin = key_bin(key);
            if (bin > bstar) {
                const uint32_t at = atomicAdd(&my_nsel, 1u);
                if (at < (uint32_t)kClusterMaxK) my_sel[at] = key;
            } else if (bin == bstar) {
                const uint32_t at = atomicAdd(&my_ncand, 1u);
                if (at < (uint32_t)kClusterCand) my_cand[at] = key;
            }
        };
        const bool vec_ok = p.seg_len == 0 && ((reinterpret_cast<uintptr_t>(srow) & 15) == 0);
        if (vec_ok) {
            const int64_t hi4 = lo + ((hi - lo) & ~(int64_t)3);
#pragma unroll 2
            for (int64_t j = lo + 4 * (int64_t)t; j < hi4; j += 4 * kTopkThreads) {
                const float4 v = *reinterpret_cast<const float4*>(srow + j);
                push(v.x, j); push(v.y, j + 1); push(v.z, j + 2); push(v.w, j + 3);
            }
            for (int64_t j = hi4 + t; j < hi; j += kTopkThreads) push(srow[j], j);
        } else {
#pragma unroll 4
            for (int64_t j = lo + t; j < hi; j += kTopkThreads) push(score_at(j), j);
        }
    }
    __syncthreads();
    if (CS > 1 || cand_global) {
        ClusterShared* sh0 = cluster.map_shared_rank(&sh, 0);
        // a CTA whose own candidate list overflowed reports a count beyond any capacity: the resolver
        // then rescans the row instead of trusting the lists
        const uint32_t nc = my_ncand > (uint32_t)kClusterCand ? 0x40000000u : my_ncand;
        if (t == 0) {
            base_sel = atomicAdd(&sh0->nsel, my_nsel);
            base_cand = atomicAdd(&sh0->ncand, nc);
        }
        __syncthreads();
        uint64_t* sel0 = cluster.map_shared_rank(sel, 0);
        uint64_t* cand0 = cand_global ? cand : cluster.map_shared_rank(sel + kClusterMaxK, 0);
        // read everything this thread will move before anyone writes (rank 0's source is its destination array)
        constexpr int kSelPer = kClusterMaxK / kTopkThreads, kCandPer = kClusterCand / kTopkThreads;
        uint64_t vs[kSelPer], vc[kCandPer];
        const uint32_t ns = min(my_nsel, (uint32_t)kClusterMaxK), ncl = min(my_ncand, (uint32_t)kClusterCand);
#pragma unroll
        for (int u = 0; u < kSelPer; ++u) vs[u] = (t + u * kTopkThreads < ns) ? my_sel[t + u * kTopkThreads] : 0;
#pragma unroll
        for (int u = 0; u < kCandPer; ++u) vc[u] = (t + u * kTopkThreads < ncl) ? my_cand[t + u * kTopkThreads] : 0;
        cluster.sync();               // all CTAs hold their keys in registers and know their offsets
#pragma unroll
        for (int u = 0; u < kSelPer; ++u) {
            const uint32_t i = t + u * kTopkThreads;
            if (i < ns && base_sel + i < (uint32_t)kClusterMaxK) sel0[base_sel + i] = vs[u];
        }
        if (nc < 0x40000000u) {
#pragma unroll
            for (int u = 0; u < kCandPer; ++u) {
                const uint32_t i = t + u * kTopkThreads;
                if (i < ncl && base_cand + i < cand_capacity) cand0[base_cand + i] = vc[u];
            }
        }
    } else if (t == 0) {
        sh.nsel = my_nsel;            // single CTA, lists already in place
        sh.ncand = my_ncand;
    }
    cluster.sync();
    if (rank != 0) return;

    // ---- first CTA: resolve, order, emit — all in shared memory
    int32_t* out_idx = p.out_idx + (size_t)row * p.out_stride;
    float* out_val = p.out_val ? p.out_val + (size_t)row * p.out_stride : nullptr;
    const bool own = p.own_hi > p.own_lo;
    const uint32_t nsel = min(sh.nsel, (uint32_t)kClusterMaxK);
    const uint32_t ncand_total = sh.ncand;
    const bool overflow = ncand_total > cand_capacity;
    uint32_t need = k - above;
    if (sh.nsel != above && t == 0) atomicOr(p.status, TIDAL_DEV_TOPK_OVERFLOW);

    // Few candidates in shared memory (the usual case: a 12-bit first digit leaves a few dozen keys in the
    // threshold bin): rank them directly — keys are distinct, so the `need` largest are those with fewer
    // than `need` larger ones — instead of up to seven more radix passes with four barriers each.
    const bool few = !overflow && !cand_global && ncand_total <= 256u && need <= ncand_total;
    if (few) {
        if ((uint32_t)t < ncand_total) {
            const uint64_t key = cand[t];
            uint32_t larger = 0;
            for (uint32_t i = 0; i < ncand_total; ++i) larger += cand[i] > key ? 1u : 0u;
            if (larger < need) {
                const uint32_t at = nsel + atomicAdd(&sh.cnt, 1u);
                if (at < (uint32_t)kClusterMaxK) sel[at] = key;
            }
        }
        __syncthreads();
    }
    uint64_t prefix = (uint64_t)bstar << 52;
    uint64_t known_mask = 0xFFFull << 52;
    bool done = few || (need == ncand_total);
    for (int shift = 44; !done && shift >= -4; shift -= 8) {
        const int sft = shift < 0 ? 0 : shift;
        const int nb = shift < 0 ? 16 : 256;
        const uint32_t dmask = (uint32_t)nb - 1u;
        if (t < 256) h[t] = 0;
        __syncthreads();
        for_each_cluster_candidate(p, row, bstar, cand, ncand_total, overflow, [&](uint64_t key) {
            if ((key & known_mask) == prefix) atomicAdd(&h[(uint32_t)(key >> sft) & dmask], 1u);
        });
        __syncthreads();
        if (t < 32) warp_find_digit(h, nb, need, &sh.digit, &sh.need, &sh.done);
        __syncthreads();
        prefix |= (uint64_t)sh.digit << sft;
        known_mask |= (uint64_t)dmask << sft;
        need = sh.need;
        done = sh.done != 0;
        __syncthreads();
    }
    const uint64_t thr = prefix;

    // winners: sel[0, nsel) plus the candidates at or above the threshold, appended behind them
    if (!few) {
        for_each_cluster_candidate(p, row, bstar, cand, ncand_total, overflow, [&](uint64_t key) {
            if (key >= thr) {
                const uint32_t at = nsel + atomicAdd(&sh.cnt, 1u);
                if (at < (uint32_t)kClusterMaxK) sel[at] = key;
            }
        });
        __syncthreads();
    }
    const uint32_t got = min(nsel + sh.cnt, k);
    if (nsel + sh.cnt != k && t == 0) atomicOr(p.status, TIDAL_DEV_TOPK_OVERFLOW);
    // order by position: a key's low word is 0xFFFFFFFF - position, so rank by descending low word
    uint64_t mine[kClusterMaxK / kTopkThreads];
    uint32_t rank_of[kClusterMaxK / kTopkThreads];
#pragma unroll
    for (int u = 0; u < kClusterMaxK / kTopkThreads; ++u) {
        const uint32_t j = t + u * kTopkThreads;
        rank_of[u] = 0;
        mine[u] = 0;
        if (j < got) {
            mine[u] = sel[j];
            const uint32_t lowm = (uint32_t)mine[u];
            uint32_t r = 0;
            for (uint32_t i = 0; i < got; ++i) r += ((uint32_t)sel[i] > lowm) ? 1u : 0u;
            rank_of[u] = r;
        }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kClusterMaxK / kTopkThreads; ++u)
        if (t + u * kTopkThreads < got) sel[rank_of[u]] = mine[u];
    __syncthreads();
    // emit in order with the ownership filter
    uint32_t before = 0;
    for (uint32_t base = 0; base < got; base += kTopkThreads) {
        const uint32_t j = base + t;
        int32_t v = 0;
        float sc = 0.f;
        bool keep = false;
        if (j < got) {
            const uint64_t key = sel[j];
            const uint32_t pos = key_pos(key);
            v = p.in_idx ? p.in_idx[elem_off(p, p.in_idx_stride, row, pos)] : (int32_t)pos + p.idx_offset;
            keep = !own || (v >= p.own_lo && v < p.own_hi);
            if (out_val) sc = (p.force_last && (int64_t)pos == p.n - 1) ? score_at(pos) : key_to_float((uint32_t)(key >> 32));
        }
        const uint32_t incl = block_scan_incl(keep ? 1u : 0u, ws);
        if (keep) {
            const uint32_t at = before + incl - 1;
            out_idx[at] = own ? v - p.own_lo : v;
            if (out_val) out_val[at] = sc;
        }
        if (t == kTopkThreads - 1) sh.cnt = before + incl;
        __syncthreads();
        before = sh.cnt;
        __syncthreads();
    }
    if (t == 0 && p.out_count) p.out_count[row] = (int32_t)before;
    if (p.hist)
        for (int i = t; i < kBins; i += kTopkThreads) p.hist[(size_t)row * kBins + i] = 0;
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
        int cs = 8;
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
