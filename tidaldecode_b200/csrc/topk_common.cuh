// Device code of the row-wise top-k that more than one kernel uses: key construction, the block-wide
// scans and threshold searches, and the one-launch "cluster row" routine (see topk.cu for the algorithm).
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace tidal {

constexpr int kBins = TIDAL_TOPK_BINS;
constexpr int kTopkThreads = 1024;
constexpr int kSortMax = 4096;        // winners are position-sorted up to this k
constexpr int kRankSortMax = 256;     // ... by counting up to this k (k^2 / threads comparisons), by a bitonic network above
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
static __device__ void find_threshold_bin(const uint32_t* h, uint32_t* ws, uint32_t k, int* bin_out, uint32_t* above_out) {
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

// Count one key's digit in a shared-memory histogram with the lanes of the warp that hold the same digit
// combined into one atomic: candidates of one threshold bin often share their next digits too (a cluster of
// near-equal scores), and thousands of single atomics on one shared-memory word serialise.  (Not for the
// first digit of a whole row: there the 4096 bins spread the keys and the match costs more than it saves —
// measured 46 against 32 us on 8 rows of 131 072 scores.)
__device__ __forceinline__ void count_digit(uint32_t* h, uint32_t digit) {
    const unsigned peers = __match_any_sync(__activemask(), digit);
    if ((threadIdx.x & 31) == (unsigned)(__ffs(peers) - 1)) atomicAdd(&h[digit], (uint32_t)__popc(peers));
}

// Reserve one slot of a list whose fill count is `counter` for every lane that calls this together (the lanes
// currently converged in the caller's branch): one atomic per group instead of one per lane.
__device__ __forceinline__ uint32_t append_slot(uint32_t* counter) {
    const unsigned m = __activemask();
    const int lane = threadIdx.x & 31, leader = __ffs(m) - 1;
    uint32_t base = 0;
    if (lane == leader) base = atomicAdd(counter, (uint32_t)__popc(m));
    base = __shfl_sync(m, base, leader);
    return base + (uint32_t)__popc(m & ((1u << lane) - 1u));
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

// ------------------------------------------------------------------ cluster path
constexpr int kClusterMaxK = 2048;            // winners kept in shared memory
constexpr int kClusterCountSortMax = 256;     // winners ordered by counting up to this many, by a bitonic network above
constexpr int kClusterCand = 4096;            // candidates kept in shared memory
constexpr int64_t kClusterMaxN = 1 << 21;
constexpr int64_t kClusterSmemCandMaxN = 1 << 16;   // longer rows keep their candidates in the workspace
constexpr size_t kClusterSmem = sizeof(uint32_t) * kBins                          // h
                                + sizeof(uint64_t) * (kClusterMaxK + kClusterCand)    // this CTA's own lists / local histogram
                                + sizeof(uint64_t) * (kClusterMaxK + kClusterCand);   // the lists gathered in the first CTA

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

// One row of the one-launch path, run by the cluster of CS CTAs that `row_of_cluster` belongs to (CS = 1: a single
// CTA).  `csm`: kClusterSmem bytes of dynamic shared memory, 16-byte aligned, at the same offset in every CTA of
// the cluster.  Every thread of every CTA of the cluster must call it; CTAs other than the first return early.
// Callable from other kernels (the peer exchange ranks its candidates with it) and several times per kernel:
// a __syncthreads() must separate two calls.
__device__ __forceinline__ void topk_cluster_row(TopkParams p, const int row, unsigned char* csm) {
    uint32_t* h = reinterpret_cast<uint32_t*>(csm);                                   // [kBins]
    uint64_t* my_sel = reinterpret_cast<uint64_t*>(csm + sizeof(uint32_t) * kBins);   // [kClusterMaxK] found by this CTA
    uint64_t* my_cand = my_sel + kClusterMaxK;                                        // [kClusterCand]
    uint64_t* g_sel = my_cand + kClusterCand;                                         // [kClusterMaxK] gathered (first CTA's is used)
    uint64_t* g_cand = g_sel + kClusterMaxK;                                          // [kClusterCand]
    // Candidates of the threshold bin: in shared memory for short rows; long rows can put thousands of
    // keys into one bin (e.g. 1 % of 1 M tokens with high affinity), so theirs go to the workspace.
    const bool cand_global = p.n > kClusterSmemCandMaxN && p.cand != nullptr;
    const uint32_t cand_capacity = cand_global ? (uint32_t)min(p.cand_cap, (int64_t)0x7fffffff) : (uint32_t)kClusterCand;
    uint32_t* h_local = reinterpret_cast<uint32_t*>(my_sel);                          // own-slice histogram (no-hist path)
    __shared__ uint32_t ws[32];
    __shared__ ClusterShared sh;

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned CS = cluster.num_blocks();
    const unsigned rank = cluster.block_rank();
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
    const bool gather = CS > 1 || cand_global;       // lists travel to the first CTA (or to the workspace)

    // ---- digit-0 histogram of the whole row into h
    if (p.hist) {
        // The first CTA's counters must be initialised before anyone adds to them: arrive now (thread 0's
        // store above is released by its own arrive), wait only right before the first remote add.
        if (gather) cluster_arrive_release();
        for (int i = t; i < kBins; i += kTopkThreads) h[i] = p.hist[(size_t)row * kBins + i];
        __syncthreads();
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
    //      over to the first CTA's gather lists: one remote atomic per CTA and list instead of one per key
    __shared__ uint32_t my_nsel, my_ncand, base_sel, base_cand;
    if (t == 0) { my_nsel = 0; my_ncand = 0; }
    __syncthreads();
    {
        auto push = [&](float v, int64_t j) {
            const uint64_t key = make_key(v, (uint32_t)j, p.n, p.force_last);
            const int bin = key_bin(key);
            if (bin > bstar) {
                const uint32_t at = append_slot(&my_nsel);
                if (at < (uint32_t)kClusterMaxK) my_sel[at] = key;
            } else if (bin == bstar) {
                const uint32_t at = append_slot(&my_ncand);
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
    uint64_t* sel = my_sel;                           // the lists the first CTA resolves from
    uint64_t* cand = my_cand;
    if (gather) {
        if (p.hist) cluster_wait();                   // (the no-hist path has passed two full cluster barriers)
        ClusterShared* sh0 = cluster.map_shared_rank(&sh, 0);
        // a CTA whose own candidate list overflowed reports a count beyond any capacity: the resolver
        // then rescans the row instead of trusting the lists
        const uint32_t nc = my_ncand > (uint32_t)kClusterCand ? 0x40000000u : my_ncand;
        if (t == 0) {
            base_sel = atomicAdd(&sh0->nsel, my_nsel);
            base_cand = atomicAdd(&sh0->ncand, nc);
        }
        __syncthreads();
        // the gather lists are written by nobody else's scan, so every CTA copies as soon as it knows its offsets
        uint64_t* sel0 = cluster.map_shared_rank(g_sel, 0);
        uint64_t* cand0 = cand_global ? p.cand + (size_t)row * p.cand_cap : cluster.map_shared_rank(g_cand, 0);
        const uint32_t ns = min(my_nsel, (uint32_t)kClusterMaxK), ncl = min(my_ncand, (uint32_t)kClusterCand);
        for (uint32_t i = t; i < ns; i += kTopkThreads)
            if (base_sel + i < (uint32_t)kClusterMaxK) sel0[base_sel + i] = my_sel[i];
        if (nc < 0x40000000u)
            for (uint32_t i = t; i < ncl; i += kTopkThreads)
                if (base_cand + i < cand_capacity) cand0[base_cand + i] = my_cand[i];
        sel = g_sel;
        cand = cand_global ? p.cand + (size_t)row * p.cand_cap : g_cand;
        cluster.sync();                               // everything pushed to the first CTA has landed
    } else if (t == 0) {
        sh.nsel = my_nsel;            // single CTA, lists already in place
        sh.ncand = my_ncand;
    }
    if (!gather) __syncthreads();
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
    // Candidates that went to the workspace but would fit shared memory after all are brought in: the passes
    // below then run on shared memory, and a handful of them is ranked directly like any short row's.
    bool cand_in_smem = !cand_global;
    if (cand_global && !overflow && ncand_total <= (uint32_t)kClusterCand) {
        for (uint32_t i = t; i < ncand_total; i += kTopkThreads) g_cand[i] = cand[i];
        __syncthreads();
        cand = g_cand;
        cand_in_smem = true;
    }
    const bool few = !overflow && cand_in_smem && ncand_total <= 256u && need <= ncand_total;
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
            if ((key & known_mask) == prefix) count_digit(h, (uint32_t)(key >> sft) & dmask);
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
    // order by position: a key's low word is 0xFFFFFFFF - position, so order by descending low word.
    // Few winners: every thread counts how many precede its own (got^2 / threads comparisons: 16 us at
    // got = 1024, 1 us at 256); more: a bitonic network over the list in shared memory (about 60 steps).
    if (got <= (uint32_t)kClusterCountSortMax) {
        uint64_t mine = 0;
        uint32_t rank_of = 0;
        if ((uint32_t)t < got) {
            mine = sel[t];
            const uint32_t lowm = (uint32_t)mine;
            for (uint32_t i = 0; i < got; ++i) rank_of += ((uint32_t)sel[i] > lowm) ? 1u : 0u;
        }
        __syncthreads();
        if ((uint32_t)t < got) sel[rank_of] = mine;
        __syncthreads();
    } else {
        uint32_t np2 = 2 * (uint32_t)kClusterCountSortMax;
        while (np2 < got) np2 <<= 1;
        for (uint32_t j = got + t; j < np2; j += kTopkThreads) sel[j] = 0ull;      // low word 0 = the largest position: sorts last
        __syncthreads();
        for (uint32_t size = 2; size <= np2; size <<= 1) {
            for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
                for (uint32_t j = t; j < np2 / 2; j += kTopkThreads) {
                    const uint32_t lo2 = 2 * j - (j & (stride - 1)), hi2 = lo2 + stride;
                    const bool desc = (lo2 & size) == 0;
                    const uint64_t a = sel[lo2], b = sel[hi2];
                    if (((uint32_t)a < (uint32_t)b) == desc) {
                        sel[lo2] = b;
                        sel[hi2] = a;
                    }
                }
                __syncthreads();
            }
        }
    }
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

// ------------------------------------------------------------------ one CTA, rows whose order is the wanted order
// A row that one CTA handles alone (the gathered candidates of all ranks: world * k scores) needs neither the
// winners' list nor a sort: find the exact key T of the k-th largest score — first digit by histogram, the rest
// among the threshold bin's candidates — and then walk the row once more IN ORDER, keeping what is >= T: the
// output comes out in ascending place (and the ownership filter is part of the same compaction).  Thread t owns
// the run of consecutive places [t * E, (t + 1) * E); for rows of up to 8 * kTopkThreads scores it loads its keys
// and values once and keeps them in registers through all three steps, so the row is read from memory once and
// the whole routine is a handful of block-wide barriers — no sorting network (ordering 1024 winners by a bitonic
// network alone costs more than all of this).  Same result as topk_cluster_row, bit for bit.
// Returns false — for all threads alike, nothing written — if the threshold bin holds more candidates than
// shared memory takes; the caller then uses topk_cluster_row.  `csm`: kClusterSmem bytes.
constexpr int kOrderedRegs = 8;       // places per thread that are kept in registers
__device__ __forceinline__ bool topk_ordered_row(const TopkParams& p, const int row, unsigned char* csm) {
    uint32_t* h = reinterpret_cast<uint32_t*>(csm);                                   // [kBins]
    uint64_t* cand = reinterpret_cast<uint64_t*>(csm + sizeof(uint32_t) * kBins);     // [kClusterCand]
    __shared__ uint32_t ws[32];
    __shared__ uint32_t s_ncand, s_digit, s_need, s_done;
    __shared__ unsigned long long s_T;
    const int t = threadIdx.x;
    const int64_t n = p.n;
    const uint32_t k = (uint32_t)p.k;
    const int per = (int)((n + kTopkThreads - 1) / kTopkThreads);       // places per thread
    const int64_t j0 = (int64_t)t * per;
    const int cnt = (int)max((int64_t)0, min(n, j0 + per) - j0);
    const bool in_regs = per <= kOrderedRegs;
    const bool own = p.own_hi > p.own_lo;
    // offsets of the run's places: within a segment consecutive, one division for the whole run
    uint32_t seg = 0, off = (uint32_t)j0;
    if (p.seg_len) {
        seg = (uint32_t)(j0 / p.seg_len);
        off = (uint32_t)(j0 - (int64_t)seg * p.seg_len);
    }
    auto place_off = [&](int i, int64_t stride) -> size_t {             // element offset of place j0 + i
        if (!p.seg_len) return (size_t)row * stride + (size_t)(j0 + i);
        uint32_t sg = seg, o = off + (uint32_t)i;
        while (o >= (uint32_t)p.seg_len) {
            o -= (uint32_t)p.seg_len;
            ++sg;
        }
        return (size_t)sg * p.seg_stride + (size_t)row * stride + o;
    };
    auto key_of = [&](int i) -> uint64_t {
        return make_key(p.scores[place_off(i, p.row_stride)], (uint32_t)(j0 + i), n, p.force_last);
    };
    auto value_of = [&](int i) -> int32_t {
        return p.in_idx ? p.in_idx[place_off(i, p.in_idx_stride)] : (int32_t)(j0 + i) + p.idx_offset;
    };
    uint64_t rk[kOrderedRegs];
    int32_t rv[kOrderedRegs];
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < kOrderedRegs; ++i) {
            rk[i] = i < cnt ? key_of(i) : 0ull;
            rv[i] = i < cnt ? value_of(i) : 0;
        }
    }
    for (int i = t; i < kBins; i += kTopkThreads) h[i] = 0;
    if (t == 0) s_ncand = 0;
    __syncthreads();
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < kOrderedRegs; ++i)
            if (i < cnt) atomicAdd(&h[key_bin(rk[i])], 1u);
    } else {
        for (int i = 0; i < cnt; ++i) atomicAdd(&h[key_bin(key_of(i))], 1u);
    }
    __syncthreads();
    int bstar;
    uint32_t above;
    find_threshold_bin(h, ws, k, &bstar, &above);
    uint32_t need = k - above;                          // winners among the threshold bin's keys (>= 1)
    auto collect = [&](uint64_t key) {
        if (key_bin(key) == bstar) {
            const uint32_t at = append_slot(&s_ncand);
            if (at < (uint32_t)kClusterCand) cand[at] = key;
        }
    };
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < kOrderedRegs; ++i)
            if (i < cnt) collect(rk[i]);
    } else {
        for (int i = 0; i < cnt; ++i) collect(key_of(i));
    }
    __syncthreads();
    const uint32_t nc = s_ncand;
    if (nc > (uint32_t)kClusterCand) return false;
    if (nc <= (uint32_t)kTopkThreads) {
        // keys are distinct: T is the candidate with exactly need - 1 larger ones
        if ((uint32_t)t < nc) {
            const uint64_t key = cand[t];
            uint32_t larger = 0;
            for (uint32_t i = 0; i < nc; ++i) larger += cand[i] > key ? 1u : 0u;
            if (larger == need - 1) s_T = key;
        }
    } else {
        // 8-bit radix passes over key bits 51..0 of the candidates until the digit's population is what is needed
        uint64_t prefix = (uint64_t)bstar << 52, known_mask = 0xFFFull << 52;
        bool done = false;
        for (int shift = 44; !done && shift >= -4; shift -= 8) {
            const int sft = shift < 0 ? 0 : shift;
            const int nb = shift < 0 ? 16 : 256;
            const uint32_t dmask = (uint32_t)nb - 1u;
            if (t < 256) h[t] = 0;
            __syncthreads();
            for (uint32_t i = t; i < nc; i += kTopkThreads) {
                const uint64_t key = cand[i];
                if ((key & known_mask) == prefix) count_digit(h, (uint32_t)(key >> sft) & dmask);
            }
            __syncthreads();
            if (t < 32) warp_find_digit(h, nb, need, &s_digit, &s_need, &s_done);
            __syncthreads();
            prefix |= (uint64_t)s_digit << sft;
            known_mask |= (uint64_t)dmask << sft;
            need = s_need;
            done = s_done != 0;
            __syncthreads();
        }
        // winners among the candidates: key >= prefix (all keys of the last digit's group win)
        if (t == 0) s_T = prefix;
    }
    __syncthreads();
    const uint64_t T = s_T;
    // ---- the row once more, in order
    auto kept = [&](uint64_t key, int32_t v) -> bool { return key >= T && (!own || (v >= p.own_lo && v < p.own_hi)); };
    uint32_t mine = 0;
    if (in_regs) {
#pragma unroll
        for (int i = 0; i < kOrderedRegs; ++i) mine += (i < cnt && kept(rk[i], rv[i])) ? 1u : 0u;
    } else {
        for (int i = 0; i < cnt; ++i)
            if (key_of(i) >= T) mine += kept(T, value_of(i)) ? 1u : 0u;
    }
    const uint32_t incl = block_scan_incl(mine, ws);
    uint32_t at = incl - mine;
    int32_t* out_idx = p.out_idx + (size_t)row * p.out_stride;
    float* out_val = p.out_val ? p.out_val + (size_t)row * p.out_stride : nullptr;
    if (mine) {
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < kOrderedRegs; ++i)
                if (i < cnt && kept(rk[i], rv[i])) {
                    out_idx[at] = own ? rv[i] - p.own_lo : rv[i];
                    if (out_val) out_val[at] = p.scores[place_off(i, p.row_stride)];
                    ++at;
                }
        } else {
            for (int i = 0; i < cnt; ++i)
                if (key_of(i) >= T) {
                    const int32_t v = value_of(i);
                    if (kept(T, v)) {
                        out_idx[at] = own ? v - p.own_lo : v;
                        if (out_val) out_val[at] = p.scores[place_off(i, p.row_stride)];
                        ++at;
                    }
                }
        }
    }
    if (t == kTopkThreads - 1 && p.out_count) p.out_count[row] = (int32_t)incl;
    __syncthreads();
    return true;
}

}  // namespace tidal
