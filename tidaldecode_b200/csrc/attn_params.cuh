// Parameters shared by the two decode-attention kernels (CUDA-core and tensor-core).
#pragma once

#include <climits>

#include <cooperative_groups.h>

#include "common.cuh"

namespace tidal {

struct AttnParams {
    const void* q;
    void* o;
    const char* kv;
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* seq_lens;
    int32_t seq_len;
    const int32_t* sel_idx;
    const int32_t* sel_counts;
    int32_t sel_rows, sel_count, sel_physical, extra_page;
    int64_t sel_stride;
    float* scores;
    int32_t score_rows;
    int64_t score_stride;
    uint32_t* hist;
    int32_t force_last;
    float* part_o;   // [B][Hq][nchunks][D]
    float* part_ml;  // [B][Hq][nchunks][2]
    float* shard_m;  // optional [B][Hq]
    float* shard_l;
    float* shard_o;  // optional [B][Hq][D]
    uint32_t* status;
    int32_t B, Hq, Hkv, page_size;
    int64_t num_pages;
    float sm_scale;
    int32_t nchunks;
    int32_t HC;       // KV heads per CTA
    int32_t greal;    // Hq / Hkv (the kernel's G is 1 in per-q-head list mode)
    int32_t per_head; // 1: head slice index is a q head, HC == 1
    int32_t T, S, TG; // tokens per stage, stages, token groups
    int32_t CW;       // consumer warps
    int32_t PW;       // producer warps (1, 2 or 4), the first warps of the CTA
    int32_t kv_fused; // 1: the CTA takes every KV head and page_size is 1, so a token's K row and V row are
                      // adjacent in the pool and arrive in one copy (stage layout: token-major, K then V)
    int32_t cluster;  // > 1: that many CTAs along the chunk dimension form a cluster that covers the whole
                      // token list and merges through distributed shared memory (then nchunks == cluster)
    uint32_t recv_off; // cluster > 1: byte offset (in dynamic shared memory) of the CTA's receive block
    int32_t nsuper;    // cluster > 1: clusters that share one token list (nchunks == cluster * nsuper); > 1: each cluster
                       // leaves its merged share in part_o / part_ml and the last one to arrive finishes it
    uint32_t* xc_count; // [B][head slices][kMaxCluster] arrivals of those clusters, zero at rest
};

__host__ __device__ inline size_t round16(size_t x) { return (x + 15) & ~(size_t)15; }

// Head-summed logits are reduced across the CTA's heads once per "super-block" of R stages, not
// per stage: slots park their per-head logits in shared memory [2][R*T][HC] (double-buffered, so one
// named barrier per super-block is enough) and all consumer threads then sum, store and count them.
__host__ __device__ inline int score_block_stages(int T, int HC) {
    int r = 2048 / (T * HC);          // 8 KB per buffer
    return r < 1 ? 1 : (r > 16 ? 16 : r);
}
__host__ __device__ inline size_t score_smem_bytes(int T, int HC) {
    return round16((size_t)2 * score_block_stages(T, HC) * T * HC * sizeof(float));
}


// The tokens one CTA streams: entries [tok0, tok0 + ntok) of the token list of sequence b (the whole
// sequence, or the selection list `sel_row` with the newest token appended).
struct TokenList {
    int b, sel_row, list_len, seq_len_b, tok0, ntok;
};

// Looking up where list entry `li` lives takes two steps, both free of side effects so that the
// loads of many entries can be in flight together:
// list_entry: the entry's value — a token position, a pool page (sel_physical), or kExtraEntry for
// the newest token appended behind a selection list;
// entry_row: the pool row of its K vector in units of one token's K bytes (page * 2 * page_size +
// entry; the V row lies page_size rows further).  A bad index sets *bad and yields row 0.
constexpr int kExtraEntry = INT_MIN + 1;
constexpr int kNoEntry = INT_MIN;           // a lane without an entry in this block
__device__ __forceinline__ int list_entry(const AttnParams& p, const TokenList& tl, int li) {
    if (!p.sel_idx) return li;
    if (li >= tl.list_len) return kExtraEntry;
    return p.sel_idx[((size_t)tl.b * p.sel_rows + tl.sel_row) * p.sel_stride + li];
}
__device__ __forceinline__ uint32_t entry_row(const AttnParams& p, const TokenList& tl, int e, bool* bad) {
    int64_t page;
    int entry = 0;
    bool ok = true;
    if (e == kExtraEntry) {
        page = p.extra_page;
    } else if (p.sel_idx && p.sel_physical) {
        page = e;
    } else {
        ok = (e >= 0 && e < tl.seq_len_b);
        const int pos = ok ? e : 0;
        const int pg = pos / p.page_size;
        entry = pos - pg * p.page_size;
        page = p.page_table ? p.page_table[(size_t)tl.b * p.pt_stride + pg] : (int64_t)tl.b * p.pt_stride + pg;
    }
    if (!ok || page < 0 || page >= p.num_pages) {
        *bad = true;
        return 0u;
    }
    return (uint32_t)(page * 2 * p.page_size + entry);
}

constexpr int kAddrBlock = 256;     // list entries whose pool rows are looked up in one go (a multiple of every stage size)
constexpr int kMaxProducerWarps = 4;

// The producer warps of both attention kernels (p.PW of them, 1, 2 or 4): per token one bulk copy of
// the K row and one of the V row (row_bytes each, the CTA's head slice at byte head_off of the token)
// into stage it % S of the ring (stage_stride bytes per stage): token t's K row at t * pitch, its V
// row v_base further.  One warp gets a copy accepted every ~70 cycles whatever its size (measured), so
// rows of 1-2 KB need several warps to keep the SM's load path busy: of every 32 consecutive tokens
// warp w issues those that fall on its lanes [w * 32 / PW, (w + 1) * 32 / PW) (a copy is issued per
// lane in any case, so narrow warps lose nothing), which splits even a 32-token stage evenly.
// With p.kv_fused the two rows are adjacent in the pool and in the stage (v_base == row_bytes) and
// travel as one copy; if the tokens themselves are contiguous as well (no list, no page table) and
// rows are unpadded (pitch == 2 * row_bytes), a whole stage is one copy.
// Completion is counted on full_bar[s] (warp 0 announces the stage's bytes; copies of the other warps
// that land first only drive the count negative for a moment); a stage is refilled once the consumers
// have released it through empty_bar[s].
// Where a row needs a lookup (a selection list or a page table), the rows of kAddrBlock entries are
// looked up at once and parked in src_row ([2][kAddrBlock], double-buffered): the first block by all
// threads of the CTA before the roles split (fill_first_rows), each later block by the producer warps
// (every lane kAddrBlock / 32 independent loads, each warp for its own tokens) when they enter the
// block before it: a stage then costs no dependent global load.  The refill is kept out of line — the
// kernels are short enough for cold instruction fetches to show, and lists of up to kAddrBlock
// entries per CTA never reach it.
__device__ __forceinline__ bool rows_direct(const AttnParams& p) {
    return !p.sel_idx && !p.page_table;       // the row follows from the token index alone: nothing to hide
}
__device__ __forceinline__ int pw_shift(const AttnParams& p) { return p.PW == 4 ? 2 : (p.PW == 2 ? 1 : 0); }
// every thread of the CTA, before the barrier that precedes the role split
__device__ __forceinline__ void fill_first_rows(const AttnParams& p, const TokenList& tl, uint32_t* src_row) {
    if (rows_direct(p)) return;
    const int n = min(kAddrBlock, tl.ntok);
    bool bad = false;
    for (int t = threadIdx.x; t < n; t += blockDim.x) src_row[t] = entry_row(p, tl, list_entry(p, tl, tl.tok0 + t), &bad);
    if (bad) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
}
// rows of the block of entries that starts at `first`, lanes [lane_lo, lane_hi) of every 32 entries, into dst
static __device__ __noinline__ void refill_rows(const AttnParams& p, const TokenList tl, uint32_t* dst, int first, int lane, int lane_lo,
                                         int lane_hi) {
    constexpr int PL = kAddrBlock / 32;
    const bool active = lane >= lane_lo && lane < lane_hi;
    bool bad = false;
    int e[PL];
#pragma unroll
    for (int j = 0; j < PL; ++j) {
        const int t = first + j * 32 + lane;
        e[j] = (active && t < tl.ntok) ? list_entry(p, tl, tl.tok0 + t) : kNoEntry;
    }
#pragma unroll
    for (int j = 0; j < PL; ++j)
        if (e[j] != kNoEntry) dst[j * 32 + lane] = entry_row(p, tl, e[j], &bad);
    if (bad) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
}
template <int MAXPW>   // 1: a single producer warp (p.PW == 1), every lane issues; else p.PW <= MAXPW warps
__device__ __forceinline__ void produce_stages(const AttnParams& p, const TokenList& tl, uint32_t* src_row, int pw, int lane, int S,
                                               int TT, int n_iters, uint32_t row_bytes, uint32_t pitch, uint32_t v_base,
                                               size_t stage_stride, size_t head_off, size_t tok_bytes,
                                               unsigned char* stage_base, uint64_t* full_bar, uint64_t* empty_bar,
                                               volatile int* abort_flag) {
    constexpr int AB = kAddrBlock;
    const int lanes = MAXPW == 1 ? 32 : 32 >> pw_shift(p);   // lanes of every 32-token group that are this warp's
    const int lane_lo = MAXPW == 1 ? 0 : pw * lanes;
    const bool active = MAXPW == 1 || (lane >= lane_lo && lane < lane_lo + lanes);
    const size_t plane = (size_t)p.page_size * tok_bytes;
    const bool direct = rows_direct(p);
    const bool whole_stage = p.kv_fused && direct && pitch == 2u * row_bytes;
    // direct rows: sequence b starts at page b * pt_stride and pages follow the positions (the host has
    // checked the range); page_size 1 needs no division
    const uint32_t row0 = (uint32_t)((int64_t)tl.b * p.pt_stride * 2 * p.page_size);
    auto direct_row = [&](int li) -> uint32_t {
        if (p.page_size == 1) return row0 + 2u * (uint32_t)li;
        const int pg = li / p.page_size;
        return row0 + (uint32_t)(pg * 2 * p.page_size + (li - pg * p.page_size));
    };
    const uint32_t max_row = (uint32_t)(p.num_pages * 2 * p.page_size);
    int base = 0;                                         // first entry of the block being issued
    const uint32_t* cur = src_row;                        // its rows (block 0 was parked by fill_first_rows)
    if (!direct && AB < tl.ntok) refill_rows(p, tl, src_row + AB, AB, lane, lane_lo, lane_lo + lanes);
    for (int it = 0; it < n_iters; ++it) {
        const int s = it % S;
        const int t_first = it * TT;
        if (!direct && t_first == base + AB) {
            base = t_first;
            const int half = (base / AB) & 1;
            cur = src_row + half * AB;
            __syncwarp();                                 // this warp is done with the other half
            if (base + AB < tl.ntok) refill_rows(p, tl, src_row + (half ^ 1) * AB, base + AB, lane, lane_lo, lane_lo + lanes);
        }
        const int valid = min(TT, tl.ntok - t_first);
        const int rel = t_first - base;                   // the stage's first token within the block
        // A warp waits for a stage to be released only if it has something to do there (warp 0 always:
        // it announces the bytes).  With stages shorter than 32 tokens a warp owns tokens in every
        // other stage only; were it to wait on the others too, a warp that fell behind (in a refill)
        // could find such a barrier two phases ahead — the consumers do not need it there — and wait
        // for a phase that only completes after its own next copies: a deadlock.
        bool mine = pw == 0;
        if (MAXPW != 1 && !whole_stage) {
            bool has = false;
            for (int gb = rel & ~31; gb < rel + valid; gb += 32) has |= active && gb + lane >= rel && gb + lane < rel + valid;
            mine |= __any_sync(0xffffffffu, has) != 0;
        }
        if (!mine) continue;
        if (it >= S && !mbar_wait_bounded(&empty_bar[s], ((it / S) - 1) & 1, abort_flag, p.status)) break;   // gave up: issue nothing more
        if (pw == 0 && lane == 0) mbar_arrive_expect_tx(&full_bar[s], (uint32_t)valid * 2u * row_bytes);
        __syncwarp();
        unsigned char* kdst = stage_base + (size_t)s * stage_stride;
        if (whole_stage) {
            if (pw == 0 && lane == 0)
                bulk_g2s(kdst, p.kv + (size_t)direct_row(tl.tok0 + t_first) * tok_bytes, (uint32_t)valid * 2u * row_bytes, &full_bar[s]);
        } else {
            auto issue = [&](int tb) {                    // tb: token within the block
                uint32_t row = direct ? direct_row(tl.tok0 + base + tb) : cur[tb];
                if (row >= max_row) {                     // never copy from outside the pool, whatever the row cache holds
                    atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
                    row = 0;
                }
                const char* ksrc = p.kv + (size_t)row * tok_bytes + head_off;
                unsigned char* dst = kdst + (size_t)(tb - rel) * pitch;
                if (p.kv_fused) {
                    bulk_g2s(dst, ksrc, 2u * row_bytes, &full_bar[s]);
                } else {
                    bulk_g2s(dst, ksrc, row_bytes, &full_bar[s]);
                    bulk_g2s(dst + v_base, ksrc + plane, row_bytes, &full_bar[s]);
                }
            };
            if (MAXPW == 1) {
                for (int t = lane; t < valid; t += 32) issue(rel + t);
            } else {
                for (int gb = rel & ~31; gb < rel + valid; gb += 32) {
                    const int tb = gb + lane;
                    if (active && tb >= rel && tb < rel + valid) issue(tb);
                }
            }
        }
        if (pw == 0 && lane == 0 && it == 0) TIDAL_STAMP(4);
        if (pw == 0 && lane == 0 && it == 1) TIDAL_STAMP(13);
        if (pw == 0 && lane == 0 && it == n_iters - 1) TIDAL_STAMP(5);
    }
    // Nothing of this CTA may still be in flight when it retires.  The consumers waited on every full
    // barrier unless a wait ran out; then the barriers no longer tell (some warps stopped issuing), so
    // every producer warp simply outlasts its own copies: a millisecond, against microseconds of flight.
    if (*abort_flag)
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
}

// Bytes of the per-CTA result block [HC*G][D] + [HC*G][2] that store_attention_result reads.
__host__ __device__ inline size_t cta_result_bytes(int HC, int G, int D) { return (size_t)HC * G * (D + 2) * sizeof(float); }

// Final step of both attention kernels.  cta_o[(hg)*D + d] and cta_ml[hg*2 + {0,1}] hold this CTA's
// un-normalised output, running maximum (log2 domain) and denominator for its HC*G query heads
// (D a power of two, both arrays 16-byte aligned).
// One CTA per token list chunk: written out as a split-KV partial (or as the result when there is a
// single chunk).  A cluster (at most kMaxCluster CTAs): its CTAs cover the whole list and CTA r
// finishes the r-th share of the outputs.  Every CTA pushes the matching share of its block (and its
// maxima and denominators) into the receive block of the CTA that finishes it — posted stores through
// distributed shared memory, no round trip — and after one cluster barrier each CTA merges what it
// received from local shared memory and writes final values: no partials in global memory, no merge
// kernel.  `recv` is that receive block (cluster_recv_bytes() bytes, touched by nothing else); the
// kernel must have ARRIVED at the cluster barrier at its start (cluster_arrive_relaxed, every thread); the
// matching wait is here, before the first store into another CTA, so that every CTA is known to be running.
// A thread owns four consecutive output elements; every thread of the CTA must call this.
constexpr int kMaxCluster = 16;        // 8 is the portable limit; 16 needs the non-portable-size attribute (WsLayout::xc_off holds 16 counters per list)
template <typename T>
struct alignas(sizeof(T) * 4) Pack4 {
    T v[4];
};
__host__ __device__ inline size_t cluster_recv_bytes(int HC, int G, int D, int CS) {
    const int units = HC * G * (D / 4);
    const int per = (units + CS - 1) / CS;
    return (size_t)CS * per * 16 + (size_t)CS * HC * G * 8;
}
template <typename T>
__device__ __forceinline__ void store_attention_result(const AttnParams& p, const float* cta_o, const float* cta_ml, float* recv,
                                                       int HC, int G, int D, int qh0, int b, int chunk) {
    namespace cg = cooperative_groups;
    const int qshift = 31 - __clz(D >> 2);            // float4 per row = 1 << qshift
    const int units = (HC * G) << qshift;
    auto put_final = [&](int hg, int d, float4 acc, float M, float L) {
        const size_t ph = (size_t)b * p.Hq + qh0 + hg;
        if (p.o) {
            const bool some = L > 0.f;
            Pack4<T> pk;
            pk.v[0] = from_f32<T>(some ? acc.x / L : 0.f);
            pk.v[1] = from_f32<T>(some ? acc.y / L : 0.f);
            pk.v[2] = from_f32<T>(some ? acc.z / L : 0.f);
            pk.v[3] = from_f32<T>(some ? acc.w / L : 0.f);
            *reinterpret_cast<Pack4<T>*>(reinterpret_cast<T*>(p.o) + ph * D + d) = pk;
        }
        if (p.shard_o) {
            *reinterpret_cast<float4*>(p.shard_o + ph * D + d) = acc;
            if (d == 0) {
                p.shard_m[ph] = M;
                p.shard_l[ph] = L;
            }
        }
    };
    if (p.cluster <= 1) {
        __syncthreads();
        for (int u = threadIdx.x; u < units; u += blockDim.x) {
            const int hg = u >> qshift, d = (u - (hg << qshift)) * 4;
            const float4 acc = *reinterpret_cast<const float4*>(cta_o + (size_t)hg * D + d);
            const float M = cta_ml[2 * hg], L = cta_ml[2 * hg + 1];
            if (p.nchunks == 1) {
                put_final(hg, d, acc, M, L);
            } else {
                const size_t ph = (size_t)b * p.Hq + qh0 + hg;
                *reinterpret_cast<float4*>(p.part_o + (ph * p.nchunks + chunk) * D + d) = acc;
                if (d == 0) *reinterpret_cast<float2*>(p.part_ml + (ph * p.nchunks + chunk) * 2) = make_float2(M, L);
            }
        }
        return;
    }
    cg::cluster_group cluster = cg::this_cluster();
    const int CS = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int HG = HC * G;
    const int per = (units + CS - 1) / CS;            // float4 units each CTA finishes
    float2* recv_ml = reinterpret_cast<float2*>(recv + (size_t)CS * per * 4);     // [CS][HG], after [CS][per] float4
    __syncthreads();                                  // this CTA's block is complete
    cluster_wait();                                   // every CTA of the cluster has started (arrived at its top)
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
        const int dest = u / per, local = u - dest * per;
        float* dst = cluster.map_shared_rank(recv, dest) + ((size_t)rank * per + local) * 4;
        *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(cta_o + (size_t)u * 4);
    }
    for (int i = threadIdx.x; i < HG * CS; i += blockDim.x) {
        const int dest = i / HG, hg = i - dest * HG;
        cluster.map_shared_rank(recv_ml, dest)[rank * HG + hg] = make_float2(cta_ml[2 * hg], cta_ml[2 * hg + 1]);
    }
    if (threadIdx.x == 0) TIDAL_STAMP(9);
    cluster.sync();                                   // release / acquire: everything pushed to this CTA has landed
    if (threadIdx.x == 0) TIDAL_STAMP(10);
    const int hi = min(units, (rank + 1) * per);
    const int NS = p.nsuper, sup = chunk / CS;         // clusters on this list, and which of them this is
    for (int u = rank * per + threadIdx.x; u < hi; u += blockDim.x) {
        const int hg = u >> qshift, d = (u - (hg << qshift)) * 4, local = u - rank * per;
        float M = -INFINITY, L = 0.f;
        for (int r = 0; r < CS; ++r) M = fmaxf(M, recv_ml[r * HG + hg].x);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < CS; ++r) {
            const float2 ml = recv_ml[r * HG + hg];
            const float w = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - M);
            const float4 v = *reinterpret_cast<const float4*>(recv + ((size_t)r * per + local) * 4);
            acc.x = fmaf(w, v.x, acc.x);
            acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z);
            acc.w = fmaf(w, v.w, acc.w);
            L = fmaf(w, ml.y, L);
        }
        if (NS <= 1) {
            put_final(hg, d, acc, M, L);
        } else {
            const size_t ph = (size_t)b * p.Hq + qh0 + hg;
            __stcg(reinterpret_cast<float4*>(p.part_o + (ph * NS + sup) * D + d), acc);
            if (d == 0) __stcg(reinterpret_cast<float2*>(p.part_ml + (ph * NS + sup) * 2), make_float2(M, L));
        }
    }
    if (threadIdx.x == 0) TIDAL_STAMP(11);
    if (NS <= 1) return;
    // Several clusters on one list: CTA `rank` of each holds the same share of the outputs.  The last of them to
    // arrive (one counter per list and rank, left at zero again) merges the shares of all and writes the result.
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t* cnt = p.xc_count + ((size_t)b * gridDim.y + blockIdx.y) * kMaxCluster + rank;
        const uint32_t seen = atomicAdd(cnt, 1u);
        s_last = seen == (uint32_t)NS - 1u;
        if (s_last) *cnt = 0u;
        __threadfence();
    }
    __syncthreads();
    if (!s_last) return;
    for (int u = rank * per + threadIdx.x; u < hi; u += blockDim.x) {
        const int hg = u >> qshift, d = (u - (hg << qshift)) * 4;
        const size_t ph = (size_t)b * p.Hq + qh0 + hg;
        float M = -INFINITY, L = 0.f;
        for (int c = 0; c < NS; ++c) M = fmaxf(M, __ldcg(p.part_ml + (ph * NS + c) * 2));
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = 0; c < NS; ++c) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (ph * NS + c) * 2));
            const float w = (ml.x == -INFINITY) ? 0.f : fast_exp2(ml.x - M);
            const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + (ph * NS + c) * D + d));
            acc.x = fmaf(w, v.x, acc.x);
            acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z);
            acc.w = fmaf(w, v.w, acc.w);
            L = fmaf(w, ml.y, L);
        }
        put_final(hg, d, acc, M, L);
    }
}

// Tensor-core kernel (decode_attn_mma.cu): 16-bit storage, up to 16 query heads per
// KV head, HC in {1,2,4,8} KV heads per CTA, 8 consumer warps.
constexpr int kMmaWarps = 8;
constexpr int kMmaTile = 16;            // tokens one warp takes from a stage
constexpr int kMmaMaxProducers = 2;
size_t attn_mma_smem_bytes(int S, int HC, int G, int D, bool sum_heads);
int launch_attn_mma(const AttnParams& p, int D, int dtype, dim3 grid, size_t smem, cudaStream_t st, int* query);

}  // namespace tidal
