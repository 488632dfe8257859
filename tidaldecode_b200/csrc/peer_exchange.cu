// All-gather of one small block per rank over NVLink peer stores, for the per-layer exchange of
// sequence-sharded decode attention (softmax partials and top-k candidates: a few KB to a few MB), with
// what follows the exchange done in the same launch.  A collective library launch costs more than this
// exchange moves in time; here every rank's kernel
//   1. stores its block into its slot of every peer's staging buffer (plain peer stores through
//      pointers the host obtained by exchanging memory handles; no multicast),
//   2. publishes, per CTA, the number of the current exchange in that CTA's flag word on every peer (one
//      releasing store per peer: no atomics, no second level of signalling),
//   3. waits — with an iteration limit — until the flags of every CTA of every rank on this GPU show the
//      current exchange, and
//   4. works on the staged blocks in place: copies them to the caller's receive buffer (if one is given),
//      merges the ranks' softmax partials (m, l, o) into the attention output (if asked), and ranks the
//      ranks' top-k candidates into the global selection, keeping the positions this rank owns (if asked:
//      the one-CTA form of the top-k, one row per CTA), so that a selection layer is attention -> local
//      top-k -> this launch, and a sparse layer attention -> this launch.
// Staging and counters are double-buffered by the parity of an exchange counter kept in device memory
// and advanced by the last CTA to finish, so nothing is reset between exchanges: a rank can be at most
// one exchange ahead of another, because it needs the other's arrivals to finish the one in between.
// Flags carry exchange numbers, not counts: a call waits for the flags of as many CTAs per rank as it runs
// itself (every rank passes the same arguments, hence launches the same grid), so calls of different sizes
// and grids may follow each other on one set of buffers, and a flag that arrives twice or late harms nothing.
#include "topk_common.cuh"

namespace tidal {

constexpr int kXchgThreads = kTopkThreads;       // 1024: the candidate ranking is the top-k's one-CTA form
constexpr int kXchgMaxCtas = TIDAL_XCHG_MAX_CTAS;  // all resident at once (one CTA per SM), so no CTA waits for an SM
constexpr int kXchgMaxWorld = 16;
constexpr uint32_t kXchgSpinLimit = 1u << 22;    // default wait limit (about half a second)

struct ExchangeParams {
    const uint4* send;
    int64_t nvec;                 // 16-byte vectors in a block
    int64_t slot_vec;             // vectors between the blocks of two ranks (staging and receive buffer alike)
    uint4* const* peer_stage;     // [world]: every rank's staging buffer [2][world][slot_vec], as mapped on this GPU
    uint32_t* const* peer_count;  // [world]: every rank's flag words [2][world][kXchgMaxCtas]
    uint4* out;                   // local receive buffer [world][slot_vec], or nullptr
    uint32_t* state;              // local: [0] exchanges completed, [1] CTAs done, [2] unused, [3] status sink
    uint32_t* status;
    uint32_t spin_limit;          // iterations a CTA polls for the other ranks before it gives up
    int rank, world;
    // optional merge of the ranks' softmax partials: fp32 word offsets of m [rows], l [rows], o [rows][D] in a block
    void* merge_out;
    int64_t m_off, l_off, o_off;
    int merge_rows, merge_dim, merge_dtype;
    // optional ranking of the ranks' candidates: scores [rows][k] fp32 and positions [rows][k] int32 at these word
    // offsets of a block; per row the `select` best of the world * k, those in [own_lo, own_hi) written as
    // position - own_lo to sel_out[row][...] in ascending order, their number to sel_count[row]
    int cand_rows, cand_k, cand_select;
    int64_t cs_off, ci_off;
    int32_t own_lo, own_hi;
    int32_t* sel_out;
    int64_t sel_stride;
    int32_t* sel_count;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kXchgThreads) peer_all_gather_kernel(const ExchangeParams p) {
    extern __shared__ __align__(16) unsigned char xsm[];      // kClusterSmem bytes when candidates are ranked
    pdl_wait();
    pdl_launch_dependents();
    // every CTA reads the counter before the last one to finish advances it
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(&p.state[0]) + 1u;
    const int par = (int)(e & 1u);
    const int64_t stride = (int64_t)gridDim.x * kXchgThreads;
    const int64_t first = (int64_t)blockIdx.x * kXchgThreads + threadIdx.x;

    // 1. this rank's block into its slot on every peer
    const int64_t my_slot = ((int64_t)par * p.world + p.rank) * p.slot_vec;
    for (int64_t i = first; i < p.nvec; i += stride) {
        const uint4 v = p.send[i];
        for (int r = 0; r < p.world; ++r) p.peer_stage[r][my_slot + i] = v;
    }
    // 2. this CTA's flag on every peer: the barrier orders the CTA's stores before the releasing stores of the
    //    lanes that publish (a release is cumulative over what its thread has observed), one lane per peer
    __syncthreads();
    if ((int)threadIdx.x < p.world)
        st_release_sys(&p.peer_count[threadIdx.x][((size_t)par * p.world + p.rank) * kXchgMaxCtas + blockIdx.x], e);

    // 3. wait for the flags of every CTA of every rank on this GPU (bounded: a missing rank becomes a status bit,
    //    not a hang); the acquiring loads and the barrier order every thread's later reads of the staged blocks
    for (int i = threadIdx.x; i < p.world * (int)gridDim.x; i += kXchgThreads) {
        const int r = i / (int)gridDim.x, c = i - r * (int)gridDim.x;
        const uint32_t* f = &p.peer_count[p.rank][((size_t)par * p.world + r) * kXchgMaxCtas + c];
        bool ok = false;
        for (uint32_t it = 0; it < p.spin_limit; ++it) {
            if ((int32_t)(ld_acquire_sys(f) - e) >= 0) {
                ok = true;
                break;
            }
            if (it > 64) __nanosleep(64);
        }
        if (!ok && p.status) atomicOr(p.status, TIDAL_DEV_WAIT_TIMEOUT);
    }
    __syncthreads();

    // 4. staged blocks into the receive buffer
    const uint4* stage = p.peer_stage[p.rank] + (int64_t)par * p.world * p.slot_vec;
    if (p.out)
        for (int r = 0; r < p.world; ++r)
            for (int64_t i = first; i < p.nvec; i += stride) p.out[(int64_t)r * p.slot_vec + i] = stage[(int64_t)r * p.slot_vec + i];
    //    the merge of the ranks' partials, in rank order (the arithmetic of merge_shards_kernel); a thread owns four
    //    consecutive output elements when the rows allow 16-byte accesses, and all loads of a rank are independent
    if (p.merge_out) {
        const float* st = reinterpret_cast<const float*>(stage);
        const int64_t slot_words = p.slot_vec * 4;
        const int D = p.merge_dim;
        const bool vec = (D % 4 == 0) && (p.o_off % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.merge_out) & 15) == 0);
        const int lanes = vec ? D / 4 : D;                 // work items per row
        const int64_t total = (int64_t)p.merge_rows * lanes;
        for (int64_t u = first; u < total; u += stride) {
            const int64_t r = u / lanes;
            const int d = (int)(u - r * lanes) * (vec ? 4 : 1);
            float M = -INFINITY;
            for (int s = 0; s < p.world; ++s) M = fmaxf(M, st[s * slot_words + p.m_off + r]);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float L = 0.f;
#pragma unroll 4
            for (int s = 0; s < p.world; ++s) {
                const float ms = st[s * slot_words + p.m_off + r];
                const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
                const float* po = st + s * slot_words + p.o_off + r * D + d;
                if (vec) {
                    const float4 v = *reinterpret_cast<const float4*>(po);
                    acc.x = fmaf(w, v.x, acc.x);
                    acc.y = fmaf(w, v.y, acc.y);
                    acc.z = fmaf(w, v.z, acc.z);
                    acc.w = fmaf(w, v.w, acc.w);
                } else {
                    acc.x = fmaf(w, po[0], acc.x);
                }
                L = fmaf(w, st[s * slot_words + p.l_off + r], L);
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            const float vals[4] = {L > 0.f ? acc.x / L : 0.f, L > 0.f ? acc.y / L : 0.f, L > 0.f ? acc.z / L : 0.f,
                                   L > 0.f ? acc.w / L : 0.f};
            (void)inv;
            const int64_t at = r * D + d;
            const int nout = vec ? 4 : 1;
            if (p.merge_dtype == TIDAL_DTYPE_F16) {
                __half* o = reinterpret_cast<__half*>(p.merge_out) + at;
                if (vec) {
                    *reinterpret_cast<__half2*>(o) = __floats2half2_rn(vals[0], vals[1]);
                    *reinterpret_cast<__half2*>(o + 2) = __floats2half2_rn(vals[2], vals[3]);
                } else o[0] = __float2half_rn(vals[0]);
            } else if (p.merge_dtype == TIDAL_DTYPE_BF16) {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.merge_out) + at;
                if (vec) {
                    *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(vals[0], vals[1]);
                    *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(vals[2], vals[3]);
                } else o[0] = __float2bfloat16_rn(vals[0]);
            } else {
                float* o = reinterpret_cast<float*>(p.merge_out) + at;
                for (int i = 0; i < nout; ++i) o[i] = vals[i];
            }
        }
    }
    //    and the global selection from the ranks' candidates: row r of rank s's block holds cand_k (score, position)
    //    pairs; the row of world * cand_k candidates is ranked in place (segments one block apart), ties towards
    //    the lower rank and place, which is the lower position because ranks hold ascending ranges
    if (p.cand_rows > 0) {
        TopkParams tp;
        const int64_t slot_words = p.slot_vec * 4;
        tp.scores = reinterpret_cast<const float*>(stage) + p.cs_off;
        tp.in_idx = reinterpret_cast<const int32_t*>(stage) + p.ci_off;
        tp.in_idx_stride = p.cand_k;
        tp.rows = p.cand_rows;
        tp.n = (int64_t)p.world * p.cand_k;
        tp.row_stride = p.cand_k;
        tp.k = p.cand_select;
        tp.out_idx = p.sel_out;
        tp.out_val = nullptr;
        tp.out_stride = p.sel_stride;
        tp.idx_offset = 0;
        tp.force_last = 0;
        tp.own_lo = p.own_lo;
        tp.own_hi = p.own_hi;
        tp.out_count = p.sel_count;
        tp.hist = nullptr;
        tp.row_state = nullptr;
        tp.cand = nullptr;
        tp.sel = nullptr;
        tp.cand_cap = 0;
        tp.status = p.status ? p.status : &p.state[3];
        tp.seg_len = p.cand_k;
        tp.seg_stride = slot_words;
        tp.row_len = nullptr;
        for (int row = blockIdx.x; row < p.cand_rows; row += gridDim.x) {
            // the candidates' order is the positions' order: threshold, then one ordered pass (no winners' list, no sort)
            if (!topk_ordered_row(tp, row, xsm)) {
                __syncthreads();
                topk_cluster_row(tp, row, xsm);          // a threshold bin too crowded for shared memory
            }
            __syncthreads();
        }
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1) {
            p.state[1] = 0;
            *reinterpret_cast<volatile uint32_t*>(&p.state[0]) = e;
        }
    }
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_peer_all_gather(const tidal_exchange_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_send && a->d_peer_stage && a->d_peer_count && a->d_state, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(a->d_recv || a->d_merge_out || a->cand_rows > 0, TIDAL_ERR_ARG,
                  "nothing to do: no receive buffer, no merge output, no candidates to rank");
    const int64_t words = a->bytes / 4;
    if (a->d_merge_out) {
        TIDAL_REQUIRE(a->merge_rows >= 1 && a->merge_head_dim >= 1 && a->merge_dtype >= 0 && a->merge_dtype <= 2, TIDAL_ERR_ARG,
                      "bad merge geometry");
        TIDAL_REQUIRE(a->merge_m_off >= 0 && a->merge_m_off + a->merge_rows <= words && a->merge_l_off >= 0 &&
                          a->merge_l_off + a->merge_rows <= words && a->merge_o_off >= 0 &&
                          a->merge_o_off + (int64_t)a->merge_rows * a->merge_head_dim <= words,
                      TIDAL_ERR_ARG, "the partials lie outside the exchanged bytes");
    }
    TIDAL_REQUIRE(a->world >= 2 && a->world <= kXchgMaxWorld && a->rank >= 0 && a->rank < a->world, TIDAL_ERR_ARG,
                  "bad rank %d / world %d (2..%d ranks)", a->rank, a->world, kXchgMaxWorld);
    TIDAL_REQUIRE(a->bytes > 0 && a->bytes % 16 == 0 && a->slot_bytes % 16 == 0 && a->bytes <= a->slot_bytes, TIDAL_ERR_ARG,
                  "bytes (%lld) and slot_bytes (%lld) must be multiples of 16, bytes <= slot_bytes", (long long)a->bytes,
                  (long long)a->slot_bytes);
    TIDAL_REQUIRE((((uintptr_t)a->d_send | (uintptr_t)a->d_recv) & 15) == 0, TIDAL_ERR_ARG, "send and recv must be 16-byte aligned");
    TIDAL_REQUIRE(a->wait_limit >= 0, TIDAL_ERR_ARG, "negative wait_limit");
    TIDAL_REQUIRE(a->cand_rows >= 0, TIDAL_ERR_ARG, "negative cand_rows");
    if (a->cand_rows > 0) {
        const int64_t n = (int64_t)a->world * a->cand_k, per = (int64_t)a->cand_rows * a->cand_k;
        TIDAL_REQUIRE(a->cand_k >= 1 && a->cand_select >= 1 && a->cand_select < n, TIDAL_ERR_ARG,
                      "candidates: need 1 <= cand_select (%d) < world * cand_k (%lld)", a->cand_select, (long long)n);
        TIDAL_REQUIRE(a->cand_select <= kClusterMaxK && n <= kClusterSmemCandMaxN, TIDAL_ERR_ARG,
                      "candidates are ranked in shared memory: cand_select <= %d and world * cand_k <= %lld (rank larger sets "
                      "with tidal_topk on the receive buffer)", kClusterMaxK, (long long)kClusterSmemCandMaxN);
        TIDAL_REQUIRE(a->cand_score_off >= 0 && a->cand_score_off + per <= words && a->cand_idx_off >= 0 &&
                          a->cand_idx_off + per <= words, TIDAL_ERR_ARG, "the candidates lie outside the exchanged bytes");
        TIDAL_REQUIRE(a->d_sel_out != nullptr && a->sel_stride >= a->cand_select, TIDAL_ERR_ARG,
                      "candidates need d_sel_out with sel_stride >= cand_select");
    }
    ExchangeParams p;
    p.send = (const uint4*)a->d_send;
    p.nvec = a->bytes / 16;
    p.slot_vec = a->slot_bytes / 16;
    p.peer_stage = (uint4* const*)a->d_peer_stage;
    p.peer_count = (uint32_t* const*)a->d_peer_count;
    p.out = (uint4*)a->d_recv;
    p.state = a->d_state;
    p.status = a->d_status;
    p.spin_limit = a->wait_limit > 0 ? (uint32_t)a->wait_limit : kXchgSpinLimit;
    p.rank = a->rank;
    p.world = a->world;
    p.merge_out = a->d_merge_out;
    p.m_off = a->merge_m_off; p.l_off = a->merge_l_off; p.o_off = a->merge_o_off;
    p.merge_rows = a->merge_rows; p.merge_dim = a->merge_head_dim; p.merge_dtype = a->merge_dtype;
    p.cand_rows = a->cand_rows; p.cand_k = a->cand_k; p.cand_select = a->cand_select;
    p.cs_off = a->cand_score_off; p.ci_off = a->cand_idx_off;
    p.own_lo = a->own_lo; p.own_hi = a->own_hi;
    p.sel_out = a->d_sel_out; p.sel_stride = a->sel_stride; p.sel_count = a->d_sel_count;
    // a CTA per candidate row, enough CTAs to move the block in two passes and to merge two outputs per thread;
    // all resident at once
    int64_t ctas = (p.nvec + 2 * kXchgThreads - 1) / (2 * kXchgThreads);
    if (ctas < a->cand_rows) ctas = a->cand_rows;
    if (a->d_merge_out) {
        const int64_t by_merge = ((int64_t)a->merge_rows * a->merge_head_dim / 4 + kXchgThreads - 1) / kXchgThreads;   // one float4 per thread
        if (ctas < by_merge) ctas = by_merge;
    }
    if (ctas < 1) ctas = 1;
    if (ctas > kXchgMaxCtas) ctas = kXchgMaxCtas;
    const size_t smem = a->cand_rows > 0 ? kClusterSmem : 0;
    TIDAL_CUDA_OK(cudaFuncSetAttribute(peer_all_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kClusterSmem));
    TIDAL_CUDA_OK(launch_pdl(peer_all_gather_kernel, dim3((unsigned)ctas), dim3(kXchgThreads), smem, (cudaStream_t)stream, 1, p));
    count_launch();
    return TIDAL_OK;
}

extern "C" int tidal_peer_exchange_reset(uint32_t* d_count, uint32_t* d_state, int world, void* stream) {
    TIDAL_REQUIRE(d_count && d_state, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(world >= 2 && world <= kXchgMaxWorld, TIDAL_ERR_ARG, "bad world %d (2..%d ranks)", world, kXchgMaxWorld);
    TIDAL_CUDA_OK(cudaMemsetAsync(d_count, 0, sizeof(uint32_t) * 2 * world * kXchgMaxCtas, (cudaStream_t)stream));
    TIDAL_CUDA_OK(cudaMemsetAsync(d_state, 0, sizeof(uint32_t) * 4, (cudaStream_t)stream));
    return TIDAL_OK;
}
