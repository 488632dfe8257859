// All-gather of one small block per rank over NVLink peer stores, for the per-layer exchange of
// sequence-sharded decode attention (softmax partials and top-k candidates: a few KB to a few MB).
// A collective library launch costs more than this exchange moves in time; here every rank's kernel
//   1. stores its block into its slot of every peer's staging buffer (plain peer stores through
//      pointers the host obtained by exchanging memory handles; no multicast),
//   2. fences, and adds 1 to its arrival counter on every peer (one add per CTA),
//   3. waits — with an iteration limit — until every rank's counter on this GPU shows all CTAs of the
//      current exchange, and
//   4. copies the staged blocks into the caller's receive buffer, which the kernels that follow in the
//      stream read with fixed addresses (the same graph can be replayed), and — if asked — merges the
//      ranks' softmax partials (m, l, o) found in the blocks into the attention output on the spot, so
//      that the exchange of a sparse layer is followed by no merge launch at all.
// Staging and counters are double-buffered by the parity of an exchange counter kept in device memory
// and advanced by the last CTA to finish, so nothing is reset between exchanges: a rank can be at most
// one exchange ahead of another, because it needs the other's arrivals to finish the one in between.
// The number of CTAs follows from slot_bytes alone — a property of the buffers, not of the call — so
// that the arrivals expected per exchange are the same whatever each exchange carries: calls that move
// fewer bytes than a slot holds (a sparse layer sends only partials, a selection layer also its
// candidates) may be mixed freely on one set of buffers.
#include "common.cuh"

namespace tidal {

constexpr int kXchgThreads = 256;
constexpr int kXchgMaxCtas = 32;
constexpr int kXchgMaxWorld = 16;
constexpr uint32_t kXchgSpinLimit = 1u << 22;    // default wait limit (about half a second)

// CTAs of every exchange on buffers with slots of slot_vec 16-byte vectors
__host__ __device__ inline int exchange_ctas(int64_t slot_vec) {
    int64_t c = (slot_vec + kXchgThreads - 1) / kXchgThreads;
    return (int)(c < 1 ? 1 : (c > kXchgMaxCtas ? kXchgMaxCtas : c));
}

struct ExchangeParams {
    const uint4* send;
    int64_t nvec;                 // 16-byte vectors in a block
    int64_t slot_vec;             // vectors between the blocks of two ranks (staging and receive buffer alike)
    uint4* const* peer_stage;     // [world]: every rank's staging buffer [2][world][slot_vec], as mapped on this GPU
    uint32_t* const* peer_count;  // [world]: every rank's arrival counters [2][world]
    uint4* out;                   // local receive buffer [world][slot_vec]
    uint32_t* epoch;              // local: exchanges completed
    uint32_t* fin;                // local: CTAs of the current exchange that are done
    uint32_t* status;
    uint32_t spin_limit;          // iterations a CTA polls for the other ranks before it gives up
    int rank, world;
    // optional merge of the ranks' softmax partials: fp32 word offsets of m [rows], l [rows], o [rows][D] in a block
    void* merge_out;
    int64_t m_off, l_off, o_off;
    int merge_rows, merge_dim, merge_dtype;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kXchgThreads) peer_all_gather_kernel(const ExchangeParams p) {
    pdl_wait();
    pdl_launch_dependents();
    // every CTA reads the counter before the last one to finish advances it
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1u;
    const int par = (int)(e & 1u);
    const uint32_t target = ((e + 1u) / 2u) * gridDim.x;          // arrivals per rank after this exchange, for this parity
    const int64_t stride = (int64_t)gridDim.x * kXchgThreads;
    const int64_t first = (int64_t)blockIdx.x * kXchgThreads + threadIdx.x;

    // 1. this rank's block into its slot on every peer
    const int64_t my_slot = ((int64_t)par * p.world + p.rank) * p.slot_vec;
    for (int64_t i = first; i < p.nvec; i += stride) {
        const uint4 v = p.send[i];
        for (int r = 0; r < p.world; ++r) p.peer_stage[r][my_slot + i] = v;
    }
    // 2. the stores of the whole CTA are ordered before its arrival
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < p.world) atomicAdd_system(&p.peer_count[threadIdx.x][par * p.world + p.rank], 1u);

    // 3. wait for every rank's arrivals on this GPU (bounded: a missing rank becomes a status bit, not a hang)
    if ((int)threadIdx.x < p.world) {
        const uint32_t* c = &p.peer_count[p.rank][par * p.world + threadIdx.x];
        bool ok = false;
        for (uint32_t it = 0; it < p.spin_limit; ++it) {
            if ((int32_t)(ld_acquire_sys(c) - target) >= 0) {
                ok = true;
                break;
            }
            if (it > 64) __nanosleep(64);
        }
        if (!ok && p.status) atomicOr(p.status, TIDAL_DEV_WAIT_TIMEOUT);
    }
    __syncthreads();
    __threadfence_system();

    // 4. staged blocks into the receive buffer
    const uint4* stage = p.peer_stage[p.rank] + (int64_t)par * p.world * p.slot_vec;
    if (p.out)
        for (int r = 0; r < p.world; ++r)
            for (int64_t i = first; i < p.nvec; i += stride) p.out[(int64_t)r * p.slot_vec + i] = stage[(int64_t)r * p.slot_vec + i];
    //    and the merge of the ranks' partials, in rank order (the arithmetic of merge_shards_kernel)
    if (p.merge_out) {
        const float* st = reinterpret_cast<const float*>(stage);
        const int64_t slot_words = p.slot_vec * 4;
        const int64_t total = (int64_t)p.merge_rows * p.merge_dim;
        for (int64_t idx = first; idx < total; idx += stride) {
            const int64_t r = idx / p.merge_dim;
            const int d = (int)(idx - r * p.merge_dim);
            float M = -INFINITY;
            for (int s = 0; s < p.world; ++s) M = fmaxf(M, st[s * slot_words + p.m_off + r]);
            float acc = 0.f, L = 0.f;
            for (int s = 0; s < p.world; ++s) {
                const float ms = st[s * slot_words + p.m_off + r];
                const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
                acc = fmaf(w, st[s * slot_words + p.o_off + r * p.merge_dim + d], acc);
                L = fmaf(w, st[s * slot_words + p.l_off + r], L);
            }
            const float v = L > 0.f ? acc / L : 0.f;
            if (p.merge_dtype == TIDAL_DTYPE_F16) reinterpret_cast<__half*>(p.merge_out)[idx] = __float2half_rn(v);
            else if (p.merge_dtype == TIDAL_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(p.merge_out)[idx] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(p.merge_out)[idx] = v;
        }
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.fin, 1u) == gridDim.x - 1) {
            *p.fin = 0;
            *reinterpret_cast<volatile uint32_t*>(p.epoch) = e;
        }
    }
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_peer_all_gather(const tidal_exchange_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_send && a->d_peer_stage && a->d_peer_count && a->d_state, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(a->d_recv || a->d_merge_out, TIDAL_ERR_ARG, "neither a receive buffer nor a merge output given");
    if (a->d_merge_out) {
        TIDAL_REQUIRE(a->merge_rows >= 1 && a->merge_head_dim >= 1 && a->merge_dtype >= 0 && a->merge_dtype <= 2, TIDAL_ERR_ARG,
                      "bad merge geometry");
        const int64_t words = a->bytes / 4;
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
    ExchangeParams p;
    p.send = (const uint4*)a->d_send;
    p.nvec = a->bytes / 16;
    p.slot_vec = a->slot_bytes / 16;
    p.peer_stage = (uint4* const*)a->d_peer_stage;
    p.peer_count = (uint32_t* const*)a->d_peer_count;
    p.out = (uint4*)a->d_recv;
    p.epoch = a->d_state;
    p.fin = a->d_state + 1;
    p.status = a->d_status;
    p.spin_limit = a->wait_limit > 0 ? (uint32_t)a->wait_limit : kXchgSpinLimit;
    p.rank = a->rank;
    p.world = a->world;
    p.merge_out = a->d_merge_out;
    p.m_off = a->merge_m_off; p.l_off = a->merge_l_off; p.o_off = a->merge_o_off;
    p.merge_rows = a->merge_rows; p.merge_dim = a->merge_head_dim; p.merge_dtype = a->merge_dtype;
    // the CTA count follows from the slot size alone: the same for every call on these buffers, on every rank
    const int ctas = exchange_ctas(p.slot_vec);
    TIDAL_CUDA_OK(launch_pdl(peer_all_gather_kernel, dim3((unsigned)ctas), dim3(kXchgThreads), 0, (cudaStream_t)stream, 1, p));
    count_launch();
    return TIDAL_OK;
}

extern "C" int tidal_peer_exchange_ctas(int64_t slot_bytes) {
    if (slot_bytes <= 0 || slot_bytes % 16) return TIDAL_ERR_ARG;
    return exchange_ctas(slot_bytes / 16);
}

extern "C" int tidal_peer_exchange_reset(uint32_t* d_count, uint32_t* d_state, int world, void* stream) {
    TIDAL_REQUIRE(d_count && d_state, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(world >= 2 && world <= kXchgMaxWorld, TIDAL_ERR_ARG, "bad world %d (2..%d ranks)", world, kXchgMaxWorld);
    TIDAL_CUDA_OK(cudaMemsetAsync(d_count, 0, sizeof(uint32_t) * 2 * world, (cudaStream_t)stream));
    TIDAL_CUDA_OK(cudaMemsetAsync(d_state, 0, sizeof(uint32_t) * 2, (cudaStream_t)stream));
    return TIDAL_OK;
}
