// Causal attention of a block of new query rows over one sequence's paged KV ("prefill"), on the
// 5th-generation tensor cores: tcgen05.mma with operands in shared memory (Q, K, V) and in tensor memory (P)
// and the accumulators in tensor memory.  Takes the place of prefill_with_paged_kv_cache (tidal/ops/csrc/batch_prefill.cu:27-117,
// kernels/include/prefill/prefill.cuh:688-870, an mma.sync kernel).
//
// A row block = 128 query rows of one query head = the 128 lanes of tensor memory; a CTA holds one row
// block (short calls) or two that share every K/V tile.  It walks the KV tokens its rows may see in
// tiles of 128.  Per row block and tile:
//   S = Q K^T     8 (D=128) MMAs of 128x128x16, Q and K as K-major operands in shared memory with the
//                 128-byte swizzle, S (fp32) in the row block's 128 S columns of tensor memory
//   softmax       thread t owns row t (tcgen05.ld 32x32b: lane = row) and holds its 128 S values in registers
//                 (the softmax warps take registers from the other warps: setmaxnreg); P = exp2(..) rounded
//                 to the storage type goes back into the first 64 of the S columns (two values per column),
//                 running sum in registers
//   O += P V      8 MMAs of 128xDx16 with P as the A operand read from tensor memory and V rows as they
//                 lie in the cache (MN-major B operand); O stays in tensor memory and is rescaled only
//                 when a row's maximum has grown by more than 2^8
// S is single-buffered per row block (512 columns = 2 x (128 S + 128 O)), so a row block's chain is
// softmax_j -> PV_j -> QK_(j+1) -> softmax_(j+1); the two row blocks of a CTA run half a period apart and
// keep the tensor core busy during each other's softmax.  K and V tiles travel through one ring of five
// 32 KB slots in the order K_0 V_0 K_1 V_1 ..., fetched by dedicated warps (cp.async, 16 bytes per
// request; a warp of its own looks the page ids of a tile's rows up two tiles ahead and parks them in a small
// table in shared memory).
// Every wait on an mbarrier is bounded; a CTA that gives up sets TIDAL_DEV_WAIT_TIMEOUT, still frees its
// tensor memory and returns.
#include <cmath>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"

namespace tidal {

constexpr int kPfRows = 128;     // query rows per CTA = MMA M = TMEM lanes
constexpr int kPfTile = 128;     // KV tokens per tile
constexpr int kPfRing = 5;       // K/V tiles in flight in shared memory
#ifndef TIDAL_PF_LAG
#define TIDAL_PF_LAG 1
#endif
constexpr int kPfProducerWarps = 8;   // warps that fetch K and V tiles: a warp keeps only so many copies in flight, the rate grows with the warps
constexpr int kPfExtraThreads = 32 * kPfProducerWarps + 128;  // warp groups beside the softmax threads: the producer warps; the MMA warp, the lookup warp and two spares
// Registers per thread after the role split (setmaxnreg, a warp-group operation).  The softmax threads hold a whole
// S row of 128 values and take registers from the other warps.  A CTA starts with `launch` registers per thread
// (what the launch bound leaves: the register file divided by the threads, rounded down to 8; ptxas reports the
// same figure as "Used N registers"), the auxiliary groups give back down to `aux`, the softmax groups grow to
// `softmax`; the static_assert keeps the request inside what was given back, so that no setmaxnreg.inc can wait
// for registers that never come.
template <int SUB>
struct PfRegs {
    static constexpr int threads = 128 * SUB + kPfExtraThreads;
    static constexpr int launch = 65536 / threads / 8 * 8;
    static constexpr int softmax = SUB == 2 ? 176 : 200, aux = SUB == 2 ? 40 : 96;
    static_assert((launch - aux) * kPfExtraThreads >= (softmax - launch) * 128 * SUB, "register pool");
    static_assert(softmax >= launch && aux <= launch, "setmaxnreg direction");
};

struct PrefillParams {
    const void* q;        // [n_q][Hq][D]
    void* o;              // [n_q][Hq][D]
    const void* kv;       // [pages][2][page_size][Hkv][D]
    const int32_t* pages; // page ids of this sequence, in order
    uint32_t* status;
    int64_t kv_len;
    int64_t num_pages;    // pages in the pool: a table entry outside [0, num_pages) is skipped (zero rows) and reported
    int n_q, Hq, Hkv, page_size;
    int ps_shift;         // log2(page_size) when that is a power of two, else -1 (the kernels then divide)
    int causal;
    float scale_log2;     // softmax scale x log2(e)
};

// ------------------------------------------------------------------ tcgen05 wrappers
__device__ __forceinline__ void tc_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// A operand in tensor memory (lane = row, two 16-bit values of consecutive k per column), B through a descriptor
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
template <uint32_t N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Shared-memory operand descriptor, 128-byte swizzle, atoms of 8 rows x 128 bytes (1024-byte aligned).
//   K-major operand (rows = M or N, 64 elements of K per row): `sbo` = bytes between 8-row groups.
//   MN-major operand (rows = K, 64 elements of M/N per row): `sbo` = bytes between 8-row (K) groups,
//   `lbo` = bytes between blocks of 64 elements along M/N.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version of this architecture
    d |= (uint64_t)2 << 61;   // 128-byte swizzle
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulator, A K-major, B K- or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int dtype_bf16, int b_mn_major, int M, int N) {
    return (1u << 4) | ((uint32_t)dtype_bf16 << 7) | ((uint32_t)dtype_bf16 << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Byte offset of the 16-byte chunk `c16` of row `r` in an operand tile of `rows` rows: blocks of 64
// elements (8 chunks) are stored one after the other, each [rows][128 bytes] with the chunk index
// XOR-ed with the row's low 3 bits (what the 128-byte swizzle of the descriptor expects).
__device__ __forceinline__ uint32_t sw128_offset(int rows, int r, int c16) {
    return (uint32_t)((c16 >> 3) * rows * 128 + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}

// Waits of this kernel: mbarrier.try_wait with a suspend-time hint, so that a waiting warp sleeps in hardware
// until the phase completes (or the hint runs out) instead of polling — a polling warp takes issue slots
// from the warps it is waiting for.  Bounded: 2^15 tries of 16 us; on expiry the wait raises *abort_flag
// (every other wait of the CTA then returns at once) and ORs TIDAL_DEV_WAIT_TIMEOUT into *status.
__device__ __forceinline__ bool mbar_try_wait_suspended(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mma_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
    for (uint32_t i = 0; i < (1u << 15); ++i) {
        if (mbar_try_wait_suspended(bar, parity, 16384u)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicOr(status, TIDAL_DEV_WAIT_TIMEOUT);
    return false;
}

// Two-wide fp32 arithmetic and the three-input maximum of this architecture: the softmax warps are short of issue
// slots, and these halve the multiply-adds, the additions and the comparisons per score.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// A wait whose outcome the whole warp agrees on: a lane that gave up must not leave the others in the loop.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
    return __all_sync(0xffffffffu, mma_wait(bar, parity, abort_flag, status));
}

// Roles (warp-specialised; nothing in the loop is a block-wide barrier):
//   warps [0, 4 SUB)          softmax: thread t owns query row t of the CTA (lane of tensor memory = row)
//   the next eight warps      producers: page lookups and cp.async of the K and V tiles into the ring
//   the next warp             issues every tcgen05.mma (one lane) and commits them to the barriers below
//   the next warp             looks up the page ids of each tile's rows, two tiles ahead of the copies
//   the last two warps        only complete the warp group (setmaxnreg is a warp-group operation)
// Barriers (mbarrier; the i-th completion of a barrier is waited for with parity i & 1):
//   full[5], empty[5]         ring slots, tile i of the sequence K_0 V_0 K_1 V_1 ... uses slot i % 5:
//                             producers -> MMA warp (one arrival per producer warp, after the copies have landed and
//                             been made visible to the async proxy); tcgen05.commit after the last MMA that reads
//                             the slot -> producers
//   sfull[SUB]                commit after QK_t of a row block -> its softmax warps: S_t is complete (and, the pipe
//                             being in order, so is PV_(t-1): O may be rescaled)
//   pfull[SUB]                softmax warps -> MMA warp: P_t is in tensor memory, O has been rescaled if it had to be
//                             (4 arrivals)
//   pvdone[SUB]               commit after PV_t: awaited before the epilogue reads O
//   alldone                   commit at the very end: no MMA is in flight when tensor memory is freed
//   idsfull[2], idsempty[2]   lookup warp <-> producers: the page ids of tile t are in table t & 1 / every producer warp
//                             has read them (one arrival per producer warp)
template <typename T, int D, int SUB>
__global__ void __launch_bounds__(128 * SUB + kPfExtraThreads, 1) prefill_attn_kernel(const __grid_constant__ PrefillParams p) {
    constexpr int kSoftmaxThreads = 128 * SUB, kProducerThreads = 32 * kPfProducerWarps, kRows = kPfRows * SUB;
    constexpr int kChunks = D / 8;                    // 16-byte chunks per row
    constexpr uint32_t kQBytes = kPfRows * D * 2, kTileBytes = kPfTile * D * 2;
    constexpr uint32_t kSubCols = kPfTile + D;        // tensor-memory columns of one row block: S (P in its first half), then O
    constexpr uint32_t kTmemCols = SUB * kSubCols <= 256 ? 256 : 512;
    constexpr int kFull = 0, kEmpty = kPfRing, kSFull = 2 * kPfRing, kPFull = kSFull + SUB, kPvDone = kPFull + SUB,
                  kAllDone = kPvDone + SUB, kIdsFull = kAllDone + 1, kIdsEmpty = kIdsFull + 2, kNumBars = kIdsEmpty + 2;
    static_assert(kNumBars * 8 + 8 <= 256, "barrier block");
    static_assert(32 % kChunks == 0 && kPfTile % (kPfProducerWarps * 32 / kChunks) == 0, "producer mapping");
    // No static shared memory: the dynamic segment starts at offset 0 with the alignment the swizzled
    // operand tiles need (224 KB + 256 bytes with two row blocks at D = 128).
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sRing = sQ + SUB * kQBytes;
    uint64_t* bar = reinterpret_cast<uint64_t*>(sRing + kPfRing * kTileBytes);
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bar + kNumBars);
    int& abort_flag = *reinterpret_cast<int*>(&tmem_slot + 1);
    int32_t* pgtab = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(bar) + 256);   // [2][kPfTile] page ids, -1 = row reads as zeros

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_qt = (p.n_q + kRows - 1) / kRows;
    const int qt = n_qt - 1 - (int)blockIdx.x;        // longest rows first
    const int h = blockIdx.y, kvh = h / (p.Hq / p.Hkv);
    const int q0 = qt * kRows;
    const int64_t pos0 = p.kv_len - p.n_q + q0;       // position of row 0 of this CTA
    const int rows_here = min(kRows, p.n_q - q0);
    const int64_t kv_end = p.causal ? min(p.kv_len, pos0 + rows_here) : p.kv_len;   // tokens any row of the CTA sees
    const int n_tiles = (int)((kv_end + kPfTile - 1) / kPfTile);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kNumBars; ++i)
            mbar_init(&bar[i], (i < kEmpty || i >= kIdsEmpty) ? (uint32_t)kPfProducerWarps : (i >= kPFull && i < kPvDone) ? 4u : 1u);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tc_alloc(&tmem_slot, kTmemCols);
        tc_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_wait();
    pdl_launch_dependents();
    bool bad_page = false;

    if (tid < kSoftmaxThreads) {
        // ================================================================== softmax: one thread per query row
        reg_inc<PfRegs<SUB>::softmax>();
        const int sub = warp >> 2;
        const uint32_t t_s = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)sub * kSubCols;   // this thread's lane: S columns of its row block
        const uint32_t t_o = t_s + kPfTile;
        uint64_t* sfull = bar + kSFull + sub;
        uint64_t* pfull = bar + kPFull + sub;
        uint64_t* pvdone = bar + kPvDone + sub;
        // The output row stays in tensor memory, scaled by 2^(-m_ref * scale); m_ref follows the running
        // maximum only when that has grown by more than 2^8, so that most tiles need no rescaling pass.
        float m_ref = -INFINITY, l_run = 0.f;
        const int64_t my_pos = pos0 + tid;
        const int64_t lim = p.causal ? min(p.kv_len - 1, my_pos) : p.kv_len - 1;   // last visible token
        bool alive = true;
        for (int j = 0; j < n_tiles; ++j) {
            if (!warp_wait(sfull, (uint32_t)(j & 1), &abort_flag, p.status)) { alive = false; break; }
            tc_fence_after();
            const int64_t t0 = (int64_t)j * kPfTile;
            const bool edge = t0 + kPfTile - 1 > lim;         // some column of this row is masked
            // ---- the whole S row into registers, one wait
            float s[kPfTile];
#pragma unroll
            for (int c0 = 0; c0 < kPfTile; c0 += 32) tc_ld32(t_s + c0, s + c0);
            tc_wait_ld();
            if (edge) {
#pragma unroll
                for (int c = 0; c < kPfTile; ++c) s[c] = (t0 + c <= lim) ? s[c] : -INFINITY;
            }
            float mx4[4] = {m_ref, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < kPfTile; c += 8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) mx4[i] = max3(mx4[i], s[c + i], s[c + 4 + i]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const bool grow = (mx - m_ref) * p.scale_log2 > 8.f;      // also true while m_ref = -inf
            float alpha = 1.f;
            if (grow) {
                alpha = fast_exp2((m_ref - mx) * p.scale_log2);       // 0 for m_ref = -inf
                l_run *= alpha;
                m_ref = mx;
            }
            const float mb = (m_ref == -INFINITY ? 0.f : m_ref) * p.scale_log2;
            // ---- P = exp2(S * scale - m_ref * scale), two values per column, into the first half of the S columns
            const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), negmb2 = pack2(-mb, -mb);
            uint64_t sum2[2] = {0ull, 0ull};         // four running sums, two per register pair
#pragma unroll
            for (int c0 = 0; c0 < kPfTile; c0 += 32) {
                uint32_t w[16];
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    float e[8];
#pragma unroll
                    for (int u = 0; u < 8; u += 2) {
                        float x0, x1;
                        unpack2(fma2(pack2(s[c0 + c8 * 8 + u], s[c0 + c8 * 8 + u + 1]), scale2, negmb2), x0, x1);
                        e[u] = fast_exp2(x0);
                        e[u + 1] = fast_exp2(x1);
                        sum2[(u >> 1) & 1] = add2(sum2[(u >> 1) & 1], pack2(e[u], e[u + 1]));   // fp32 sum of the unrounded weights; P itself is rounded once, by the pack below
                    }
                    const uint4 v = Vec16<T>::from_float(e);
                    w[c8 * 4] = v.x;
                    w[c8 * 4 + 1] = v.y;
                    w[c8 * 4 + 2] = v.z;
                    w[c8 * 4 + 3] = v.w;
                }
                tc_st16(t_s + c0 / 2, w);
            }
            // O row *= alpha in the warps where some row's reference moved (tile 0: PV overwrites O anyway).
            // PV_(j-1) is complete: S_j's commit covers every MMA issued before it.
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll
                for (int d0 = 0; d0 < D; d0 += 32) {
                    float t[32];
                    tc_ld32(t_o + d0, t);
                    tc_wait_ld();
#pragma unroll
                    for (int u = 0; u < 32; ++u) t[u] *= alpha;
                    tc_st32(t_o + d0, t);
                }
            }
            {
                float a0, a1, a2, a3;
                unpack2(sum2[0], a0, a1);
                unpack2(sum2[1], a2, a3);
                l_run += (a0 + a1) + (a2 + a3);
            }
            tc_wait_st();
            tc_fence_before();        // the tensor-memory loads and stores above are ordered before the arrival
            __syncwarp();
            if (lane == 0) mbar_arrive(pfull);
        }
        if (alive) alive = warp_wait(pvdone, (uint32_t)((n_tiles - 1) & 1), &abort_flag, p.status);
        tc_fence_after();
        if (alive) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.o) + ((int64_t)(q0 + tid) * p.Hq + h) * D);
#pragma unroll
            for (int d0 = 0; d0 < D; d0 += 32) {
                float t[32];
                __syncwarp();
                tc_ld32(t_o + d0, t);
                tc_wait_ld();
                if (tid < rows_here) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float e[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) e[u] = t[c * 8 + u] * inv;
                        dst[d0 / 8 + c] = Vec16<T>::from_float(e);
                    }
                }
            }
        }
    } else if (tid < kSoftmaxThreads + kProducerThreads) {
        // ================================================================== producers
        // kChunks consecutive threads share a row.  Step i fetches tile i of the sequence K_0 V_0 K_1 V_1 ...
        // as one cp.async group and announces the group of the step before.  The page ids of a tile's rows come
        // from the table the lookup warp fills two tiles ahead, so no copy waits for a lookup.
        reg_dec<PfRegs<SUB>::aux>();
        const int pt = tid - kSoftmaxThreads;
        constexpr int kRowStep = kProducerThreads / kChunks, kRowsPerThread = kPfTile / kRowStep;
        const T* q = reinterpret_cast<const T*>(p.q);
        const T* kv = reinterpret_cast<const T*>(p.kv);
        const int64_t row_elems = (int64_t)p.Hkv * D;
        const uint32_t ps = (uint32_t)p.page_size;
        const int my_c = pt % kChunks, my_r0 = pt / kChunks;
        const T* kv_head = kv + (int64_t)kvh * D + my_c * 8;
        auto stage_kv = [&](uint8_t* dst, uint32_t t0, int buf, int which) {
            const uint32_t base = smem_u32(dst);
            int32_t pg[kRowsPerThread];          // all ids first: a copy (an asm with a memory clobber) lets no later load pass it
#pragma unroll
            for (int i = 0; i < kRowsPerThread; ++i) pg[i] = pgtab[buf * kPfTile + my_r0 + i * kRowStep];
#pragma unroll
            for (int i = 0; i < kRowsPerThread; ++i) {
                const int r = my_r0 + i * kRowStep;
                const int64_t page = pg[i];
                const bool ok = page >= 0;
                const uint32_t slot = p.ps_shift >= 0 ? (t0 + r) & (ps - 1u) : (t0 + r) % ps;
                const T* src = ok ? kv_head + ((page * 2 + which) * ps + slot) * row_elems : kv;
                cp_async16(base + sw128_offset(kPfTile, r, my_c), src, ok ? 16u : 0u);
            }
        };
        auto announce = [&](int slot) {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar[kFull + slot]);
        };
        {
            const uint32_t base = smem_u32(sQ);
#pragma unroll 4
            for (int r = my_r0; r < kRows; r += kRowStep) {
                const bool ok = r < rows_here;
                const T* src = ok ? q + ((int64_t)(q0 + r) * p.Hq + h) * D + my_c * 8 : q;
                cp_async16(base + (r >> 7) * kQBytes + sw128_offset(kPfRows, r & 127, my_c), src, ok ? 16u : 0u);
            }
        }
        bool alive = true;
        // A tile is announced kLag steps after its copies were issued.  Measured: one step is best with a ring of
        // five (two or three leave the MMA warp waiting for tiles: 8.4 -> 9.7 -> 12 ms on a 32 K prompt); what bounds
        // a step is the rate at which the load/store unit accepts a warp's copies, not the wait for the group.
        constexpr int kLag = TIDAL_PF_LAG;
        static_assert(kLag >= 1 && kLag <= 3 && kLag + 2 <= kPfRing, "the ring holds the tiles in flight and the two being read");
        int slot = 0;
        uint32_t wrap = 0;             // (i / ring) & 1
        for (int i = 0; i < 2 * n_tiles; ++i) {
            const int j = i >> 1;
            if (i >= kPfRing && !warp_wait(&bar[kEmpty + slot], wrap ^ 1u, &abort_flag, p.status)) { alive = false; break; }
            if (!(i & 1) && !warp_wait(&bar[kIdsFull + (j & 1)], (uint32_t)((j >> 1) & 1), &abort_flag, p.status)) { alive = false; break; }
            stage_kv(sRing + (uint32_t)slot * kTileBytes, (uint32_t)j * kPfTile, j & 1, i & 1);
            cp_async_commit();
            if (i >= kLag) {
                cp_async_wait<kLag>();
                announce(slot >= kLag ? slot - kLag : slot - kLag + kPfRing);
            }
            if (i & 1) {                   // V_j issued: this warp has read table j & 1 for the last time
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar[kIdsEmpty + (j & 1)]);
            }
            if (++slot == kPfRing) {
                slot = 0;
                wrap ^= 1u;
            }
        }
        // the last kLag tiles, oldest first (slot = that of tile 2 n_tiles)
        if (kLag >= 3) {
            cp_async_wait<2>();
            if (alive && 2 * n_tiles >= 3) announce((slot + 2 * kPfRing - 3) % kPfRing);
        }
        if (kLag >= 2) {
            cp_async_wait<1>();
            if (alive && 2 * n_tiles >= 2) announce((slot + 2 * kPfRing - 2) % kPfRing);
        }
        cp_async_wait<0>();
        if (alive) announce((slot + 2 * kPfRing - 1) % kPfRing);
    } else if (warp == (kSoftmaxThreads + kProducerThreads) / 32) {
        // ================================================================== MMA issue (one lane of this warp)
        reg_dec<PfRegs<SUB>::aux>();
        constexpr uint32_t idesc_qk = instr_desc(sizeof(T) == 2 && !std::is_same<T, __half>::value, 0, kPfRows, kPfTile);
        constexpr uint32_t idesc_pv = instr_desc(sizeof(T) == 2 && !std::is_same<T, __half>::value, 1, kPfRows, D);
        constexpr uint32_t v_lbo = kPfTile * 128, v_sbo = 1024;   // next 64 elements of D; next 8 tokens
        // operand descriptors of the tile origins; a step along K adds a constant to the address field
        const uint64_t dq = smem_desc_sw128(smem_u32(sQ), 16, 1024), dk = smem_desc_sw128(smem_u32(sRing), 16, 1024);
        const uint64_t dv = smem_desc_sw128(smem_u32(sRing), v_lbo, v_sbo);
        auto issue_qk = [&](int sb, int slot) {     // S = Q K^T of row block sb, K in ring slot `slot`
            const uint64_t dkj = dk + (uint64_t)(((uint32_t)slot * kTileBytes) >> 4);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                const uint32_t a = sb * kQBytes + (k >> 2) * (kPfRows * 128) + (k & 3) * 32;
                const uint32_t b = (k >> 2) * (kPfTile * 128) + (k & 3) * 32;
                tc_mma_f16(tmem + sb * kSubCols, dq + (a >> 4), dkj + (b >> 4), idesc_qk, k > 0);
            }
        };
        auto issue_pv = [&](int sb, int slot, uint32_t accumulate) {   // O (+)= P V of row block sb, V in ring slot `slot`
            const uint64_t dvj = dv + (uint64_t)(((uint32_t)slot * kTileBytes) >> 4);
#pragma unroll
            for (int k = 0; k < kPfTile / 16; ++k)
                tc_mma_f16_ts(tmem + sb * kSubCols + kPfTile, tmem + sb * kSubCols + k * 8, dvj + (uint64_t)((k * 16 * 128) >> 4), idesc_pv,
                              (accumulate || k > 0) ? 1u : 0u);
        };
        int slot = 0;                 // the consumer walks the ring in sequence order
        uint32_t wrap = 0;
        auto advance = [&]() {
            if (++slot == kPfRing) {
                slot = 0;
                wrap ^= 1u;
            }
        };
        bool alive = warp_wait(&bar[kFull + 0], 0u, &abort_flag, p.status);      // Q and K_0
        if (alive && lane == 0) {
            tc_fence_after();
#pragma unroll
            for (int sb = 0; sb < SUB; ++sb) {
                issue_qk(sb, 0);
                tc_commit(&bar[kSFull + sb]);
            }
            tc_commit(&bar[kEmpty + 0]);
        }
        __syncwarp();
        advance();
        for (int j = 0; j < n_tiles && alive; ++j) {
            const int v_slot = slot;
            alive = warp_wait(&bar[kFull + v_slot], wrap, &abort_flag, p.status);       // V_j
            advance();
            const int k_slot = slot;
            const bool more = j + 1 < n_tiles;
            if (alive && more) alive = warp_wait(&bar[kFull + k_slot], wrap, &abort_flag, p.status);   // K_(j+1)
            if (more) advance();
#pragma unroll
            for (int sb = 0; sb < SUB; ++sb) {
                if (alive) alive = warp_wait(&bar[kPFull + sb], (uint32_t)(j & 1), &abort_flag, p.status);
                if (alive && lane == 0) {
                    tc_fence_after();
                    issue_pv(sb, v_slot, j > 0 ? 1u : 0u);
                    tc_commit(&bar[kPvDone + sb]);
                    if (more) {
                        issue_qk(sb, k_slot);
                        tc_commit(&bar[kSFull + sb]);
                    }
                }
                __syncwarp();
            }
            if (alive && lane == 0) {
                tc_commit(&bar[kEmpty + v_slot]);
                if (more) tc_commit(&bar[kEmpty + k_slot]);
            }
            __syncwarp();
        }
        // nothing of this CTA may still be running on the tensor core when its tensor memory is given back
        if (lane == 0) tc_commit(&bar[kAllDone]);
        __syncwarp();
        warp_wait(&bar[kAllDone], 0u, &abort_flag, p.status);
    } else if (warp == (kSoftmaxThreads + kProducerThreads) / 32 + 1) {
        // ================================================================== page lookups
        // Table t & 1 takes, for each of the 128 rows of tile t, the page that holds the token, or -1 for a row that
        // reads as zeros (past the sequence, or a page id outside the pool: reported, not followed).
        reg_dec<PfRegs<SUB>::aux>();
        const uint32_t kv_len32 = (uint32_t)p.kv_len, ps = (uint32_t)p.page_size;
        for (int t = 0; t < n_tiles; ++t) {
            if (t >= 2 && !warp_wait(&bar[kIdsEmpty + (t & 1)], (uint32_t)(((t >> 1) - 1) & 1), &abort_flag, p.status)) break;
            int32_t v[kPfTile / 32];
#pragma unroll
            for (int i = 0; i < kPfTile / 32; ++i) {
                const uint32_t tok = (uint32_t)t * kPfTile + lane + 32 * i;
                v[i] = -1;
                if (tok < kv_len32) {
                    v[i] = p.pages[p.ps_shift >= 0 ? tok >> p.ps_shift : tok / ps];
                    if (!(v[i] >= 0 && (int64_t)v[i] < p.num_pages)) {
                        bad_page = true;                         // reported once at the exit
                        v[i] = -1;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kPfTile / 32; ++i) pgtab[(t & 1) * kPfTile + lane + 32 * i] = v[i];
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar[kIdsFull + (t & 1)]);
        }
    } else {
        reg_dec<PfRegs<SUB>::aux>();      // the spare warps of the second auxiliary group
    }
    if (bad_page && p.status) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tc_dealloc(tmem, kTmemCols);
}

template <typename T, int D, int SUB>
static int launch_prefill_sub(const PrefillParams& p, cudaStream_t st) {
    // Q, the K/V ring, barriers, page-id table
    const size_t smem = (size_t)SUB * kPfRows * D * 2 + (size_t)kPfRing * kPfTile * D * 2 + 256 + 2 * kPfTile * sizeof(int32_t);
    TIDAL_CUDA_OK(cudaFuncSetAttribute(prefill_attn_kernel<T, D, SUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int n_qt = (p.n_q + kPfRows * SUB - 1) / (kPfRows * SUB);
    TIDAL_CUDA_OK(launch_pdl(prefill_attn_kernel<T, D, SUB>, dim3((unsigned)n_qt, (unsigned)p.Hq), dim3(128 * SUB + kPfExtraThreads), smem, st, 1, p));
    count_launch();
    return TIDAL_OK;
}
template <typename T, int D>
static int launch_prefill(const PrefillParams& p, cudaStream_t st) {
    // one row block per CTA when there are no more rows than that (a late chunk of a prompt, a short prompt)
    return p.n_q > kPfRows ? launch_prefill_sub<T, D, 2>(p, st) : launch_prefill_sub<T, D, 1>(p, st);
}


// ------------------------------------------------------------------ fp32 caches: CUDA cores
// kind::f16 has no fp32 operand mode and kind::tf32 would not meet a 1e-4 tolerance, so fp32 storage (the
// tiny reference-parity configuration) gets a plain tiled kernel: 64 query rows of one head per CTA, K/V tiles
// of 64 tokens in shared memory (K transposed, so that a thread's four score columns are one 16-byte read),
// 16 x 16 threads each owning a 4 x 4 block of the score tile and 4 rows x D/16 columns of the output,
// online softmax with exact exp2f.  Same page lookup and bounds rule as the tensor-core kernel.
constexpr int kPf32Rows = 64, kPf32Tile = 64;
template <int D>
__global__ void __launch_bounds__(256) prefill_f32_kernel(const __grid_constant__ PrefillParams p) {
    extern __shared__ __align__(16) float fsm[];
    float* Qs = fsm;                               // [64][D]
    float* Kt = Qs + kPf32Rows * D;                // [D][64]
    float* Vs = Kt + D * kPf32Tile;                // [64][D]
    float* Ps = Vs + kPf32Tile * D;                // [64][64]
    constexpr int DC = D / 16;                     // output columns per thread
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int n_qt = (p.n_q + kPf32Rows - 1) / kPf32Rows;
    const int qt = n_qt - 1 - (int)blockIdx.x;     // longest rows first
    const int h = blockIdx.y, kvh = h / (p.Hq / p.Hkv);
    const int q0 = qt * kPf32Rows;
    const int rows_here = min(kPf32Rows, p.n_q - q0);
    const int64_t pos0 = p.kv_len - p.n_q + q0;
    const int64_t kv_end = p.causal ? min(p.kv_len, pos0 + rows_here) : p.kv_len;
    const int n_tiles = (int)((kv_end + kPf32Tile - 1) / kPf32Tile);
    const float* q = reinterpret_cast<const float*>(p.q);
    const float* kv = reinterpret_cast<const float*>(p.kv);
    const int64_t row_elems = (int64_t)p.Hkv * D;
    bool bad_page = false;

    for (int i = tid; i < kPf32Rows * (D / 4); i += 256) {
        const int r = i / (D / 4), c4 = i - r * (D / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows_here) v = *reinterpret_cast<const float4*>(q + ((int64_t)(q0 + r) * p.Hq + h) * D + c4 * 4);
        *reinterpret_cast<float4*>(Qs + r * D + c4 * 4) = v;
    }
    float o[4][DC], m_run[4], l_run[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < DC; ++j) o[i][j] = 0.f;
    }
    for (int j = 0; j < n_tiles; ++j) {
        const int64_t t0 = (int64_t)j * kPf32Tile;
        __syncthreads();                           // the previous tile's K, V and P are no longer read
        for (int i = tid; i < kPf32Tile * (D / 4); i += 256) {
            const int c = i % kPf32Tile, d4 = i / kPf32Tile;      // consecutive threads: consecutive tokens
            const int64_t t = t0 + c;
            float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), vx = kx;
            if (t < p.kv_len) {
                const int64_t pi = t / p.page_size, slot = t - pi * p.page_size;
                const int64_t page = p.pages[pi];
                if (page >= 0 && page < p.num_pages) {
                    const float* src = kv + ((page * 2) * p.page_size + slot) * row_elems + (int64_t)kvh * D + d4 * 4;
                    kx = *reinterpret_cast<const float4*>(src);
                    vx = *reinterpret_cast<const float4*>(src + (int64_t)p.page_size * row_elems);
                } else {
                    bad_page = true;
                }
            }
            Kt[(d4 * 4 + 0) * kPf32Tile + c] = kx.x;
            Kt[(d4 * 4 + 1) * kPf32Tile + c] = kx.y;
            Kt[(d4 * 4 + 2) * kPf32Tile + c] = kx.z;
            Kt[(d4 * 4 + 3) * kPf32Tile + c] = kx.w;
            *reinterpret_cast<float4*>(Vs + c * D + d4 * 4) = vx;
        }
        __syncthreads();
        // S block: rows ty*4.., columns tx*4..
        float s[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
#pragma unroll 8
        for (int d = 0; d < D; ++d) {
            const float4 kc = *reinterpret_cast<const float4*>(Kt + d * kPf32Tile + tx * 4);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float qa = Qs[(ty * 4 + a) * D + d];
                s[a][0] = fmaf(qa, kc.x, s[a][0]);
                s[a][1] = fmaf(qa, kc.y, s[a][1]);
                s[a][2] = fmaf(qa, kc.z, s[a][2]);
                s[a][3] = fmaf(qa, kc.w, s[a][3]);
            }
        }
        // online softmax per row (the 16 threads of a row are the 16 lanes of a half warp)
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int64_t my_pos = pos0 + ty * 4 + a;
            const int64_t lim = p.causal ? min(p.kv_len - 1, my_pos) : p.kv_len - 1;
            float mx = m_run[a];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                s[a][b] = (t0 + tx * 4 + b <= lim) ? s[a][b] * p.scale_log2 : -INFINITY;
                mx = fmaxf(mx, s[a][b]);
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float msafe = mx == -INFINITY ? 0.f : mx;
            const float alpha = exp2f(m_run[a] - msafe);          // 0 while nothing has been seen
            float sum = 0.f;
            float4 pr;
            pr.x = exp2f(s[a][0] - msafe);
            pr.y = exp2f(s[a][1] - msafe);
            pr.z = exp2f(s[a][2] - msafe);
            pr.w = exp2f(s[a][3] - msafe);
            sum = (pr.x + pr.y) + (pr.z + pr.w);
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            m_run[a] = mx;
            l_run[a] = fmaf(l_run[a], alpha, sum);
#pragma unroll
            for (int c = 0; c < DC; ++c) o[a][c] *= alpha;
            *reinterpret_cast<float4*>(Ps + (ty * 4 + a) * kPf32Tile + tx * 4) = pr;
        }
        __syncthreads();
        // O block: rows ty*4.., columns tx*DC..
#pragma unroll 4
        for (int c = 0; c < kPf32Tile; ++c) {
            float vv[DC];
#pragma unroll
            for (int u = 0; u < DC; u += 4) {
                const float4 v4 = *reinterpret_cast<const float4*>(Vs + c * D + tx * DC + u);
                vv[u] = v4.x; vv[u + 1] = v4.y; vv[u + 2] = v4.z; vv[u + 3] = v4.w;
            }
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float pa = Ps[(ty * 4 + a) * kPf32Tile + c];
#pragma unroll
                for (int u = 0; u < DC; ++u) o[a][u] = fmaf(pa, vv[u], o[a][u]);
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int r = ty * 4 + a;
        if (r >= rows_here) continue;
        const float inv = l_run[a] > 0.f ? 1.f / l_run[a] : 0.f;
        float* dst = reinterpret_cast<float*>(p.o) + ((int64_t)(q0 + r) * p.Hq + h) * D + tx * DC;
#pragma unroll
        for (int u = 0; u < DC; u += 4)
            *reinterpret_cast<float4*>(dst + u) = make_float4(o[a][u] * inv, o[a][u + 1] * inv, o[a][u + 2] * inv, o[a][u + 3] * inv);
    }
    if (bad_page && p.status) atomicOr(p.status, TIDAL_DEV_BAD_INDEX);
}

template <int D>
static int launch_prefill_f32(const PrefillParams& p, cudaStream_t st) {
    const size_t smem = sizeof(float) * ((size_t)kPf32Rows * D + 2 * (size_t)kPf32Tile * D + (size_t)kPf32Rows * kPf32Tile);
    TIDAL_CUDA_OK(cudaFuncSetAttribute(prefill_f32_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int n_qt = (p.n_q + kPf32Rows - 1) / kPf32Rows;
    TIDAL_CUDA_OK(launch_pdl(prefill_f32_kernel<D>, dim3((unsigned)n_qt, (unsigned)p.Hq), dim3(256), smem, st, 1, p));
    count_launch();
    return TIDAL_OK;
}

}  // namespace tidal

using namespace tidal;

extern "C" int tidal_prefill(const tidal_prefill_args* a, void* stream) {
    TIDAL_REQUIRE(a != nullptr, TIDAL_ERR_ARG, "args is NULL");
    TIDAL_REQUIRE(a->d_q && a->d_o && a->d_kv && a->d_page_table, TIDAL_ERR_ARG, "null pointer");
    TIDAL_REQUIRE(a->dtype >= 0 && a->dtype <= 2, TIDAL_ERR_ARG, "unknown dtype %d", a->dtype);
    TIDAL_REQUIRE(a->head_dim == 64 || a->head_dim == 128, TIDAL_ERR_ARG, "head_dim %d not supported (64, 128)", a->head_dim);
    TIDAL_REQUIRE(a->num_qo_heads >= 1 && a->num_kv_heads >= 1 && a->num_qo_heads % a->num_kv_heads == 0, TIDAL_ERR_ARG,
                  "num_qo_heads (%d) must be a multiple of num_kv_heads (%d)", a->num_qo_heads, a->num_kv_heads);
    TIDAL_REQUIRE(a->num_qo_heads <= 65535, TIDAL_ERR_ARG, "too many heads");
    TIDAL_REQUIRE(a->kv_len < ((int64_t)1 << 31) - kPfTile, TIDAL_ERR_ARG, "kv_len too large");
    TIDAL_REQUIRE(a->page_size >= 1 && a->n_q >= 1 && a->kv_len >= a->n_q, TIDAL_ERR_ARG,
                  "need page_size >= 1, n_q >= 1 and kv_len (%lld) >= n_q (%d): the cache already holds the new rows",
                  (long long)a->kv_len, a->n_q);
    TIDAL_REQUIRE((((uintptr_t)a->d_q | (uintptr_t)a->d_o | (uintptr_t)a->d_kv) & 15) == 0, TIDAL_ERR_ARG,
                  "q, o and the pool must be 16-byte aligned");
    TIDAL_REQUIRE(a->num_pages >= 1, TIDAL_ERR_ARG, "num_pages (pages in the pool) must be given");
    PrefillParams p;
    p.q = a->d_q;
    p.o = a->d_o;
    p.kv = a->d_kv;
    p.pages = a->d_page_table;
    p.status = a->d_status;
    p.kv_len = a->kv_len;
    p.num_pages = a->num_pages;
    p.n_q = a->n_q;
    p.Hq = a->num_qo_heads;
    p.Hkv = a->num_kv_heads;
    p.page_size = a->page_size;
    p.ps_shift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == a->page_size) p.ps_shift = sh;
    p.causal = a->causal ? 1 : 0;
    const float sc = a->sm_scale > 0.f ? a->sm_scale : 1.f / sqrtf((float)a->head_dim);
    p.scale_log2 = sc * kLog2e;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == TIDAL_DTYPE_F32) return a->head_dim == 128 ? launch_prefill_f32<128>(p, st) : launch_prefill_f32<64>(p, st);
    if (a->dtype == TIDAL_DTYPE_F16)
        return a->head_dim == 128 ? launch_prefill<__half, 128>(p, st) : launch_prefill<__half, 64>(p, st);
    return a->head_dim == 128 ? launch_prefill<__nv_bfloat16, 128>(p, st) : launch_prefill<__nv_bfloat16, 64>(p, st);
}
