// Parameters shared by the two decode-attention kernels (CUDA-core and tensor-core).
#pragma once

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
    int32_t cluster;  // > 1: that many CTAs along the chunk dimension form a cluster that covers the whole
                      // token list and merges through distributed shared memory (then nchunks == cluster)
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


// Bytes of the per-CTA result block [HC*G][D] + [HC*G][2] that store_attention_result reads.
__host__ __device__ inline size_t cta_result_bytes(int HC, int G, int D) { return (size_t)HC * G * (D + 2) * sizeof(float); }

// Final step of both attention kernels.  cta_o[(hg)*D + d] and cta_ml[hg*2 + {0,1}] hold this CTA's
// un-normalised output, running maximum (log2 domain) and denominator for its HC*G query heads.
// One CTA per token list chunk: written out as a split-KV partial (or as the result when there is a
// single chunk).  A cluster: its CTAs cover the whole list; each merges a share of the outputs from
// all CTAs' blocks through distributed shared memory and writes final values, so no partials and no
// merge kernel are needed.  Every thread of the CTA must call this.
template <typename T>
__device__ __forceinline__ void store_attention_result(const AttnParams& p, const float* cta_o, const float* cta_ml, int HC,
                                                       int G, int D, int qh0, int b, int chunk) {
    namespace cg = cooperative_groups;
    const int nout = HC * G * D;
    auto put_final = [&](int idx, float acc, float M, float L) {
        const int d = idx % D, hg = idx / D;
        const size_t ph = (size_t)b * p.Hq + qh0 + hg;
        if (p.o) reinterpret_cast<T*>(p.o)[ph * D + d] = from_f32<T>(L > 0.f ? acc / L : 0.f);
        if (p.shard_o) {
            p.shard_o[ph * D + d] = acc;
            if (d == 0) {
                p.shard_m[ph] = M;
                p.shard_l[ph] = L;
            }
        }
    };
    if (p.cluster <= 1) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < nout; idx += blockDim.x) {
            const int d = idx % D, hg = idx / D;
            const float acc = cta_o[idx], M = cta_ml[2 * hg], L = cta_ml[2 * hg + 1];
            if (p.nchunks == 1) {
                put_final(idx, acc, M, L);
            } else {
                const size_t ph = (size_t)b * p.Hq + qh0 + hg;
                p.part_o[(ph * p.nchunks + chunk) * D + d] = acc;
                if (d == 0) {
                    p.part_ml[(ph * p.nchunks + chunk) * 2] = M;
                    p.part_ml[(ph * p.nchunks + chunk) * 2 + 1] = L;
                }
            }
        }
        return;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                   // every CTA's block is complete and visible
    const int CS = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int per = (nout + CS - 1) / CS;
    const int hi = min(nout, (rank + 1) * per);
    for (int idx = rank * per + threadIdx.x; idx < hi; idx += blockDim.x) {
        const int hg = idx / D;
        float M = -INFINITY;
        for (int r = 0; r < CS; ++r) M = fmaxf(M, cluster.map_shared_rank(cta_ml, r)[2 * hg]);
        float acc = 0.f, L = 0.f;
        for (int r = 0; r < CS; ++r) {
            const float* ml = cluster.map_shared_rank(cta_ml, r);
            const float m = ml[2 * hg];
            const float w = (m == -INFINITY) ? 0.f : fast_exp2(m - M);
            acc = fmaf(w, cluster.map_shared_rank(cta_o, r)[idx], acc);
            L = fmaf(w, ml[2 * hg + 1], L);
        }
        put_final(idx, acc, M, L);
    }
    cluster.sync();                                   // nobody leaves while its block may still be read
}

// Tensor-core kernel (decode_attn_mma.cu): 16-bit storage, up to 16 query heads per
// KV head, HC in {1,2,4,8} KV heads per CTA, 8 consumer warps.
constexpr int kMmaWarps = 8;
constexpr int kMmaTile = 16;            // tokens one warp takes from a stage
size_t attn_mma_smem_bytes(int S, int HC, int G, int D, bool sum_heads);
int launch_attn_mma(const AttnParams& p, int D, int dtype, dim3 grid, size_t smem, cudaStream_t st);

}  // namespace tidal
