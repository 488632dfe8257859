// Parameters shared by the two decode-attention kernels (CUDA-core and tensor-core).
#pragma once

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

// Tensor-core kernel (decode_attn_mma.cu): 16-bit storage, up to 16 query heads per
// KV head, HC in {1,2,4,8} KV heads per CTA, 8 consumer warps.
constexpr int kMmaWarps = 8;
constexpr int kMmaTile = 16;            // tokens one warp takes from a stage
size_t attn_mma_smem_bytes(int S, int HC, int D, bool sum_heads);
int launch_attn_mma(const AttnParams& p, int D, int dtype, dim3 grid, size_t smem, cudaStream_t st);

}  // namespace tidal
