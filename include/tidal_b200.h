/*
 * tidal_b200 — C ABI of the B200 (sm_100a) decode-attention path of TidalDecode.
 *
 * Conventions
 *   - every pointer named d_* or documented "device" is a CUDA device pointer on
 *     the current device; `stream` is a cudaStream_t passed as void*;
 *   - no entry point allocates, frees or synchronises, except tidal_ws_init
 *     (one memset on the stream) and tidal_ws_status (one blocking 4-byte read);
 *   - return value: 0 = launched; negative = argument rejected on the host
 *     (message via tidal_last_error()); device-side faults (a bounded wait that
 *     ran out, an out-of-range index that was skipped) are recorded in the
 *     workspace and read back with tidal_ws_status();
 *   - KV pool layout ("NHD", one pool per layer) is the reference's
 *     [pages][2][page_size][Hkv][D] with K at plane 0 and V at plane 1
 *     (kernels/include/decode/decode_page.cuh:191-200,223-234;
 *     tidal/utils/kv_cache.py:21-25).
 *
 * Each entry point names the reference interface it stands in for
 * (paths relative to the TidalDecode repository).
 */
#ifndef TIDAL_B200_H_
#define TIDAL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TIDAL_DTYPE_F16 0
#define TIDAL_DTYPE_BF16 1
#define TIDAL_DTYPE_F32 2

#define TIDAL_OK 0
#define TIDAL_ERR_ARG (-1)      /* bad shape / null pointer / unsupported combination */
#define TIDAL_ERR_WORKSPACE (-2) /* workspace too small or misaligned */
#define TIDAL_ERR_CUDA (-3)      /* a CUDA runtime call failed (launch error) */

/* device-side status bits, tidal_ws_status() */
#define TIDAL_DEV_WAIT_TIMEOUT 1u /* an mbarrier wait hit its iteration limit */
#define TIDAL_DEV_BAD_INDEX 2u    /* a token/page index was out of range and skipped */
#define TIDAL_DEV_TOPK_OVERFLOW 4u /* internal top-k buffer overflow (result invalid) */

/* Library version (major*10000 + minor*100 + patch). */
int tidal_version(void);

/* Message of the last negative return on this host thread. */
const char* tidal_last_error(void);

/* Kernels this library has launched since it was loaded (all threads). */
uint64_t tidal_launch_count(void);

/* ---------------------------------------------------------------- workspace
 * Stands in for BatchDecodeHandler::BeginForward's per-call cudaMallocAsync of
 * the split-KV scratch (kernels/include/decode/decode_handler.cuh:73-136) and
 * for the top-k `buf` (tidal/utils/controller.py:164-168): the caller allocates
 * one buffer once, sized by tidal_ws_bytes, and passes it to every call.
 *   max_rows   = rows the top-k may see at once (B for head-summed scores,
 *                B*Hq for per-head scores);
 *   max_n      = longest score row;
 * The buffer must be 256-byte aligned.  tidal_ws_init (same geometry as given to
 * tidal_ws_bytes) must run once, and again after any non-zero tidal_ws_status,
 * before the first use: it records the geometry on the host under the buffer's
 * address and zeroes the counters, which kernels leave zero at rest.
 * Calls that share one workspace must not overlap on the GPU. */
size_t tidal_ws_bytes(int max_batch, int num_qo_heads, int head_dim, int max_rows, int64_t max_n);
int tidal_ws_init(void* d_ws, size_t ws_bytes, int max_batch, int num_qo_heads, int head_dim, int max_rows,
                  int64_t max_n, void* stream);
/* Forget a workspace (host bookkeeping only; the memory stays the caller's). */
int tidal_ws_release(void* d_ws);
/* Blocking: returns the OR of TIDAL_DEV_* bits seen since the last init (>= 0),
 * or a negative TIDAL_ERR_*. */
int tidal_ws_status(void* d_ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------------- decode attention
 * One decode step of attention for `batch` sequences, one new query each.
 * Stands in for BatchDecodeWithPagedKVCachePyTorchWrapper::Forward
 * (tidal/ops/csrc/approx_attn.cu:68-151 → BatchDecodeWithPagedKVCacheKernel,
 * kernels/include/decode/decode_attn.cuh:446-658, plus VariableLengthMergeStates
 * :1012-1020), for all three layer kinds:
 *   full layer       sel_idx = NULL, scores_out = NULL
 *   selection layer  sel_idx = NULL, scores_out != NULL  (attends to ALL tokens and
 *                    writes the pre-softmax logits q·k/sqrt(D) in fp32 —
 *                    src/tidal_build/modify_llama.py:105-120)
 *   sparse layer     sel_idx != NULL (attends only to the listed tokens — :121-133)
 */
typedef struct tidal_attn_args {
    /* tensors */
    const void* d_q;            /* [batch][Hq][D], dtype */
    void* d_o;                  /* [batch][Hq][D], dtype; may be NULL if d_part_* given */
    const void* d_kv;           /* pool of this layer */
    const int32_t* d_page_table;/* [batch][page_table_stride] page ids; NULL: page j of
                                   sequence b is page b*page_table_stride + j */
    int64_t page_table_stride;
    const int32_t* d_seq_lens;  /* [batch] tokens per sequence, or NULL → all = seq_len */
    int32_t seq_len;            /* host-side upper bound of (and default for) the lengths */
    /* selection list (sparse layer) */
    const int32_t* d_sel_idx;   /* [batch][sel_rows][sel_stride] token positions, or NULL */
    int32_t sel_rows;           /* 1 = one shared list per sequence, Hq = one per q head */
    int32_t sel_count;          /* entries per list */
    int64_t sel_stride;         /* elements between lists */
    int32_t sel_physical;       /* 1: entries are pool page ids, page_size must be 1
                                   (tidal/utils/controller.py:20,122-137) */
    const int32_t* d_sel_counts;/* NULL, or [batch][sel_rows] valid entries per list (<= sel_count):
                                   lists that tidal_topk filtered to one shard's positions */
    int32_t extra_page;         /* >= 0: also attend this pool page — the newest token, as
                                   the reference appends it (decode_attn.cuh:726-730); -1 none */
    /* logits out (selection layer) */
    float* d_scores;            /* NULL, or [batch][score_rows][score_stride] fp32; column = token position,
                                   or, with a selection list, the entry's place in the list (newest token last) */
    int32_t score_rows;         /* 1 = summed over all Hq heads, Hq = per q head */
    int64_t score_stride;
    uint32_t* d_hist;           /* NULL, or [batch*score_rows][TIDAL_TOPK_BINS] zeroed counters
                                   that receive the first radix digit of every logit, so that
                                   tidal_topk can skip its own histogram pass (see there) */
    int32_t force_last;         /* histogram counts the newest token as +inf (kernel-path rule) */
    /* un-normalised partials out (sequence-sharded KV); all three or none */
    float* d_part_m;            /* [batch][Hq]   running max, log2 domain */
    float* d_part_l;            /* [batch][Hq]   sum of exp2(s - m) */
    float* d_part_o;            /* [batch][Hq][D] sum of exp2(s - m) * v */
    /* geometry */
    int32_t batch, num_qo_heads, num_kv_heads, head_dim, page_size, dtype;
    int64_t num_pages;          /* pages in the pool, for the bounds check */
    float sm_scale;             /* <= 0 → 1/sqrt(D) */
    int32_t num_chunks;         /* 0 = planner's choice; else force the KV split */
    int32_t heads_per_cta;      /* 0 = planner's choice; else KV heads one CTA covers */
    int32_t use_tensor_cores;   /* 0 = when 2..16 query heads share a KV head (f16/bf16); 1 = whenever
                                   possible; -1 = never (CUDA-core kernel) */
} tidal_attn_args;

int tidal_decode_attention(const tidal_attn_args* args, void* d_ws, size_t ws_bytes, void* stream);

/* The planner's choice of CTAs along the KV split for `tokens` tokens per list and
 * batch*head_slices lists; what PartitionPagedKVCacheBinarySearchMinNumPagePerBatch
 * computes in the reference (decode_attn.cuh:763-791). Pure host arithmetic. */
int tidal_plan_chunks(int batch, int head_slices, int tokens, int min_tokens_per_chunk, int sm_count);

/* ------------------------------------------------------------------ top-k
 * Row-wise top-k of fp32 scores → unsorted-set semantics, emitted in ascending
 * index order when k <= 4096.  Stands in for topk_filtering
 * (tidal/ops/csrc/topk.cu:7-44 → decode_select_k, RAFT radix select) and for
 * torch.topk at src/tidal_build/modify_llama.py:118.  k >= n selects everything
 * (:112-113).  Exact ties are broken towards the lower index, so equal inputs
 * give equal sets on every rank.
 *   d_scores  [rows][row_stride] fp32
 *   d_in_idx  NULL, or [rows][row_stride] int32: emit d_in_idx[j] instead of j
 *             (the reference's `estimated_indices`, topk.cu:9)
 *   d_out_idx [rows][out_stride] int32, first min(k,n) entries written
 *   d_out_val NULL or [rows][out_stride] fp32, scores of the emitted entries
 *   d_hist    NULL, or the histogram tidal_decode_attention filled for exactly
 *             these rows (then pass the same force_last)
 *   idx_offset added to emitted positions (global position of a shard's first token)
 *   own_lo/own_hi  when own_hi > own_lo, only emitted values v with own_lo <= v < own_hi
 *             are written, as v - own_lo, and d_out_count[row] receives how many
 *             (the rank-local part of a global selection); otherwise d_out_count,
 *             if given, receives min(k, n)
 */
#define TIDAL_TOPK_BINS 4096
typedef struct tidal_topk_args {
    const float* d_scores;
    const int32_t* d_in_idx;
    int64_t in_idx_stride;      /* elements between rows of d_in_idx; 0 = one row shared by all */
    int32_t rows;
    int64_t n, row_stride;
    int32_t k;
    int32_t* d_out_idx;
    float* d_out_val;
    int64_t out_stride;
    int32_t idx_offset, force_last;
    int32_t own_lo, own_hi;
    int32_t* d_out_count;
    uint32_t* d_hist;
    int32_t seg_len;            /* 0, or: a row is made of segments of seg_len elements that lie seg_stride */
    int64_t seg_stride;         /*    elements apart (element j of row r is at (j/seg_len)*seg_stride +
                                      r*row_stride + j%seg_len); d_in_idx is addressed the same way.  This is how the
                                      per-rank candidate blocks of an all-gathered buffer are ranked in place.
                                      Needs k <= 2048 and n <= 2097152. */
    const int32_t* d_row_len;   /* NULL, or [rows] int32 on the device: the length of each row; n is then only their
                                   upper bound and force_last refers to the row's own last element.  For decode steps
                                   replayed as a CUDA graph, where lengths grow without the host's involvement.
                                   Same limits as seg_len. */
} tidal_topk_args;
int tidal_topk(const tidal_topk_args* args, void* d_ws, size_t ws_bytes, void* stream);

/* ------------------------------------------------ top-k without a workspace
 * Has no counterpart in the reference.  Same selection as tidal_topk, for callers
 * that are not in a position to hand over (or allocate) a workspace: a plugin that
 * was given only its input and output buffers by a host runtime which owns all device
 * memory, or a decode loop that runs under a "no allocator calls after warm-up" rule
 * because cudaMalloc/cudaFree may synchronise the device and stall every stream.
 * The scratch the kernel needs (the lists of certain and candidate keys and the fault
 * word) lives in a fixed ~2 MB array inside the library image instead; each GPU that
 * loads the library keeps that array until the process exits.
 *
 * Limits (anything beyond is refused with TIDAL_ERR_ARG and a message): at most 8 rows
 * per call, rows of at most 262144 scores, k at most 16384; d_hist and d_row_len must be
 * NULL and seg_len, seg_stride 0 (contiguous rows whose length is n).
 * The call itself allocates nothing and frees nothing.  Its first use on a device
 * looks up the array's device address (cudaGetSymbolAddress, with that device
 * current) and caches it, so make that first call outside any stream capture.
 * All calls on one device share the array, which still holds what the previous call
 * left there: nothing in it needs to start at zero except the fault word, which is
 * sticky by design; two calls whose kernels can overlap on the GPU (different streams,
 * no dependency) would overwrite each other's lists — order them.
 * d_status: NULL, or a device word of the caller's that receives TIDAL_DEV_* bits
 * instead of the internal fault word. */
int tidal_topk_static(const tidal_topk_args* args, uint32_t* d_status, void* stream);
/* Blocking: the TIDAL_DEV_* bits that calls with d_status == NULL have left in the internal fault
 * word of the current device since it was last cleared (>= 0), or a negative TIDAL_ERR_*; clear != 0
 * zeroes the word afterwards (on `stream`, ordered after the read).  Has no counterpart in the
 * reference either; allocates nothing. */
int tidal_topk_static_status(int clear, void* stream);

/* ------------------------------------------------------ RoPE + KV append
 * Rotates q (in place) and the new k, then writes k,v into their pool slots.
 * Stands in for apply_rope_in_place + append_kv_cache_decode / _prefill
 * (tidal/ops/csrc/page.cu:212-253, 6-99, 101-210 → QKApplyRotaryInPlaceKernel
 * decode_page.cuh:639-687, AppendPagedKVCache{Decode,Prefill}Kernel :393-557).
 * Token i (of n_tokens = batch*tokens_per_seq) belongs to sequence
 * b = i / tokens_per_seq at position pos0[b] + i % tokens_per_seq.
 *   d_q  [n_tokens][Hq][D] or NULL;  d_k, d_v [n_tokens][Hkv][D] (d_v NULL: no append)
 *   d_pos0     [batch] int32 device, or NULL → every sequence starts at `pos0`
 *   d_inv_freq [D/2] fp32 device or NULL → theta^(-2i/D) computed in the kernel
 *   rope_mode  0 none; 1 reference-model rounding (cos, sin and both products rounded
 *              to dtype: src/models/llama_tidaldecoding.py:200-220,255-279);
 *              2 fp32 rotation rounded once (decode_page.cuh:650-669)
 *   k is rotated in place as well when rotate_k_in_place != 0 (the reference op does).
 */
typedef struct tidal_rope_append_args {
    void* d_q;
    void* d_k;
    const void* d_v;
    void* d_kv;                  /* pool of this layer, or NULL: rotate only */
    const int32_t* d_page_table; /* as in tidal_attn_args */
    int64_t page_table_stride;
    const int32_t* d_pos0;
    int32_t pos0;
    const float* d_inv_freq;
    float rope_theta, rope_scale;
    int32_t rope_mode, rotate_k_in_place;
    int32_t batch, tokens_per_seq, num_qo_heads, num_kv_heads, head_dim, page_size, dtype;
    int64_t num_pages;
    uint32_t* d_status;          /* NULL or a device word that receives TIDAL_DEV_* bits */
    const void* d_q_src;         /* NULL, or [n_tokens][Hq][D]: the queries are read from here and their rotated
                                    rows written to d_q, so the source survives (a projection's output buffer that
                                    is reused, a benchmark's resident inputs) */
    int32_t kv_pos_base;         /* position that the first slot of each sequence in this pool holds (0 unless the pool
                                    is one rank's shard [lo, hi) of a sequence-sharded context: then lo); the token at
                                    position p is rotated by p and written to slot p - kv_pos_base */
} tidal_rope_append_args;

int tidal_rope_append(const tidal_rope_append_args* args, void* stream);

/* ------------------------------------------------- Quest page metadata (legacy)
 * The reference keeps, next to the KV pool, a second paged pool of the same layout with one ENTRY per
 * KV page: plane 0 holds the element-wise maximum, plane 1 the minimum of the page's keys; its append
 * kernels maintain it (kernels/include/decode/decode_page.cuh:393-444 for one new token, :466-557 for a
 * prompt) and estimate_attn_score reads it (tidal/ops/csrc/estimate.cu:6-84 -> MaxPossibleSampleWithPagedKVCache,
 * kernels/include/decode/decode_attn.cuh:141-172, 249-405).  TidalDecode's own layers use neither; they are
 * here for callers of the reference's full operator surface.
 *
 * tidal_update_page_meta recomputes the entries of the KV pages that hold positions [first_pos, seq_len)
 * of every sequence from the keys now in the pool (call it after the append: one token -> first_pos =
 * seq_len - 1).  Entry e of a sequence (= its e-th KV page) lives in metadata page
 * d_meta_table[b][e / meta_page_size] (NULL: page b * meta_table_stride + e / meta_page_size), slot
 * e % meta_page_size.  Recomputing from the pool instead of folding the new key into the stored bounds
 * gives the same values and needs no "first token of a page" initialisation. */
typedef struct {
    const void* d_kv;            /* [num_pages][2][page_size][Hkv][D] */
    void* d_meta;                /* [num_meta_pages][2][meta_page_size][Hkv][D] */
    const int32_t* d_page_table; /* as in tidal_attn_args */
    int64_t page_table_stride;
    const int32_t* d_meta_table;
    int64_t meta_table_stride;
    int32_t batch, num_kv_heads, head_dim, page_size, meta_page_size, dtype;
    int64_t num_pages, num_meta_pages;
    int32_t first_pos, seq_len;
    uint32_t* d_status;          /* NULL or a device word that receives TIDAL_DEV_* bits */
} tidal_page_meta_args;
int tidal_update_page_meta(const tidal_page_meta_args* args, void* stream);

/* out[b][h][e] = sum_d max(q[b][h][d] * max_e[d], q[b][h][d] * min_e[d]) for the first n_entries entries of
 * every sequence: an upper bound of q.k over the keys of KV page e (no 1/sqrt(D) scale, as in the
 * reference).  The reference leaves out the last entry — the page still being filled — by passing
 * n_entries = entries - 1 (estimate.cu:52-54).  Query head h reads KV head h / (Hq / Hkv). */
typedef struct {
    const void* d_q;             /* [batch][Hq][D] */
    const void* d_meta;
    const int32_t* d_meta_table;
    int64_t meta_table_stride;
    void* d_out;                 /* [batch][Hq][out_stride] of out_dtype */
    int64_t out_stride;
    int32_t batch, num_qo_heads, num_kv_heads, head_dim, meta_page_size, n_entries, dtype, out_dtype;
    int64_t num_meta_pages;
    uint32_t* d_status;
} tidal_estimate_args;
int tidal_estimate(const tidal_estimate_args* args, void* stream);

/* -------------------------------------------- cross-shard merge of partials
 * o[b][h][:] = sum_r 2^(m_r-M) o_r / sum_r 2^(m_r-M) l_r over `shards` sets of
 * partials laid out [shards][batch*Hq(*D)] — what every rank runs after the
 * all-gather when the KV cache is sharded by sequence.  Same arithmetic as the
 * reference's merge across KV chunks (decode_attn.cuh:213-232, state_t::merge). */
int tidal_merge_partials(const float* d_m, const float* d_l, const float* d_o, int shards, int batch,
                         int num_qo_heads, int head_dim, void* d_out, int dtype, void* stream);
/* Same, with the shards' blocks shard_stride elements apart in each of d_m, d_l, d_o (the
 * packed receive buffer of an all-gather is merged in place). */
int tidal_merge_partials_strided(const float* d_m, const float* d_l, const float* d_o, int64_t shard_stride, int shards,
                                 int batch, int num_qo_heads, int head_dim, void* d_out, int dtype, void* stream);

/* ------------------------------------------------------------------ RMSNorm
 * y[r][:] = x[r][:] * rsqrt(mean(x[r]^2) + eps) * weight, fp32 statistics.  Stands in for
 * rms_norm_forward (tidal/ops/csrc/rms_norm.cu:185-213); not part of the attention path, on the
 * reference's operator surface next to it.  hidden must be a multiple of 8 (4 for fp32).
 * round_before_weight = 1 rounds the normalised value to dtype before the weight, as the
 * reference's PyTorch model does (src/models/llama_tidaldecoding.py:122-127). */
int tidal_rms_norm(const void* d_x, const void* d_weight, void* d_y, int64_t rows, int hidden, float eps, int dtype,
                   int round_before_weight, void* stream);

/* ------------------------------------------------------- decode-step linear
 * y[M][N] = x[M][K] * W[N][K]^T for M <= 8 rows of activations (one token per sequence), W in the
 * layout of torch.nn.Linear.weight, fp32 accumulation.  Replaces, in one launch, what the
 * reference's decoder layer issues as separate ops around each projection at decode time
 * (tidal/models/llama.py:182-208: rms_norm_forward, the cuBLAS GEMV of nn.Linear, the residual
 * add; tidal/models/llama.py:160-170: act_fn(gate_proj(x)) * up_proj(x)):
 *   d_norm_weight != NULL   x is RMS-normalised first (weight [K], norm_eps, rounding as in tidal_rms_norm);
 *   d_residual != NULL      y = round(x W^T) + residual ([M][N], may be d_y itself);
 *   TIDAL_LINEAR_SILU_MUL   W stacks the gate rows over the up rows (N = 2 F): y[M][F] = silu(gate) * up,
 *                           each factor rounded to dtype as the separate torch ops would.
 * K must be a multiple of 8 (4 for fp32); x, W and the norm weight 16-byte aligned. */
#define TIDAL_LINEAR_PLAIN 0
#define TIDAL_LINEAR_SILU_MUL 1
typedef struct {
    const void* d_x;            /* [M][K] */
    const void* d_w;            /* [N][K] */
    void* d_y;                  /* [M][N], or [M][N/2] for TIDAL_LINEAR_SILU_MUL */
    const void* d_residual;     /* optional */
    const void* d_norm_weight;  /* optional [K] */
    float norm_eps;
    int32_t norm_round_before_weight;
    int32_t M, N, K;
    int32_t dtype;
    int32_t epilogue;
    uint32_t* d_status;         /* optional: TIDAL_DEV_* bits are OR-ed in (a wait on the staging ring that ran out) */
    int32_t static_weights;     /* 1: W was not written by the kernel that precedes this call in the stream (model
                                 * weights): the kernel starts fetching W before it is ordered after that kernel */
} tidal_linear_args;
int tidal_decode_linear(const tidal_linear_args* args, void* stream);

/* The q|k|v projection of a decoder layer with tidal_rope_append folded in: W stacks the Hq query
 * heads, the Hkv key heads and the Hkv value heads ((Hq + 2 Hkv) * D rows); q comes out rotated in
 * rope->d_q ([M][Hq][D]), k (rotated) and v go straight into the slot of each sequence's newest token
 * in the paged KV pool.  `lin` gives x, W, M, K and the optional RMSNorm (d_y, d_residual and epilogue
 * are ignored); `rope` gives the destinations and the RoPE as for tidal_rope_append (batch = M,
 * tokens_per_seq = 1; d_k and d_v are ignored).  f16/bf16 only. */
#define TIDAL_LINEAR_QKV_ROPE 2
int tidal_decode_qkv(const tidal_linear_args* lin, const tidal_rope_append_args* rope, void* stream);

/* ------------------------------------------------------- peer all-gather
 * All-gather of one block per rank over NVLink peer stores, for the per-layer exchange of
 * sequence-sharded KV (no reference counterpart; stands where a library all-gather would), with the
 * work that follows the exchange done in the same launch: the merge of the ranks' softmax partials
 * and the ranking of their top-k candidates.  Every rank runs one process per GPU and calls this
 * with the same `bytes`; when the kernel has finished, d_recv (if given) holds rank r's block at
 * byte r * slot_bytes.  Memory the caller sets up once:
 *   staging   per rank 2 * world * slot_bytes bytes, mapped on every rank (CUDA IPC / fabric handles);
 *             d_peer_stage[r] is rank r's staging buffer as addressed from this GPU (r = rank: its own);
 *   flags     per rank 2 * world * TIDAL_XCHG_MAX_CTAS uint32, zeroed, mapped the same way: d_peer_count[r];
 *   d_state   4 uint32 of this rank's own memory, zeroed.
 * d_peer_stage and d_peer_count are device arrays of `world` pointers.  Nothing is reset between
 * calls.  Contract across calls on one set of buffers: slot_bytes, world and rank never change; `bytes`
 * and the optional parts may differ from call to call (every CTA of a rank publishes the NUMBER of the
 * exchange in its own flag word on every peer, and a call waits for as many flags per rank as it has
 * CTAs itself) as long as every rank passes the same values in the same call; the ranks issue their
 * calls in the same order, each counting its own calls.
 * A rank that never arrives makes the others' bounded waits run out (wait_limit polls, 0 = the
 * default of about half a second): TIDAL_DEV_WAIT_TIMEOUT is OR-ed into *d_status (if given) and the
 * call completes with incomplete data.  If the ranks' call counts no longer agree after that (a rank
 * skipped the call rather than being late), every later call on these buffers would time out or read
 * stale blocks: tidal_peer_exchange_reset must run on EVERY rank, with no exchange in flight anywhere
 * (a host-side barrier before and after), before the buffers are used again. */
#define TIDAL_XCHG_MAX_CTAS 64
typedef struct {
    const void* d_send;
    void* d_recv;                /* NULL when only the merge / the ranking are wanted */
    int64_t bytes;               /* multiple of 16, <= slot_bytes */
    int64_t slot_bytes;          /* multiple of 16 */
    void* const* d_peer_stage;
    uint32_t* const* d_peer_count;
    uint32_t* d_state;
    uint32_t* d_status;
    int32_t rank, world;
    /* optional: the blocks hold softmax partials of sequence-sharded attention — m [rows], l [rows],
     * o [rows][head_dim] fp32 at these word offsets — and the kernel also writes their exact merge (as
     * tidal_merge_partials would) to d_merge_out [rows][head_dim] of merge_dtype */
    void* d_merge_out;
    int64_t merge_m_off, merge_l_off, merge_o_off;
    int32_t merge_rows, merge_head_dim, merge_dtype;
    int32_t wait_limit;          /* polls before a CTA gives up on the other ranks; 0 = default */
    /* optional (cand_rows > 0): the blocks also hold every rank's top-k candidates — scores
     * [cand_rows][cand_k] fp32 and global positions [cand_rows][cand_k] int32 at these word offsets, each
     * rank's in ascending position order, ranks holding ascending position ranges — and the kernel ranks,
     * per row, the world * cand_k candidates as tidal_topk would (k = cand_select, ties towards the lower
     * position): the selected positions p with own_lo <= p < own_hi are written as p - own_lo, ascending,
     * to d_sel_out[row * sel_stride ...] and their number to d_sel_count[row] (own_hi <= own_lo: all of
     * them, unshifted).  Limits: cand_select <= 2048, world * cand_k <= 65536, cand_select < world * cand_k. */
    int32_t cand_rows, cand_k, cand_select;
    int64_t cand_score_off, cand_idx_off;
    int32_t own_lo, own_hi;
    int32_t* d_sel_out;
    int64_t sel_stride;
    int32_t* d_sel_count;
} tidal_exchange_args;
int tidal_peer_all_gather(const tidal_exchange_args* args, void* stream);
/* Zeroes this rank's flag words (d_count = d_peer_count[rank], 2 * world * TIDAL_XCHG_MAX_CTAS words) and d_state on
 * the stream.  See tidal_peer_all_gather for when and how: every rank, nothing in flight. */
int tidal_peer_exchange_reset(uint32_t* d_count, uint32_t* d_state, int world, void* stream);

/* ------------------------------------------------------------------ prefill
 * Causal attention of n_q new query rows of ONE sequence over its paged KV, which already holds
 * the new rows' K,V (row i of q sits at position kv_len - n_q + i and sees tokens 0..that position;
 * causal = 0: every row sees all kv_len tokens).  Replaces prefill_with_paged_kv_cache
 * (tidal/ops/csrc/bsk_ops.h:78-86, tidal/ops/csrc/batch_prefill.cu:27-117, kernel
 * kernels/include/prefill/prefill.cuh:688-870); RoPE is applied beforehand (tidal_rope_append), as
 * the reference's modules do (tidal/models/SearchAttention.py:154-163).  f16/bf16 (tensor cores) or
 * fp32 (CUDA cores: the tensor cores have no fp32 operand mode), head_dim 64 or 128, NHD pool [pages][2][page_size][num_kv_heads][head_dim]; d_page_table lists the sequence's
 * pages in order.  sm_scale <= 0 means 1/sqrt(head_dim).  Allocates nothing, needs no workspace. */
typedef struct {
    const void* d_q;             /* [n_q][num_qo_heads][head_dim] */
    void* d_o;                   /* [n_q][num_qo_heads][head_dim] */
    const void* d_kv;
    const int32_t* d_page_table; /* [ceil(kv_len / page_size)] */
    uint32_t* d_status;          /* optional: TIDAL_DEV_* bits are OR-ed in */
    int64_t kv_len;
    int32_t n_q, num_qo_heads, num_kv_heads, head_dim, page_size, dtype, causal;
    float sm_scale;
    int64_t num_pages;           /* pages in the pool: a table entry outside [0, num_pages) is not followed (its
                                    tokens read as zeros) and TIDAL_DEV_BAD_INDEX is OR-ed into *d_status */
} tidal_prefill_args;
int tidal_prefill(const tidal_prefill_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TIDAL_B200_H_ */
