/*
 * twilight_b200 -- C ABI of the Select-then-Prune decode path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle, launches
 * on that stream and returns; no entry point allocates, frees, synchronises or keeps state
 * (apart from one-time cudaFuncSetAttribute calls).  All buffers, workspaces included, are
 * owned by the caller.  Return value: TWL_OK (0) or a negative twl_status; nothing throws.
 *
 * The reference project (tsinghua-ideal/Twilight) binds its native code through pybind11
 * (csrc/src/sampling.cu:65-70).  Each declaration below names the reference interface it
 * stands in for.
 *
 * Shared conventions
 *   dtype        TWL_F16 or TWL_BF16: element type of q, K/V pages, page metadata and out.
 *   paged KV     FlashInfer-style CSR page table, the one the reference's GEMV call sites use
 *                (benchmark/efficiency/bench_gemv.py:437-454): kv_indptr[B+1],
 *                kv_indices[kv_indptr[B]] physical page ids, kv_last_page_len[B] in 1..16.
 *                Sequence b has n_b = kv_indptr[b+1]-kv_indptr[b] pages and
 *                (n_b-1)*16 + kv_last_page_len[b] tokens.  Page size is fixed at 16.
 *   K/V pages    [num_pages][H_kv][16][128] elements: one (page, kv-head) slab = 4 KiB.
 *   INT4 K page  [num_pages][H_kv][1280] bytes: bytes 0..1023 = 16 tokens x 64 code bytes
 *                (byte j of a token holds channel 2j in its low nibble and 2j+1 in its high
 *                nibble); bytes 1024..1279 = 16 tokens x 4 groups x {fp16 scale, fp16 min}.
 *                Dequantised value = code*scale + min.  Group = 32 channels, head_dim = 128.
 *   page meta    [num_pages][H_kv][2][128] elements: channel-wise {min, max} of the page.
 *   candidates   cand_pages[B][H_q][max_k] logical page numbers (index into the sequence's
 *                page list), ascending; cand_npages[B][H_q].  Candidate slot s of a row is
 *                token cand_pages[s/16]*16 + s%16.
 *   status       optional int32 device word; kernels OR bits of twl_device_flag into it.
 */
#ifndef TWILIGHT_B200_H_
#define TWILIGHT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TWL_API __attribute__((visibility("default")))
#else
#define TWL_API
#endif

typedef enum {
  TWL_OK = 0,
  TWL_ERR_BAD_ARG = -1,      /* null pointer, zero/negative size, inconsistent sizes   */
  TWL_ERR_MISALIGNED = -2,   /* a pointer or stride breaks the documented alignment     */
  TWL_ERR_UNSUPPORTED = -3,  /* head_dim != 128, page size != 16, unknown dtype, ...    */
  TWL_ERR_LAUNCH = -4,       /* the CUDA runtime rejected a launch (see twl_last_cuda_error) */
  TWL_ERR_TOO_LARGE = -5,    /* a size exceeds what the kernel or a workspace can hold  */
  TWL_ERR_WORKSPACE = -6     /* workspace pointer null or too small                     */
} twl_status;

typedef enum { TWL_F16 = 0, TWL_BF16 = 1 } twl_dtype;

typedef enum {
  TWL_FLAG_ITER_CAP = 1,     /* the top-p search hit its round limit                    */
  TWL_FLAG_BAD_INDEX = 2,    /* an index/page id was out of range and was skipped       */
  TWL_FLAG_WAIT_LIMIT = 4    /* a bounded wait on a copy barrier ran out                */
} twl_device_flag;

#define TWL_PAGE_SIZE 16
#define TWL_HEAD_DIM 128
#define TWL_QUANT_GROUP 32
#define TWL_K4_SLAB_BYTES 1280
#define TWL_STATIC_ATTN_MAX_ROWS 512  /* row limit (batch*query heads) of twl_sparse_decode_attn_static */

TWL_API int twl_version(void);
TWL_API const char* twl_status_string(int status);
/* cudaGetErrorString of the last launch error seen by this library on this thread. */
TWL_API const char* twl_last_cuda_error(void);

/* ---- kernel #2, reference-compatible form ------------------------------------------
 * Replaces top_p_fp32_return_mask / top_p_fp16_return_mask of csrc/src/sampling.cu:45-63
 * and :22-43 (launcher csrc/include/sampling.cuh:233-250, kernel :119-231).
 * probs: [rows][d] contiguous probabilities (rows = batch*num_heads); mask: [rows][d]
 * bytes, written 0/1; top_p_arr: [rows] fp32 or NULL (then top_p_val is used).
 * Same search as the reference: low=0, high=probs[row][0], eps=1e-5, mask = probs > low.
 * The f16 form takes fp16 or bf16 probabilities and reproduces the reference's arithmetic in that
 * type: p, eps, low, high, mid and the stop width are rounded to it, and the mass above the pivot
 * is added in it, in the order of the reference's 1024-thread block reduction (per chunk of
 * 1024*gcd(8,d) elements: the thread's items in order, a shuffle-down tree per warp, the warp
 * totals in order).  The masks equal the reference kernel's bit for bit. */
TWL_API int twl_top_p_return_mask_f32(const float* probs, uint8_t* mask, const float* top_p_arr,
                              float top_p_val, uint32_t rows, uint32_t d, int32_t* status,
                              void* stream);
TWL_API int twl_top_p_return_mask_f16(const void* probs, int dtype, uint8_t* mask,
                              const float* top_p_arr, float top_p_val, uint32_t rows,
                              uint32_t d, int32_t* status, void* stream);

/* ---- selector: Quest page scores + top-k pages ---------------------------------------
 * Replaces quest_selector of twilight/pyimpl/quest.py:17-122 using stored page metadata:
 * score(page) = sum_d max(q_d*kmax_d, q_d*kmin_d) in fp32 (quest.py:37-84; for groups of 4 or 8
 * query heads per KV head evaluated as [min|max] . [min(q,0);max(q,0)] on tensor cores), then the
 * max(1,budget/16)+(budget%16!=0) best pages per query head (quest.py:93-99), ties to the
 * lower page number.  page_scores: caller scratch [B][H_q][max_pages] fp32 (kept as an
 * output for inspection).  cand_pages rows are ascending. */
TWL_API int twl_quest_page_scores(const void* q, int dtype, const void* kmeta,
                          const int32_t* kv_indptr, const int32_t* kv_indices,
                          int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                          int32_t num_pages_total, float* page_scores, int32_t max_pages,
                          int32_t* status, void* stream);
TWL_API int twl_quest_topk_pages(const float* page_scores, int32_t max_pages,
                         const int32_t* kv_indptr, int32_t batch, int32_t num_q_heads,
                         int32_t token_budget, int32_t* cand_pages, int32_t* cand_npages,
                         int32_t max_k, void* stream);

/* Both steps in one launch: the block that finishes the scores of a (batch, kv-head) row last
 * (an atomic ticket, nobody waits) picks that row's pages.  counters: int32[batch*num_kv_heads],
 * zero on entry, left zero.  Same results as the two calls above. */
TWL_API int twl_quest_select(const void* q, int dtype, const void* kmeta, const int32_t* kv_indptr,
                             const int32_t* kv_indices, int32_t batch, int32_t num_q_heads,
                             int32_t num_kv_heads, int32_t num_pages_total, int32_t token_budget,
                             float* page_scores, int32_t max_pages, int32_t* cand_pages,
                             int32_t* cand_npages, int32_t max_k, int32_t* counters,
                             int32_t* status, void* stream);

/* ---- kernel #1: INT4 K-cache q.k estimator --------------------------------------------
 * Replaces the estimator of twilight/pyimpl/attention.py:247-255 (with quantize.py:4-13
 * applied once at cache-append time) and the absent ftka op batched_sparse_gemv_int4_k
 * (call site benchmark/efficiency/bench_gemv.py:445-454).
 * scores[b][h][s] = sm_scale * sum_d q_d*(code_d*scale_g + min_g), fp32; slots of the last
 * page past the end of the sequence are -inf; slots past the row's last candidate page are
 * not written.  score_stride must be a multiple of 16.
 * cand_pages == NULL: every page of the sequence is a candidate (slot == token position),
 * K pages are read once per KV head for its whole query-head group.
 * variant: arithmetic 0 = library default (3), 1 = fp32 FMA, 2 = packed-half FMA (about 1e-2
 * off in the logit), 3 = integer dot product; add 16 for the kernel that uses direct 128-bit
 * global loads, add 128 for the block-wide bulk-copy (TMA) ring even when a row has a single
 * query head (by default such rows use warp-private 16-byte async copies), add 64 for warp-private
 * rings fed by bulk copies (two 1280-byte cp.async.bulk per stage on the warp's own mbarrier: the
 * default's block shape and bytes in flight, the copy engine instead of per-lane copies), add 32 for the
 * integer-dot kernel on query-head groups, add 256 for 16-bit float tensor-core tiles on them (codes
 * and q exact in fp16, fp32 accumulation).  By default groups of 2, 4 or 8 heads that share a KV
 * head's pages are scored with 8-bit integer tensor-core tiles: q as 13-bit block-scaled integers
 * split into a high and a low byte (the integer dot product is exact; q is rounded to 2^-13 of the
 * head's largest element, as in the single-head kernel).  Groups of 2 and 4 heads put both bytes of
 * every head into the eight columns of ONE m16n8k32 tile per page and 32-channel quantisation
 * group (and round q to 2^-15 of the head's largest element: each byte's sum has an accumulator of its own); groups of 8 heads use one tile for the high and one for the low bytes (add 512 to use
 * that form for the smaller groups too).  The non-default variants exist for measurement. */
TWL_API int twl_estimate_int4(const void* q, int dtype, const uint8_t* k4_pages,
                      const int32_t* kv_indptr, const int32_t* kv_indices,
                      const int32_t* kv_last_page_len, const int32_t* cand_pages,
                      const int32_t* cand_npages, int32_t max_k, int32_t batch,
                      int32_t num_q_heads, int32_t num_kv_heads, int32_t num_pages_total,
                      float sm_scale, float* scores, int32_t score_stride, int32_t variant,
                      int32_t* status, void* stream);

/* ---- kernel #2: softmax + top-p threshold search + compaction -------------------------
 * Replaces top_p_unnormalized (twilight/pyimpl/top_p.py:10-15) followed by the mask op and
 * the AND/count of attention.py:280-285, emitting an index list instead of a dense mask.
 * scores: [rows][score_stride] fp32 as written by twl_estimate_int4 (rows = B*H_q);
 * out_indices[row][0..budget) = kept token positions, ascending; out_budget[row].
 * out_threshold (nullable) [rows][2] = {low, p(token 0)}.  rows with no candidate get 0.
 * A top_p above 1 skips the search and keeps every candidate whose probability is non-zero
 * (the reference's pruner "none").  Only slots below 16*(candidate pages of the row) are read.
 * Rows of up to 40960 slots are searched in shared memory, longer rows from global memory. */
TWL_API int twl_topp_prune(const float* scores, int32_t score_stride, const int32_t* kv_indptr,
                   const int32_t* kv_last_page_len, const int32_t* cand_pages,
                   const int32_t* cand_npages, int32_t max_k, int32_t batch,
                   int32_t num_q_heads, const float* top_p_arr, float top_p_val,
                   int32_t* out_indices, int32_t index_stride, int32_t* out_budget,
                   float* out_threshold, int32_t* status, void* stream);

/* Element-wise threshold pruner on the same scores, replacing elementwise_threshold of
 * twilight/pyimpl/elementwise_threshold.py:9-18: a candidate is kept when its score exceeds
 * (score of sequence token 0) - threshold; when token 0 is not a candidate every candidate is
 * kept.  Outputs as for twl_topp_prune; out_threshold = {cut, score of token 0}. */
TWL_API int twl_threshold_prune(const float* scores, int32_t score_stride, const int32_t* kv_indptr,
                                const int32_t* kv_last_page_len, const int32_t* cand_pages,
                                const int32_t* cand_npages, int32_t max_k, int32_t batch,
                                int32_t num_q_heads, float threshold, int32_t* out_indices,
                                int32_t index_stride, int32_t* out_budget, float* out_threshold,
                                int32_t* status, void* stream);

/* ---- kernel #3: sparse paged decode attention ------------------------------------------
 * Replaces attention.py:188-190 restricted to the kept tokens and :298-306 (masked fp32
 * softmax, P.V).  A row's kept tokens are cut into chunks of `chunk` tokens (a multiple of 32;
 * <= 0 selects 256; the chunk grows for rows that would need more than 32 of them) and the
 * (row, chunk) work items are dealt, long ones first, to a grid that fills the GPU once, so
 * heads with large budgets do not serialise.  The block that finishes a row's last chunk merges
 * the partial (max, sum, acc) triples; no block waits for another.
 * indices[row][0..budget) must be ascending (twl_topp_prune writes them so).  With 2, 4 or 8 query
 * heads per KV head, a (sequence, KV head) row whose heads keep, together, at least as many tokens
 * as the sequence has is served by a second kernel that reads every K/V page once for the whole
 * group and computes all its heads on tensor cores (softmax weights rounded to the model dtype
 * before P.V, as attention.py:302-304 does); the choice is made per row on the device.  That kernel
 * reads the index lists in 16-byte pieces: it is used only when `indices` is 16-byte aligned and
 * index_stride is a multiple of 4 (otherwise every row goes to the per-head kernel).
 * Limit: batch*num_q_heads <= 65536 (TWL_ERR_TOO_LARGE above).
 * workspace: twl_sparse_attn_workspace_bytes(...) bytes, 16-byte aligned; its first
 * batch*num_q_heads int32 words are arrival counters that must be zero on entry and are
 * left zero on exit.  Rows with budget 0 produce zeros. */
TWL_API size_t twl_sparse_attn_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                       int32_t index_stride, int32_t chunk);
TWL_API int twl_sparse_decode_attn(const void* q, int dtype, const void* k_pages, const void* v_pages,
                           const int32_t* kv_indptr, const int32_t* kv_indices,
                           const int32_t* indices, int32_t index_stride,
                           const int32_t* budget, int32_t batch, int32_t num_q_heads,
                           int32_t num_kv_heads, int32_t num_pages_total, float sm_scale,
                           void* out, void* workspace, size_t workspace_bytes, int32_t chunk,
                           int32_t* status, void* stream);

/* ---- attention over the estimated weights (use_estimated_weights_in_attn, -------------------
 * twilight/pyimpl/attention.py:295-296).  twl_prune_with_weights is twl_topp_prune (mode 0, value =
 * top-p) or twl_threshold_prune (mode 1, value = threshold) that also writes, next to every kept
 * token, its un-normalised softmax weight exp(estimated logit - row maximum) into
 * out_weights[rows][index_stride].  twl_sparse_decode_attn_weighted normalises those weights over
 * the kept tokens and applies them to V; K pages are not read. */
TWL_API int twl_prune_with_weights(int32_t mode, const float* scores, int32_t score_stride,
                                   const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                   const int32_t* cand_pages, const int32_t* cand_npages,
                                   int32_t max_k, int32_t batch, int32_t num_q_heads,
                                   const float* top_p_arr, float value, int32_t* out_indices,
                                   int32_t index_stride, int32_t* out_budget, float* out_threshold,
                                   float* out_weights, int32_t* status, void* stream);
TWL_API int twl_sparse_decode_attn_weighted(const void* q, int dtype, const void* k_pages,
                                            const void* v_pages, const int32_t* kv_indptr,
                                            const int32_t* kv_indices, const int32_t* indices,
                                            int32_t index_stride, const int32_t* budget,
                                            const float* weights, int32_t batch, int32_t num_q_heads,
                                            int32_t num_kv_heads, int32_t num_pages_total,
                                            float sm_scale, void* out, void* workspace,
                                            size_t workspace_bytes, int32_t chunk, int32_t* status,
                                            void* stream);

/* ---- kernel #3 without a caller workspace -------------------------------------------------
 * No counterpart in the reference.  Same computation and arguments as twl_sparse_decode_attn,
 * minus workspace/workspace_bytes: the split-KV scratch is a fixed array inside the library
 * image (about 8.4 MB per GPU that loads the library, kept until the process exits), so the
 * call itself never asks for device memory.  The array's memory is taken by the CUDA runtime when
 * the library's attention code is loaded onto a device, which (with CUDA's lazy module loading)
 * happens at the first attention call on that device, this one included: make one call per device
 * during start-up, before a memory pool claims what is left, or run with CUDA_MODULE_LOADING=EAGER.
 * It exists for hosts that cannot allocate after start-up: a serving process whose memory pool
 * already owns all free device memory, or a plugin that may only be called where cudaMalloc is
 * forbidden.
 * Limit: batch*num_q_heads <= TWL_STATIC_ATTN_MAX_ROWS, else TWL_ERR_TOO_LARGE.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call outside any stream capture.
 * Every call on a device uses the same array: the arrival counters are cleared on `stream` at
 * the start of each call, the rest is overwritten as needed; two calls whose kernels can overlap
 * on the GPU (different streams, no ordering between them) race on it and must not be issued. */
TWL_API int twl_sparse_decode_attn_static(const void* q, int dtype, const void* k_pages,
                                          const void* v_pages, const int32_t* kv_indptr,
                                          const int32_t* kv_indices, const int32_t* indices,
                                          int32_t index_stride, const int32_t* budget,
                                          int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                          int32_t num_pages_total, float sm_scale, void* out,
                                          int32_t chunk, int32_t* status, void* stream);

/* ---- the whole step behind one call -------------------------------------------------------
 * Replaces the decode branch of attention_forward, twilight/pyimpl/attention.py:188-306, with the
 * selector / estimator / pruner choices of its config dictionary (attention.py:360-376):
 * Quest page scores and top-k pages (token_budget > 0; <= 0 means selector "none"), the INT4
 * estimate, the pruner (TWL_PRUNER_TOP_P with pruner_value = p or the per-row top_p_arr,
 * TWL_PRUNER_THRESHOLD with pruner_value = the threshold, TWL_PRUNER_NONE) and the sparse
 * attention, as three launches (five with Quest; one more where 2, 4 or 8 query heads share a KV head:
 * the group attention kernel runs before the per-head one) on `stream`.
 * TWL_PRUNER_NONE keeps every candidate whose estimated probability is not zero in fp32 (the
 * reference's mask keeps all candidates, state.py:151-159 counts them all in the budget; the ones
 * dropped here weigh nothing in the attention, so the output is the same, but `budget` can be
 * smaller than the candidate count on rows with logit gaps beyond 87).
 * flags: TWL_STEP_ESTIMATED_WEIGHTS = attend with the estimated weights (attention.py:295-296);
 *        TWL_STEP_ROUND_TO_DTYPE = round the Quest page scores and the estimated logits to the model
 *        dtype where the reference's matmuls return that dtype (quest.py:76-84; attention.py:252-254,
 *        logits rounded before and after the division by sqrt(D)); two small extra launches, meant for
 *        comparisons with the reference's dtype path, not for speed.
 * All intermediates live in one caller-owned workspace of twl_step_workspace_bytes(...) bytes,
 * 256-byte aligned, ZEROED ONCE by the caller after allocation (the attention kernel's arrival
 * counters must start at zero; every call leaves them zero).  twl_step_workspace_layout gives the
 * byte offset of every part, so that a host can read the budgets (int32 [B][H_q]), the kept tokens
 * (int32 [B][H_q][stride], ascending, first budget entries valid), the candidate pages and the
 * scores after the call.  max_pages = the largest page count of a sequence (sizes the rows).
 * estimator_variant as for twl_estimate_int4 (0 = default); attn_chunk as for
 * twl_sparse_decode_attn (<= 0 selects 256). */
typedef enum { TWL_PRUNER_TOP_P = 0, TWL_PRUNER_THRESHOLD = 1, TWL_PRUNER_NONE = 2 } twl_pruner;
typedef enum { TWL_STEP_ESTIMATED_WEIGHTS = 1, TWL_STEP_ROUND_TO_DTYPE = 2 } twl_step_flag;
typedef struct {
  uint64_t attn, attn_bytes;     /* split-KV scratch of the attention kernel (first in the buffer) */
  uint64_t page_scores;          /* float [B][H_q][max_pages]          (Quest only) */
  uint64_t cand_pages;           /* int32 [B][H_q][max_k]              (Quest only) */
  uint64_t cand_npages;          /* int32 [B][H_q]                     (Quest only) */
  uint64_t scores;               /* float [B][H_q][stride] estimated logits */
  uint64_t indices;              /* int32 [B][H_q][stride] kept tokens */
  uint64_t budget;               /* int32 [B][H_q] */
  uint64_t threshold;            /* float [B][H_q][2] {cut, value of token 0} */
  uint64_t weights;              /* float [B][H_q][stride] (TWL_STEP_ESTIMATED_WEIGHTS only) */
  uint64_t total;                /* bytes of the whole workspace */
  int32_t max_k;                 /* candidate pages per row (0 without Quest) */
  int32_t stride;                /* slots per row of scores / indices / weights */
  int32_t kernels;               /* launches one call makes */
  int32_t reserved;
} twl_step_layout;
TWL_API int twl_step_workspace_layout(int32_t batch, int32_t num_q_heads, int32_t max_pages,
                                      int32_t token_budget, int32_t attn_chunk, int32_t flags,
                                      twl_step_layout* out);
TWL_API size_t twl_step_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t max_pages,
                                        int32_t token_budget, int32_t attn_chunk, int32_t flags);
TWL_API int twl_select_prune_attend_step(
    const void* q, int dtype, const void* k_pages, const void* v_pages, const uint8_t* k4_pages,
    const void* kmeta, const int32_t* kv_indptr, const int32_t* kv_indices,
    const int32_t* kv_last_page_len, int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
    int32_t num_pages_total, int32_t max_pages, int32_t token_budget, int32_t pruner,
    float pruner_value, const float* top_p_arr, float sm_scale, int32_t flags,
    int32_t estimator_variant, int32_t attn_chunk, void* out, void* workspace,
    size_t workspace_bytes, int32_t* status, void* stream);

/* scores[i] <- round(round(scores[i]) * post_scale), both roundings to `dtype` (fp16 or bf16), in
 * place on n fp32 values; the step above uses it for TWL_STEP_ROUND_TO_DTYPE.  Stands in for the
 * model-dtype results of the reference's matmuls (quest.py:76-84, attention.py:252-254). */
TWL_API int twl_round_scores(float* scores, int64_t n, int dtype, float post_scale, void* stream);

/* ---- cache-append side ------------------------------------------------------------------
 * twl_quantize_k_pages: min/max asymmetric 4-bit quantiser of quantize.py:4-13 applied per
 * group of 32 channels, arithmetic in `dtype` like the reference, packing into INT4 slabs.
 * n_slabs = num_pages*H_kv.  twl_build_page_meta: channel-wise min/max over the valid
 * tokens of every page of every sequence (the chunk maxima of quest.py:39-74 in stored
 * form).  twl_append_kv: writes one new token per sequence (its position is the last
 * token the page table describes), quantises its K and folds it into the page metadata. */
TWL_API int twl_quantize_k_pages(const void* k_pages, int dtype, uint8_t* k4_pages, int64_t n_slabs,
                         void* stream);
TWL_API int twl_build_page_meta(const void* k_pages, int dtype, void* kmeta, const int32_t* kv_indptr,
                        const int32_t* kv_indices, const int32_t* kv_last_page_len,
                        int32_t batch, int32_t num_kv_heads, int32_t num_pages_total,
                        int32_t max_pages, void* stream);
TWL_API int twl_append_kv(const void* new_k, const void* new_v, int dtype, void* k_pages,
                  void* v_pages, uint8_t* k4_pages, void* kmeta, const int32_t* kv_indptr,
                  const int32_t* kv_indices, const int32_t* kv_last_page_len, int32_t batch,
                  int32_t num_kv_heads, int32_t num_pages_total, int32_t* status,
                  void* stream);

/* Index list -> dense byte mask [rows][d] (the mask interface of twilight/pyimpl: selectors
 * and pruners return bool[B,H,1,L], attention.py:199-281).  mask must be zeroed by the caller. */
TWL_API int twl_indices_to_mask(const int32_t* indices, int32_t index_stride, const int32_t* budget,
                        int32_t rows, uint8_t* mask, int32_t d, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TWILIGHT_B200_H_ */
