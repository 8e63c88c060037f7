// The whole decode step of one attention layer behind one C call:
//   Quest page scores -> top-k pages -> INT4 estimate -> pruner -> sparse attention
// i.e. the decode branch of attention_forward in twilight/pyimpl/attention.py:188-306, issued as
// three launches (five with the Quest selector) on the caller's stream.  The intermediates live
// in ONE caller-owned workspace whose layout twl_step_workspace_layout describes, so that a host
// written in C or C++ sizes one buffer instead of six and a Python host can view the parts.
#include "common.cuh"

namespace twl {

static inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }

// x -> round(round(x) * post_scale), rounding to fp16 or bf16; -inf stays -inf.
// With post_scale = 1 this is a plain rounding of fp32 scores to the model dtype
// (the reference's matmuls return the model dtype: quest.py:76-84, attention.py:252-254).
struct RoundParams {
  float* x;
  int64_t n;
  float post_scale;
};
template <typename T>
__global__ void __launch_bounds__(256) round_scores_chain_kernel(const RoundParams p) {
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < p.n; i += (int64_t)gridDim.x * 256) {
    const float v = Elem<T>::to_f(Elem<T>::from_f(p.x[i]));
    p.x[i] = Elem<T>::to_f(Elem<T>::from_f(v * p.post_scale));
  }
}

}  // namespace twl

extern "C" int twl_round_scores(float* scores, int64_t n, int dtype, float post_scale, void* stream) {
  using namespace twl;
  if (!scores || n <= 0) return TWL_ERR_BAD_ARG;
  const int64_t want = (n + 255) / 256;
  const unsigned grid = (unsigned)(want < (int64_t)num_sms() * 8 ? want : (int64_t)num_sms() * 8);
  RoundParams rp;
  rp.x = scores; rp.n = n; rp.post_scale = post_scale;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) {
    TWL_CUDA_TRY(launch_chain(round_scores_chain_kernel<__half>, dim3(grid), dim3(256), 0, st, rp));
  } else if (dtype == TWL_BF16) {
    TWL_CUDA_TRY(launch_chain(round_scores_chain_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, rp));
  } else {
    return TWL_ERR_UNSUPPORTED;
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

extern "C" int twl_step_workspace_layout(int32_t batch, int32_t num_q_heads, int32_t max_pages,
                                         int32_t token_budget, int32_t attn_chunk, int32_t flags,
                                         twl_step_layout* out) {
  using namespace twl;
  if (!out || batch <= 0 || num_q_heads <= 0 || max_pages <= 0) return TWL_ERR_BAD_ARG;
  if (attn_chunk <= 0) attn_chunk = 256;
  if (attn_chunk % 32 != 0) return TWL_ERR_BAD_ARG;
  const size_t rows = (size_t)batch * num_q_heads;
  const bool quest = token_budget > 0;
  int32_t max_k = 0;
  if (quest) {
    max_k = (token_budget / kPage > 1 ? token_budget / kPage : 1) + (token_budget % kPage != 0 ? 1 : 0);
    if (max_k > max_pages) max_k = max_pages;
  }
  const int64_t stride64 = (int64_t)(quest ? max_k : max_pages) * kPage;
  if (stride64 > 0x7fffffff) return TWL_ERR_TOO_LARGE;
  const int32_t stride = (int32_t)stride64;
  twl_step_layout l;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += up256(bytes);
    return (uint64_t)at;
  };
  // the attention scratch comes first: its leading arrival counters must be zero on entry
  l.attn_bytes = twl_sparse_attn_workspace_bytes(batch, num_q_heads, stride, attn_chunk);
  l.attn = take(l.attn_bytes);
  l.page_scores = take(quest ? rows * (size_t)max_pages * sizeof(float) : 0);
  l.cand_pages = take(quest ? rows * (size_t)max_k * sizeof(int32_t) : 0);
  l.cand_npages = take(quest ? rows * sizeof(int32_t) : 0);
  l.scores = take(rows * (size_t)stride * sizeof(float));
  l.indices = take(rows * (size_t)stride * sizeof(int32_t));
  l.budget = take(rows * sizeof(int32_t));
  l.threshold = take(rows * 2 * sizeof(float));
  l.weights = take((flags & TWL_STEP_ESTIMATED_WEIGHTS) ? rows * (size_t)stride * sizeof(float) : 0);
  l.total = off;
  l.max_k = max_k;
  l.stride = stride;
  l.kernels = (quest ? 2 : 0) + 3 + ((flags & TWL_STEP_ROUND_TO_DTYPE) ? (quest ? 2 : 1) : 0);
  l.reserved = 0;
  *out = l;
  return TWL_OK;
}

extern "C" size_t twl_step_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t max_pages,
                                           int32_t token_budget, int32_t attn_chunk, int32_t flags) {
  twl_step_layout l;
  if (twl_step_workspace_layout(batch, num_q_heads, max_pages, token_budget, attn_chunk, flags, &l) != TWL_OK)
    return 0;
  return (size_t)l.total;
}

extern "C" int twl_select_prune_attend_step(
    const void* q, int dtype, const void* k_pages, const void* v_pages, const uint8_t* k4_pages,
    const void* kmeta, const int32_t* kv_indptr, const int32_t* kv_indices,
    const int32_t* kv_last_page_len, int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
    int32_t num_pages_total, int32_t max_pages, int32_t token_budget, int32_t pruner,
    float pruner_value, const float* top_p_arr, float sm_scale, int32_t flags,
    int32_t estimator_variant, int32_t attn_chunk, void* out, void* workspace,
    size_t workspace_bytes, int32_t* status, void* stream) {
  using namespace twl;
  if (!q || !k_pages || !v_pages || !k4_pages || !kv_indptr || !kv_indices || !kv_last_page_len || !out)
    return TWL_ERR_BAD_ARG;
  if (pruner != TWL_PRUNER_TOP_P && pruner != TWL_PRUNER_THRESHOLD && pruner != TWL_PRUNER_NONE)
    return TWL_ERR_BAD_ARG;
  const bool quest = token_budget > 0;
  if (quest && !kmeta) return TWL_ERR_BAD_ARG;
  if (attn_chunk <= 0) attn_chunk = 256;
  twl_step_layout l;
  int rc = twl_step_workspace_layout(batch, num_q_heads, max_pages, token_budget, attn_chunk, flags, &l);
  if (rc != TWL_OK) return rc;
  if (!workspace || workspace_bytes < l.total) return TWL_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return TWL_ERR_MISALIGNED;
  char* ws = static_cast<char*>(workspace);
  float* page_scores = reinterpret_cast<float*>(ws + l.page_scores);
  int32_t* cand_pages = quest ? reinterpret_cast<int32_t*>(ws + l.cand_pages) : nullptr;
  int32_t* cand_npages = quest ? reinterpret_cast<int32_t*>(ws + l.cand_npages) : nullptr;
  float* scores = reinterpret_cast<float*>(ws + l.scores);
  int32_t* indices = reinterpret_cast<int32_t*>(ws + l.indices);
  int32_t* budget = reinterpret_cast<int32_t*>(ws + l.budget);
  float* threshold = reinterpret_cast<float*>(ws + l.threshold);
  const bool est_w = (flags & TWL_STEP_ESTIMATED_WEIGHTS) != 0;
  const bool rounded = (flags & TWL_STEP_ROUND_TO_DTYPE) != 0;
  float* weights = est_w ? reinterpret_cast<float*>(ws + l.weights) : nullptr;
  const int64_t rows = (int64_t)batch * num_q_heads;

  if (quest) {
    rc = twl_quest_page_scores(q, dtype, kmeta, kv_indptr, kv_indices, batch, num_q_heads, num_kv_heads,
                               num_pages_total, page_scores, max_pages, status, stream);
    if (rc != TWL_OK) return rc;
    if (rounded) {
      rc = twl_round_scores(page_scores, rows * max_pages, dtype, 1.0f, stream);
      if (rc != TWL_OK) return rc;
    }
    rc = twl_quest_topk_pages(page_scores, max_pages, kv_indptr, batch, num_q_heads, token_budget, cand_pages,
                              cand_npages, l.max_k, stream);
    if (rc != TWL_OK) return rc;
  }
  rc = twl_estimate_int4(q, dtype, k4_pages, kv_indptr, kv_indices, kv_last_page_len, cand_pages, cand_npages,
                         l.max_k, batch, num_q_heads, num_kv_heads, num_pages_total, rounded ? 1.0f : sm_scale,
                         scores, l.stride, estimator_variant, status, stream);
  if (rc != TWL_OK) return rc;
  if (rounded) {
    rc = twl_round_scores(scores, rows * l.stride, dtype, sm_scale, stream);
    if (rc != TWL_OK) return rc;
  }
  // pruner "none" keeps every candidate with non-zero probability: a top-p above 1 does that
  const int mode = pruner == TWL_PRUNER_THRESHOLD ? 1 : 0;
  const float value = pruner == TWL_PRUNER_NONE ? 2.0f : pruner_value;
  const float* arr = pruner == TWL_PRUNER_TOP_P ? top_p_arr : nullptr;
  if (est_w) {
    rc = twl_prune_with_weights(mode, scores, l.stride, kv_indptr, kv_last_page_len, cand_pages, cand_npages,
                                l.max_k, batch, num_q_heads, arr, value, indices, l.stride, budget, threshold,
                                weights, status, stream);
  } else if (mode == 1) {
    rc = twl_threshold_prune(scores, l.stride, kv_indptr, kv_last_page_len, cand_pages, cand_npages, l.max_k,
                             batch, num_q_heads, value, indices, l.stride, budget, threshold, status, stream);
  } else {
    rc = twl_topp_prune(scores, l.stride, kv_indptr, kv_last_page_len, cand_pages, cand_npages, l.max_k, batch,
                        num_q_heads, arr, value, indices, l.stride, budget, threshold, status, stream);
  }
  if (rc != TWL_OK) return rc;
  if (est_w)
    return twl_sparse_decode_attn_weighted(q, dtype, k_pages, v_pages, kv_indptr, kv_indices, indices, l.stride,
                                           budget, weights, batch, num_q_heads, num_kv_heads, num_pages_total,
                                           sm_scale, out, ws + l.attn, (size_t)l.attn_bytes, attn_chunk, status,
                                           stream);
  return twl::sparse_decode_attn_bounded(q, dtype, k_pages, v_pages, kv_indptr, kv_indices, indices, l.stride,
                                         budget, nullptr, batch, num_q_heads, num_kv_heads, num_pages_total,
                                         sm_scale, out, ws + l.attn, (size_t)l.attn_bytes, attn_chunk, status,
                                         stream, max_pages);
}
