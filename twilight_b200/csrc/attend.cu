// Kernel #3: sparse paged decode attention over the pruned token lists.
//
// Stands in for twilight/pyimpl/attention.py:188-190 (exact q.k logits, here only for the
// kept tokens) and :298-306 (masked fp32 softmax, P.V).  The reference computes the dense
// [L] row and masks it; here a row's cost is its budget.
//
// Split-KV: the indices of one (batch, query head) row are cut into chunks of `chunk`; up to
// kMaxSplits blocks share a row, block x taking chunks x, x+splits, ... and carrying one running
// (max, sum, acc) across them.  A warp takes 32 indices at a time: each lane resolves one token to its K/V row
// through the page table, then the warp walks the 32 rows four at a time, every lane owning
// 4 of the 128 channels (one 8-byte load per K row and per V row), with an online softmax
// (running max, sum, 4 accumulators per lane).  Warps merge through shared memory; blocks of
// a row merge through the caller's workspace, and the block that arrives last (an atomic
// ticket, nobody waits) writes the output.
#include <algorithm>

#include "common.cuh"

namespace twl {

constexpr int kAttThreads = 128;
constexpr int kAttWarps = kAttThreads / 32;
constexpr int kMaxSplits = 8;        // blocks per row
constexpr float kNegBig = -3.0e38f;  // finite stand-in for -inf so that exp(m_old-m_new) is defined

struct AttParams {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* indptr;
  const int32_t* indices;
  const int32_t* idx;
  const int32_t* budget;
  void* out;
  int32_t* counters;  // [rows]
  float* part_ml;     // [rows][max_chunks][2]
  float* part_o;      // [rows][max_chunks][128]
  int32_t* status;
  int index_stride, B, Hq, Hkv, num_pages_total, chunk, max_chunks;
  float sm_scale;
};

template <typename T>
__global__ void __launch_bounds__(kAttThreads)
sparse_decode_attn_kernel(const AttParams p) {
  __shared__ float sm_o[kAttWarps][kD];
  __shared__ float sm_m[kAttWarps], sm_l[kAttWarps];
  __shared__ int sm_ticket;

  const int row = blockIdx.y, c = blockIdx.x;
  const int b = row / p.Hq, h = row % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  const int budget = min(p.budget[row], p.index_stride);
  const int n_chunks = (budget + p.chunk - 1) / p.chunk;
  const int n_parts = min(n_chunks, (int)gridDim.x);  // blocks of this row that have work
  T* out = reinterpret_cast<T*>(p.out) + (size_t)row * kD;
  if (budget <= 0) {
    if (c == 0) out[threadIdx.x] = Elem<T>::from_f(0.f);
    return;
  }
  if (c >= n_parts) return;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  const int32_t* idx = p.idx + (size_t)row * p.index_stride;
  const T* kbase = reinterpret_cast<const T*>(p.k);
  const T* vbase = reinterpret_cast<const T*>(p.v);

  // this lane's 4 channels of q, pre-multiplied by the softmax scale
  float qf[4];
  {
    uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const T*>(p.q) + (size_t)row * kD) + lane);
    float2 a = Elem<T>::to_f2(u.x), bq = Elem<T>::to_f2(u.y);
    qf[0] = a.x * p.sm_scale; qf[1] = a.y * p.sm_scale;
    qf[2] = bq.x * p.sm_scale; qf[3] = bq.y * p.sm_scale;
  }

  float m = kNegBig, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int cc = c; cc < n_chunks; cc += gridDim.x) {
  const int begin = cc * p.chunk, end = min(budget, begin + p.chunk);
  for (int t0 = begin + warp * 32; t0 < end; t0 += kAttWarps * 32) {
    // each lane resolves one token -> row number inside the K/V page arrays (-1 = skip)
    long long ro = -1;
    if (t0 + lane < end) {
      const int tok = idx[t0 + lane];
      const int pg = tok >> 4;
      if (tok >= 0 && pg < n_seq_pages) {
        const int phys = p.indices[page_base + pg];
        if (phys >= 0 && phys < p.num_pages_total)
          ro = ((long long)phys * p.Hkv + kvh) * kPage + (tok & 15);
      }
      if (ro < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
    }
    const int n_here = min(32, end - t0);
    for (int j = 0; j < n_here; j += 4) {
      uint2 kk[4], vv[4];
      bool ok[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long r = __shfl_sync(0xffffffffu, ro, (j + u) & 31);
        ok[u] = (j + u < n_here) && r >= 0;
        if (ok[u]) {
          kk[u] = ldg_stream_u2(kbase + r * kD + lane * 4);
          vv[u] = ldg_stream_u2(vbase + r * kD + lane * 4);
        } else {
          kk[u] = make_uint2(0, 0);
          vv[u] = make_uint2(0, 0);
        }
      }
      float s[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 k0 = Elem<T>::to_f2(kk[u].x), k1 = Elem<T>::to_f2(kk[u].y);
        s[u] = qf[0] * k0.x + qf[1] * k0.y + qf[2] * k1.x + qf[3] * k1.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
      }
      float m_new = m;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        s[u] = ok[u] ? s[u] : -INFINITY;
        m_new = fmaxf(m_new, s[u]);
      }
      const float scale = __expf(m - m_new);
      l *= scale;
#pragma unroll
      for (int d = 0; d < 4; ++d) acc[d] *= scale;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float pw = __expf(s[u] - m_new);
        l += pw;
        const float2 v0 = Elem<T>::to_f2(vv[u].x), v1 = Elem<T>::to_f2(vv[u].y);
        acc[0] = fmaf(pw, v0.x, acc[0]);
        acc[1] = fmaf(pw, v0.y, acc[1]);
        acc[2] = fmaf(pw, v1.x, acc[2]);
        acc[3] = fmaf(pw, v1.y, acc[3]);
      }
      m = m_new;
    }
  }
  }

  // merge the warps of this block
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
#pragma unroll
  for (int d = 0; d < 4; ++d) sm_o[warp][lane * 4 + d] = acc[d];
  __syncthreads();
  float bm = kNegBig;
#pragma unroll
  for (int w = 0; w < kAttWarps; ++w) bm = fmaxf(bm, sm_m[w]);
  float bl = 0.f, bo = 0.f;
  const int d = threadIdx.x;  // thread d owns channel d from here on
#pragma unroll
  for (int w = 0; w < kAttWarps; ++w) {
    const float f = __expf(sm_m[w] - bm);
    bl += f * sm_l[w];
    bo += f * sm_o[w][d];
  }
  if (n_parts == 1) {
    out[d] = Elem<T>::from_f(bl > 0.f ? bo / bl : 0.f);
    return;
  }
  // publish this block's partial, then take a ticket
  const size_t slot = (size_t)row * p.max_chunks + c;
  p.part_o[slot * kD + d] = bo;
  if (d == 0) {
    p.part_ml[slot * 2] = bm;
    p.part_ml[slot * 2 + 1] = bl;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) sm_ticket = atomicAdd(&p.counters[row], 1);
  __syncthreads();
  if (sm_ticket != n_parts - 1) return;
  __threadfence();
  float gm = kNegBig;
  for (int cc = 0; cc < n_parts; ++cc)
    gm = fmaxf(gm, __ldcg(&p.part_ml[((size_t)row * p.max_chunks + cc) * 2]));
  float gl = 0.f, go = 0.f;
  for (int cc = 0; cc < n_parts; ++cc) {
    const size_t s2 = (size_t)row * p.max_chunks + cc;
    const float f = __expf(__ldcg(&p.part_ml[s2 * 2]) - gm);
    gl += f * __ldcg(&p.part_ml[s2 * 2 + 1]);
    go += f * __ldcg(&p.part_o[s2 * kD + d]);
  }
  out[d] = Elem<T>::from_f(gl > 0.f ? go / gl : 0.f);
  if (threadIdx.x == 0) p.counters[row] = 0;  // leave the workspace ready for the next call
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace twl

extern "C" size_t twl_sparse_attn_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                                  int32_t index_stride, int32_t chunk) {
  if (batch <= 0 || num_q_heads <= 0 || index_stride <= 0 || chunk <= 0) return 0;
  const size_t rows = (size_t)batch * num_q_heads;
  const size_t max_chunks =
      std::min<size_t>(((size_t)index_stride + chunk - 1) / chunk, twl::kMaxSplits);
  size_t bytes = twl::align_up(rows * sizeof(int32_t), 256);
  bytes += twl::align_up(rows * max_chunks * 2 * sizeof(float), 256);
  bytes += rows * max_chunks * twl::kD * sizeof(float);
  return bytes;
}

extern "C" int twl_sparse_decode_attn(const void* q, int dtype, const void* k_pages,
                                      const void* v_pages, const int32_t* kv_indptr,
                                      const int32_t* kv_indices, const int32_t* indices,
                                      int32_t index_stride, const int32_t* budget, int32_t batch,
                                      int32_t num_q_heads, int32_t num_kv_heads,
                                      int32_t num_pages_total, float sm_scale, void* out,
                                      void* workspace, size_t workspace_bytes, int32_t chunk,
                                      int32_t* status, void* stream) {
  using namespace twl;
  if (!q || !k_pages || !v_pages || !kv_indptr || !kv_indices || !indices || !budget || !out)
    return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || index_stride <= 0 ||
      num_pages_total <= 0 || num_q_heads % num_kv_heads != 0)
    return TWL_ERR_BAD_ARG;
  if (chunk <= 0) chunk = 256;
  if (chunk % 32 != 0) return TWL_ERR_BAD_ARG;
  if (!aligned(q, 8) || !aligned(k_pages, 16) || !aligned(v_pages, 16) || !aligned(out, 2))
    return TWL_ERR_MISALIGNED;
  const size_t need = twl_sparse_attn_workspace_bytes(batch, num_q_heads, index_stride, chunk);
  if (!workspace || workspace_bytes < need) return TWL_ERR_WORKSPACE;
  if (!aligned(workspace, 16)) return TWL_ERR_MISALIGNED;
  const size_t rows = (size_t)batch * num_q_heads;
  if (rows > 65535) return TWL_ERR_TOO_LARGE;
  const size_t max_chunks = std::min<size_t>(((size_t)index_stride + chunk - 1) / chunk, kMaxSplits);
  AttParams p;
  p.q = q; p.k = k_pages; p.v = v_pages; p.indptr = kv_indptr; p.indices = kv_indices;
  p.idx = indices; p.budget = budget; p.out = out; p.status = status;
  char* ws = static_cast<char*>(workspace);
  p.counters = reinterpret_cast<int32_t*>(ws);
  ws += align_up(rows * sizeof(int32_t), 256);
  p.part_ml = reinterpret_cast<float*>(ws);
  ws += align_up(rows * max_chunks * 2 * sizeof(float), 256);
  p.part_o = reinterpret_cast<float*>(ws);
  p.index_stride = index_stride; p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads;
  p.num_pages_total = num_pages_total; p.chunk = chunk; p.max_chunks = (int)max_chunks;
  p.sm_scale = sm_scale;
  dim3 grid((unsigned)max_chunks, (unsigned)rows);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) {
    sparse_decode_attn_kernel<__half><<<grid, kAttThreads, 0, st>>>(p);
  } else if (dtype == TWL_BF16) {
    sparse_decode_attn_kernel<__nv_bfloat16><<<grid, kAttThreads, 0, st>>>(p);
  } else {
    return TWL_ERR_UNSUPPORTED;
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}
