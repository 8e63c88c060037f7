// Kernel #1: INT4 K-cache q.k estimator (paged GEMV, group-32 scale/min).
//
// Stands in for the estimator of twilight/pyimpl/attention.py:247-255 (the reference
// fake-quantises K with quantize.py:4-13 on every step; here K is quantised once when it
// is appended and only the 4-bit codes are read).
//
// Work split: one block = one row (a query head, or a KV head with its whole query-head
// group when every page is a candidate) x a run of kPagesPerBlock candidate pages.
// A lane owns one (token, 32-channel group): a warp step reads 8 tokens = 512 contiguous
// code bytes with one 128-bit load per lane plus 128 bytes of {scale,min}; the four lanes
// of a token are combined with two shuffles.  q lives in registers, already converted to
// the form the arithmetic variant wants; sum_d q_d*(c_d*s+m) = s*sum(q_d c_d) + m*sum(q_d)
// so the inner loop touches only codes.
#include "common.cuh"

namespace twl {

constexpr int kEstThreads = 256;
constexpr int kEstWarps = kEstThreads / 32;
constexpr int kPagesPerBlock = 32;  // 512 tokens, 40 KiB of INT4 cache per block
constexpr int kUnroll = 4;

enum { VAR_F32 = 1, VAR_H2 = 2, VAR_DP4A = 3 };

struct EstParams {
  const void* q;
  const uint8_t* k4;
  const int32_t* indptr;
  const int32_t* indices;
  const int32_t* last_len;
  const int32_t* cand_pages;
  const int32_t* cand_npages;
  float* scores;
  int32_t* status;
  int max_k, B, Hq, Hkv, num_pages_total, stride;
  float sm_scale;
};

// ---- per-variant query registers for one head and one 32-channel group --------------------
template <int VARIANT>
struct QRegs;

template <>
struct QRegs<VAR_F32> {
  float q[32];
  float qsum;
  __device__ __forceinline__ void init(const float* qf) {
    qsum = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      q[i] = qf[i];
      qsum += qf[i];
    }
  }
  // sum_d q_d * code_d over the lane's 32 channels
  __device__ __forceinline__ float dot(const uint4& w) const {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int n = 0; n < 8; n += 2) {
        // 2^23 + code is exact in fp32; subtracting 2^23 leaves the code
        float c0 = __uint_as_float(0x4B000000u | ((ws[j] >> (4 * n)) & 0xFu)) - 8388608.f;
        float c1 = __uint_as_float(0x4B000000u | ((ws[j] >> (4 * n + 4)) & 0xFu)) - 8388608.f;
        acc0 = fmaf(q[8 * j + n], c0, acc0);
        acc1 = fmaf(q[8 * j + n + 1], c1, acc1);
      }
    }
    return acc0 + acc1;
  }
};

template <>
struct QRegs<VAR_H2> {
  // pair k of word j = channels (8j+k, 8j+k+4): the two nibbles (w >> 4k) & 0x000F000F
  __half2 q[16];
  float qsum;
  __device__ __forceinline__ void init(const float* qf) {
    qsum = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) qsum += qf[i];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k)
        q[4 * j + k] = __floats2half2_rn(qf[8 * j + k], qf[8 * j + k + 4]);
  }
  __device__ __forceinline__ float dot(const uint4& w) const {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    const __half2 b1024 = __half2half2(__ushort_as_half(0x6400));  // 1024
    const __half2 b64 = __half2half2(__ushort_as_half(0x5400));    // 64
    float total = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t x = ws[j];
      const uint32_t y = x >> 8;
      // nibble in mantissa bits 0..3 of 0x6400 -> 1024 + c ; bits 4..7 of 0x5400 -> 64 + c
      uint32_t u0 = (x & 0x000F000Fu) | 0x64006400u;
      uint32_t u1 = (x & 0x00F000F0u) | 0x54005400u;
      uint32_t u2 = (y & 0x000F000Fu) | 0x64006400u;
      uint32_t u3 = (y & 0x00F000F0u) | 0x54005400u;
      __half2 c0 = __hsub2(*reinterpret_cast<__half2*>(&u0), b1024);
      __half2 c1 = __hsub2(*reinterpret_cast<__half2*>(&u1), b64);
      __half2 c2 = __hsub2(*reinterpret_cast<__half2*>(&u2), b1024);
      __half2 c3 = __hsub2(*reinterpret_cast<__half2*>(&u3), b64);
      __half2 acc = __hmul2(q[4 * j + 0], c0);
      acc = __hfma2(q[4 * j + 1], c1, acc);
      acc = __hfma2(q[4 * j + 2], c2, acc);
      acc = __hfma2(q[4 * j + 3], c3, acc);
      float2 f = __half22float2(acc);
      total += f.x + f.y;
    }
    return total;
  }
};

template <>
struct QRegs<VAR_DP4A> {
  // q_d ~= (256*qh_d + ql_d) * inv, qh signed byte, ql unsigned byte
  uint32_t qh_even[4], qh_odd[4], ql_even[4], ql_odd[4];
  float inv, qsum;
  __device__ __forceinline__ void init(const float* qf) {
    qsum = 0.f;
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      qsum += qf[i];
      amax = fmaxf(amax, fabsf(qf[i]));
    }
    int e = (amax > 0.f) ? (14 - ilogbf(amax)) : 0;  // amax * 2^e in [2^14, 2^15)
    e = max(-60, min(60, e));
    const float f = ldexpf(1.f, e);
    inv = ldexpf(1.f, -e);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t he = 0, ho = 0, le = 0, lo = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int a = __float2int_rn(qf[8 * j + 2 * i] * f);
        int b = __float2int_rn(qf[8 * j + 2 * i + 1] * f);
        he |= (uint32_t)((a >> 8) & 0xFF) << (8 * i);
        le |= (uint32_t)(a & 0xFF) << (8 * i);
        ho |= (uint32_t)((b >> 8) & 0xFF) << (8 * i);
        lo |= (uint32_t)(b & 0xFF) << (8 * i);
      }
      qh_even[j] = he;
      qh_odd[j] = ho;
      ql_even[j] = le;
      ql_odd[j] = lo;
    }
  }
  __device__ __forceinline__ float dot(const uint4& w) const {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    int acc_h = 0;
    unsigned acc_l = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t even = ws[j] & 0x0F0F0F0Fu;         // channels 8j+0,2,4,6
      const uint32_t odd = (ws[j] >> 4) & 0x0F0F0F0Fu;   // channels 8j+1,3,5,7
      acc_h = __dp4a((int)even, (int)qh_even[j], acc_h);
      acc_h = __dp4a((int)odd, (int)qh_odd[j], acc_h);
      acc_l = __dp4a(even, ql_even[j], acc_l);
      acc_l = __dp4a(odd, ql_odd[j], acc_l);
    }
    return (float)(acc_h * 256 + (int)acc_l) * inv;
  }
};

template <typename T>
__device__ __forceinline__ void load_q_group(const T* q, float* qf) {
  // 32 elements = 64 bytes = four 128-bit loads
  const uint4* p = reinterpret_cast<const uint4*>(q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v = __ldg(p + i);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = Elem<T>::to_f2(u[k]);
      qf[8 * i + 2 * k] = f.x;
      qf[8 * i + 2 * k + 1] = f.y;
    }
  }
}

// G = query heads that share the block's pages (1 when a candidate list is given).
template <typename T, int G, int VARIANT>
__global__ void __launch_bounds__(kEstThreads)
estimate_int4_kernel(const EstParams p) {
  const int row = blockIdx.y;
  const bool has_cand = p.cand_pages != nullptr;
  int b, kvh, h0;
  if (has_cand) {  // row = (b, query head); G == 1
    b = row / p.Hq;
    h0 = row % p.Hq;
    kvh = h0 / (p.Hq / p.Hkv);
  } else {  // row = (b, kv head); heads h0 .. h0+G-1
    b = row / p.Hkv;
    kvh = row % p.Hkv;
    h0 = kvh * G;
  }
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = has_cand ? min(p.cand_npages[b * p.Hq + h0], p.max_k) : n_seq_pages;
  if (n_pages > p.stride / kPage) {  // never write past the score row
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * kPagesPerBlock;
  if (first >= n_pages) return;
  const int n_here = min(kPagesPerBlock, n_pages - first);
  const int last_len = p.last_len[b];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane & 3, tok_in_step = lane >> 2;

  QRegs<VARIANT> qr[G];
  {
    float qf[32];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h0 + g)) * kD + grp * kGroup, qf);
      qr[g].init(qf);
    }
  }

  const int32_t* cand = has_cand ? p.cand_pages + (size_t)(b * p.Hq + h0) * p.max_k : nullptr;
  const int n_steps = n_here * 2;  // half a page per warp step
  for (int s0 = warp; s0 < n_steps; s0 += kEstWarps * kUnroll) {
    uint4 w[kUnroll];
    uint32_t sz[kUnroll];
    int slot[kUnroll];
    bool live[kUnroll], valid[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int s = s0 + u * kEstWarps;
      live[u] = s < n_steps;
      valid[u] = false;
      w[u] = make_uint4(0, 0, 0, 0);
      sz[u] = 0;
      slot[u] = 0;
      if (live[u]) {
        const int lp = first + (s >> 1);
        const int half = s & 1;
        const int seq_page = has_cand ? cand[lp] : lp;
        slot[u] = lp * kPage + half * 8 + tok_in_step;
        bool ok = seq_page >= 0 && seq_page < n_seq_pages;
        int phys = 0;
        if (ok) {
          phys = p.indices[page_base + seq_page];
          ok = phys >= 0 && phys < p.num_pages_total;
        }
        if (!ok) {
          raise_flag(p.status, TWL_FLAG_BAD_INDEX);
        } else {
          const int t = half * 8 + tok_in_step;
          valid[u] = (seq_page != n_seq_pages - 1) || (t < last_len);
          const uint8_t* slab = p.k4 + ((size_t)phys * p.Hkv + kvh) * kSlab;
          w[u] = ldg_stream_u4(slab + half * 512 + lane * 16);
          sz[u] = ldg_stream_u32(slab + kSlabCodes + half * 128 + lane * 4);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (!live[u]) continue;  // warp-uniform
      const float2 szf = __half22float2(*reinterpret_cast<const __half2*>(&sz[u]));
      float part[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        part[g] = fmaf(szf.x, qr[g].dot(w[u]), szf.y * qr[g].qsum);
        part[g] += __shfl_xor_sync(0xffffffffu, part[g], 1);
        part[g] += __shfl_xor_sync(0xffffffffu, part[g], 2);
      }
      // the four lanes of a token share the G results; lane `grp` stores heads grp, grp+4, ..
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if ((g & 3) == grp) {
          const float v = valid[u] ? part[g] * p.sm_scale : -INFINITY;
          p.scores[(size_t)(b * p.Hq + h0 + g) * p.stride + slot[u]] = v;
        }
      }
    }
  }
}

template <typename T, int G, int VARIANT>
static int launch_one(const EstParams& p, int rows, int max_row_pages, cudaStream_t st) {
  if (rows > 65535) return TWL_ERR_TOO_LARGE;
  dim3 grid((max_row_pages + kPagesPerBlock - 1) / kPagesPerBlock, rows);
  estimate_int4_kernel<T, G, VARIANT><<<grid, kEstThreads, 0, st>>>(p);
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

template <typename T, int VARIANT>
static int launch_variant(const EstParams& p, bool has_cand, int max_row_pages, cudaStream_t st) {
  if (has_cand) return launch_one<T, 1, VARIANT>(p, p.B * p.Hq, max_row_pages, st);
  const int g = p.Hq / p.Hkv;
  switch (g) {
    case 1: return launch_one<T, 1, VARIANT>(p, p.B * p.Hkv, max_row_pages, st);
    case 2: return launch_one<T, 2, VARIANT>(p, p.B * p.Hkv, max_row_pages, st);
    case 4: return launch_one<T, 4, VARIANT>(p, p.B * p.Hkv, max_row_pages, st);
    case 8: return launch_one<T, 8, VARIANT>(p, p.B * p.Hkv, max_row_pages, st);
    default: return TWL_ERR_UNSUPPORTED;
  }
}

template <typename T>
static int launch_dtype(const EstParams& p, bool has_cand, int max_row_pages, int variant,
                        cudaStream_t st) {
  switch (variant) {
    case VAR_F32: return launch_variant<T, VAR_F32>(p, has_cand, max_row_pages, st);
    case VAR_H2: return launch_variant<T, VAR_H2>(p, has_cand, max_row_pages, st);
    case 0:
    case VAR_DP4A: return launch_variant<T, VAR_DP4A>(p, has_cand, max_row_pages, st);
    default: return TWL_ERR_BAD_ARG;
  }
}

}  // namespace twl

extern "C" int twl_estimate_int4(const void* q, int dtype, const uint8_t* k4_pages,
                                 const int32_t* kv_indptr, const int32_t* kv_indices,
                                 const int32_t* kv_last_page_len, const int32_t* cand_pages,
                                 const int32_t* cand_npages, int32_t max_k, int32_t batch,
                                 int32_t num_q_heads, int32_t num_kv_heads,
                                 int32_t num_pages_total, float sm_scale, float* scores,
                                 int32_t score_stride, int32_t variant, int32_t* status,
                                 void* stream) {
  using namespace twl;
  if (!q || !k4_pages || !kv_indptr || !kv_indices || !kv_last_page_len || !scores)
    return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_pages_total <= 0 ||
      score_stride <= 0 || num_q_heads % num_kv_heads != 0)
    return TWL_ERR_BAD_ARG;
  const bool has_cand = cand_pages != nullptr;
  if (has_cand && (!cand_npages || max_k <= 0)) return TWL_ERR_BAD_ARG;
  if (score_stride % kPage != 0) return TWL_ERR_BAD_ARG;
  if (has_cand && (int64_t)max_k * kPage > score_stride) return TWL_ERR_TOO_LARGE;
  if (!aligned(q, 16) || !aligned(k4_pages, 16) || !aligned(scores, 4)) return TWL_ERR_MISALIGNED;
  EstParams p;
  p.q = q; p.k4 = k4_pages; p.indptr = kv_indptr; p.indices = kv_indices;
  p.last_len = kv_last_page_len; p.cand_pages = cand_pages; p.cand_npages = cand_npages;
  p.scores = scores; p.status = status; p.max_k = max_k; p.B = batch; p.Hq = num_q_heads;
  p.Hkv = num_kv_heads; p.num_pages_total = num_pages_total; p.stride = score_stride;
  p.sm_scale = sm_scale;
  // rows never hold more pages than the score row has room for
  const int max_row_pages = has_cand ? max_k : score_stride / kPage;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) return launch_dtype<__half>(p, has_cand, max_row_pages, variant, st);
  if (dtype == TWL_BF16) return launch_dtype<__nv_bfloat16>(p, has_cand, max_row_pages, variant, st);
  return TWL_ERR_UNSUPPORTED;
}
