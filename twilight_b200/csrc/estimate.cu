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
#include <cstdlib>

#include <cstddef>

#include "common.cuh"

namespace twl {

constexpr int kEstThreads = 256;
constexpr int kEstWarps = kEstThreads / 32;
constexpr int kPagesPerBlock = 64;  // 1024 tokens, 80 KiB of INT4 cache per block
constexpr int kUnroll = 8;

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
  int max_k, B, Hq, Hkv, num_pages_total, stride, pages_per_block, force_ring, simt_group, bulk_warp, f16_tiles, two_tiles;
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

__device__ __forceinline__ int dp4a_u8_s8(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t dp4a_u8_u8(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <>
struct __align__(16) QRegs<VAR_DP4A> {
  // q_d ~= (256*qh_d + ql_d) * inv with |256*qh+ql| < 2^13, qh a signed byte, ql an unsigned
  // byte.  Even channels sit in the low nibbles, odd channels in the high nibbles; the odd ones
  // are used unshifted (16*code), which the final >>4 undoes exactly.
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
    int e = (amax > 0.f) ? (12 - ilogbf(amax)) : 0;  // amax * 2^e in [2^12, 2^13)
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
  // integer sum_d code_d * q_int_d  (|result| < 2^22)
  __device__ __forceinline__ int idot(const uint4& w) const {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    int he = 0, ho = 0;
    uint32_t le = 0, lo = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t even = ws[j] & 0x0F0F0F0Fu;    // channels 8j+0,2,4,6
      const uint32_t odd16 = ws[j] & 0xF0F0F0F0u;   // 16 * channels 8j+1,3,5,7
      he = dp4a_u8_s8(even, qh_even[j], he);
      ho = dp4a_u8_s8(odd16, qh_odd[j], ho);
      le = dp4a_u8_u8(even, ql_even[j], le);
      lo = dp4a_u8_u8(odd16, ql_odd[j], lo);
    }
    return (he + (ho >> 4)) * 256 + (int)(le + (lo >> 4));
  }
  __device__ __forceinline__ float dot(const uint4& w) const {
    // exact int -> float for |x| < 2^22 without the conversion unit
    return (__int_as_float(0x4B400000 + idot(w)) - 12582912.f) * inv;
  }
};
static_assert(sizeof(QRegs<VAR_DP4A>) == 80 && offsetof(QRegs<VAR_DP4A>, inv) == 64 &&
                  offsetof(QRegs<VAR_DP4A>, qsum) == 68,
              "the group kernel reads this structure from shared memory as four uint4 and one float2");

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
//
// Prologue: one thread per page resolves candidate slot -> sequence page -> physical page and
// parks it in shared memory, so the streaming loop has no dependent index loads; 4*G threads
// convert q once (one per head and 32-channel group) and every thread copies the registers of
// its group from shared memory.
template <typename T, int G, int VARIANT>
__global__ void __launch_bounds__(kEstThreads)
estimate_int4_kernel(const EstParams p) {
  __shared__ int sm_phys[kPagesPerBlock];   // physical page id, -1 = skip
  __shared__ int sm_ntok[kPagesPerBlock];   // valid tokens of the page
  __shared__ QRegs<VARIANT> sm_q[G][4];

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

  const int tid = threadIdx.x;
  if (tid < n_here) {
    const int32_t* cand = has_cand ? p.cand_pages + (size_t)(b * p.Hq + h0) * p.max_k : nullptr;
    const int seq_page = has_cand ? cand[first + tid] : first + tid;
    int phys = -1;
    if (seq_page >= 0 && seq_page < n_seq_pages) {
      phys = p.indices[page_base + seq_page];
      if (phys < 0 || phys >= p.num_pages_total) phys = -1;
    }
    if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
    sm_phys[tid] = phys;
    sm_ntok[tid] = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
  } else if (tid >= kEstThreads - 4 * G) {
    const int j = tid - (kEstThreads - 4 * G);
    const int g = j >> 2, grp_j = j & 3;
    float qf[32];
    load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h0 + g)) * kD + grp_j * kGroup, qf);
    sm_q[g][grp_j].init(qf);
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  const int grp = lane & 3, tok_in_step = lane >> 2;
  QRegs<VARIANT> qr[G];
#pragma unroll
  for (int g = 0; g < G; ++g) qr[g] = sm_q[g][grp];

  const int n_steps = n_here * 2;  // half a page per warp step
  for (int s0 = warp; s0 < n_steps; s0 += kEstWarps * kUnroll) {
    uint4 w[kUnroll];
    uint32_t sz[kUnroll];
    bool valid[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int s = s0 + u * kEstWarps;
      valid[u] = false;
      w[u] = make_uint4(0, 0, 0, 0);
      sz[u] = 0;
      if (s < n_steps) {
        const int pg = s >> 1, half = s & 1;
        const int phys = sm_phys[pg];
        if (phys >= 0) {
          valid[u] = (half * 8 + tok_in_step) < sm_ntok[pg];
          const uint8_t* slab = p.k4 + ((size_t)phys * p.Hkv + kvh) * kSlab;
          w[u] = ldg_stream_u4(slab + half * 512 + lane * 16);
          sz[u] = ldg_stream_u32(slab + kSlabCodes + half * 128 + lane * 4);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int s = s0 + u * kEstWarps;
      if (s >= n_steps) break;  // warp-uniform
      const int slot = (first + (s >> 1)) * kPage + (s & 1) * 8 + tok_in_step;
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
          p.scores[(size_t)(b * p.Hq + h0 + g) * p.stride + slot] = v;
        }
      }
    }
  }
}

// ---- bulk-async-copy (TMA) staged variant -------------------------------------------------------
// One extra warp is the producer: its first lane issues one cp.async.bulk of 1280 bytes per page
// (a whole (page, kv-head) slab is contiguous and 16-byte aligned) into a ring of shared-memory
// stages, each guarded by a "full" mbarrier (transaction bytes) and an "empty" mbarrier (one
// arrival per consumer warp).  Bytes in flight are set by the ring (kStages * kStagePages *
// 1280 B per block), not by registers.  Every wait is bounded: when it runs out the block raises
// TWL_FLAG_WAIT_LIMIT, stops consuming, drains the copies it still has in flight (bounded again)
// and returns.
constexpr int kStagePages = 8;                       // 10 KiB per stage
constexpr int kStages = 4;                           // 40 KiB ring per block
constexpr int kTmaMaxPagesPerBlock = 512;            // capacity of the per-block page list
constexpr int kTmaPagesPerBlockDefault = 128;        // 160 KiB of INT4 cache per block
constexpr int kTmaThreads = kEstThreads + 32;        // 8 consumer warps + 1 producer warp
constexpr uint32_t kWaitLimit = 1u << 16;  // about a second of bounded waiting, then the error flag
constexpr uint32_t kSuspendHintNs = 20000;  // a waiting thread may sleep this long per try

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait for the phase with the given parity to complete; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

template <typename T, int G, int VARIANT>
__global__ void __launch_bounds__(kTmaThreads)
estimate_int4_tma_kernel(const EstParams p) {
  extern __shared__ __align__(128) uint8_t sm_ring[];  // kStages * kStagePages * kSlab bytes
  __shared__ __align__(8) uint64_t sm_full[kStages];
  __shared__ __align__(8) uint64_t sm_empty[kStages];
  __shared__ int sm_phys[kTmaMaxPagesPerBlock];
  __shared__ int sm_ntok[kTmaMaxPagesPerBlock];
  __shared__ QRegs<VARIANT> sm_q[G][4];

  const int row = blockIdx.y;
  const bool has_cand = p.cand_pages != nullptr;
  int b, kvh, h0;
  if (has_cand) {
    b = row / p.Hq;
    h0 = row % p.Hq;
    kvh = h0 / (p.Hq / p.Hkv);
  } else {
    b = row / p.Hkv;
    kvh = row % p.Hkv;
    h0 = kvh * G;
  }
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = has_cand ? min(p.cand_npages[b * p.Hq + h0], p.max_k) : n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * p.pages_per_block;
  if (first >= n_pages) return;
  const int n_here = min(p.pages_per_block, n_pages - first);
  const int n_stages_total = (n_here + kStagePages - 1) / kStagePages;

  const int tid = threadIdx.x;
  if (tid >= kEstThreads - 4 * G && tid < kEstThreads) {
    const int j = tid - (kEstThreads - 4 * G);
    const int g = j >> 2, grp_j = j & 3;
    float qf[32];
    load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h0 + g)) * kD + grp_j * kGroup, qf);
    sm_q[g][grp_j].init(qf);
  } else {
    const int32_t* cand = has_cand ? p.cand_pages + (size_t)(b * p.Hq + h0) * p.max_k : nullptr;
    for (int i = tid; i < n_here; i += kEstThreads - 4 * G) {
      const int seq_page = has_cand ? cand[first + i] : first + i;
      int phys = -1;
      if (seq_page >= 0 && seq_page < n_seq_pages) {
        phys = p.indices[page_base + seq_page];
        if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      }
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      sm_phys[i] = phys;
      sm_ntok[i] = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
  }
  if (tid == kEstThreads) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm_full[s], 1);
      mbar_init(&sm_empty[s], kEstWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  if (warp == kEstWarps) {
    // ---- producer ----
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int st = 0; st < n_stages_total && ok; ++st) {
        const int slot = st % kStages;
        if (st >= kStages) ok = mbar_wait(&sm_empty[slot], ((st / kStages) - 1) & 1);
        if (!ok) break;
        const int pg0 = st * kStagePages, pg1 = min(n_here, pg0 + kStagePages);
        uint32_t bytes = 0;
        for (int pg = pg0; pg < pg1; ++pg) bytes += sm_phys[pg] >= 0 ? kSlab : 0;
        mbar_arrive_expect_tx(&sm_full[slot], bytes);
        for (int pg = pg0; pg < pg1; ++pg) {
          const int phys = sm_phys[pg];
          if (phys >= 0)
            bulk_copy_g2s(sm_ring + ((size_t)slot * kStagePages + (pg - pg0)) * kSlab,
                          p.k4 + ((size_t)phys * p.Hkv + kvh) * kSlab, kSlab, &sm_full[slot]);
        }
        issued = st + 1;
      }
      if (!ok) raise_flag(p.status, TWL_FLAG_WAIT_LIMIT);
      // Drain on every path: the copies of the last stages may still be writing into this block's
      // shared memory, and a consumer whose own bounded wait ran out has returned without them.
      // The block must not end before they have landed (bounded waits again).
      for (int st = max(0, issued - kStages); st < issued; ++st)
        mbar_wait(&sm_full[st % kStages], (st / kStages) & 1);
    }
    return;
  }

  // ---- consumers ----
  const int grp = lane & 3, tok_in_step = lane >> 2;
  QRegs<VARIANT> qr[G];
#pragma unroll
  for (int g = 0; g < G; ++g) qr[g] = sm_q[g][grp];

  float* const out_rows = p.scores + (size_t)(b * p.Hq + h0) * p.stride + (size_t)first * kPage + tok_in_step;
  for (int st = 0; st < n_stages_total; ++st) {
    const int slot = st % kStages;
    if (!mbar_wait(&sm_full[slot], (st / kStages) & 1)) {
      if (lane == 0) raise_flag(p.status, TWL_FLAG_WAIT_LIMIT);
      return;  // the producer drains what it issued
    }
    const int pg0 = st * kStagePages;
    const int n_steps = (min(n_here, pg0 + kStagePages) - pg0) * 2;
    const uint8_t* stage = sm_ring + (size_t)slot * kStagePages * kSlab;
    for (int s = warp; s < n_steps; s += kEstWarps) {
      const int pgl = s >> 1, half = s & 1;
      const int pg = pg0 + pgl;
      const bool present = sm_phys[pg] >= 0;
      const bool valid = present && (half * 8 + tok_in_step) < sm_ntok[pg];
      uint4 w = make_uint4(0, 0, 0, 0);
      uint32_t sz = 0;
      if (present) {
        const uint8_t* slab = stage + pgl * kSlab;
        w = *reinterpret_cast<const uint4*>(slab + half * 512 + lane * 16);
        sz = *reinterpret_cast<const uint32_t*>(slab + kSlabCodes + half * 128 + lane * 4);
      }
      const int slot_out = pg * kPage + half * 8;
      const float2 szf = __half22float2(*reinterpret_cast<const __half2*>(&sz));
      float part[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        part[g] = fmaf(szf.x, qr[g].dot(w), szf.y * qr[g].qsum);
        part[g] += __shfl_xor_sync(0xffffffffu, part[g], 1);
        part[g] += __shfl_xor_sync(0xffffffffu, part[g], 2);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if ((g & 3) == grp) {
          const float v = valid ? part[g] * p.sm_scale : -INFINITY;
          out_rows[(size_t)g * p.stride + slot_out] = v;
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm_empty[slot]);
  }
}

// ---- warp-private cp.async ring, one lane per token (single query head per row) ------------------
// Every warp streams its own page pairs (32 tokens = 2560 bytes) through a private ring in shared
// memory with 16-byte cp.async copies, so there is no block-level barrier and no register staging:
// bytes in flight are kRingDepth-1 stages per warp.  Inside a stage lane t owns token t and all four
// 32-channel groups, so no shuffle is needed and the 32 scores go out as one 128-byte store.  A
// token's four 16-byte code chunks are stored rotated by (t>>1) so that the 8 lanes of a quarter
// warp hit 8 different bank groups when all of them read "their chunk j".
constexpr int kRingDepth = 5;
constexpr int kWarpStageBytes = 2 * kSlab;   // two pages
constexpr int kWarpPagesPerBlock = 128;

template <typename T, int VARIANT, int NW, int DEPTH, int PPB>
__global__ void __launch_bounds__(NW * 32, (220 * 1024) / (NW * DEPTH * kWarpStageBytes + 2048))
estimate_int4_warp_kernel(const EstParams p) {
  extern __shared__ __align__(128) uint8_t sm_ring[];  // NW * DEPTH * kWarpStageBytes
  __shared__ int sm_phys[PPB];
  __shared__ int sm_ntok[PPB];
  __shared__ QRegs<VARIANT> sm_q[4];

  const int row = blockIdx.y;
  const bool has_cand = p.cand_pages != nullptr;
  int b, kvh, h;
  if (has_cand) {
    b = row / p.Hq;
    h = row % p.Hq;
    kvh = h / (p.Hq / p.Hkv);
  } else {  // one query head per KV head
    b = row / p.Hkv;
    kvh = row % p.Hkv;
    h = kvh;
  }
  pdl_wait();  // candidate lists (and maybe q, the page table) come from the kernel before; nothing is read earlier
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = has_cand ? min(p.cand_npages[b * p.Hq + h], p.max_k) : n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * PPB;
  if (first >= n_pages) return;
  const int n_here = min(PPB, n_pages - first);

  const int tid = threadIdx.x;
  // four threads fetch q now and convert it later, after the first copies are on their way
  const bool q_thread = tid >= (NW * 32) - 4;
  float qf[32];
  if (q_thread)
    load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h)) * kD +
                        (tid - ((NW * 32) - 4)) * kGroup, qf);
  if (tid < PPB) {
    int phys = -1, ntok = 0;
    if (tid < n_here) {
      const int seq_page = has_cand ? p.cand_pages[(size_t)(b * p.Hq + h) * p.max_k + first + tid] : first + tid;
      if (seq_page >= 0 && seq_page < n_seq_pages) {
        phys = p.indices[page_base + seq_page];
        if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      }
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      ntok = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
    sm_phys[tid] = phys;
    sm_ntok[tid] = phys < 0 ? 0 : ntok;
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  uint8_t* const ring = sm_ring + (size_t)warp * DEPTH * kWarpStageBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const int n_pairs = (n_here + 1) >> 1;
  const int my_pairs = (n_pairs > warp) ? (n_pairs - warp + NW - 1) / NW : 0;

  // Per-lane constants of the five 16-byte copies of a stage: chunk c = c5*32+lane of the pair,
  // i.e. page c/80 and chunk r = c%80 of its slab (0..63 codes, 64..79 scale/min).
  uint32_t src16[5], dst_off[5];
  bool second[5];
#pragma unroll
  for (int c5 = 0; c5 < 5; ++c5) {
    const int c = c5 * 32 + lane;
    const int pgl = c >= 80 ? 1 : 0;
    const int r = c - pgl * 80;
    second[c5] = pgl != 0;
    src16[c5] = r;
    if (r < 64) {
      const int t = pgl * 16 + (r >> 2), g = r & 3;
      dst_off[c5] = t * 64 + (((g + (t >> 1)) & 3) << 4);
    } else {
      dst_off[c5] = 2048 + (pgl * 16 + (r - 64)) * 16;
    }
  }
  const uint4* const k4_head16 = reinterpret_cast<const uint4*>(p.k4 + (size_t)kvh * kSlab);
  const uint32_t page_stride16 = (uint32_t)(p.Hkv * (kSlab / 16));

  // issue the copies of this warp's i-th pair into the given ring slot
  auto issue = [&](int i, int slot) {
    if (i < my_pairs) {
      const int pg0 = (warp + i * NW) * 2;
      const uint32_t dst0 = ring_u32 + slot * kWarpStageBytes;
      const int phys0 = sm_phys[pg0], phys1 = sm_phys[pg0 + 1];  // missing pages hold -1
#pragma unroll
      for (int c5 = 0; c5 < 5; ++c5) {
        const int phys = second[c5] ? phys1 : phys0;
        if (phys >= 0)
          cp_async16(dst0 + dst_off[c5], k4_head16 + ((size_t)phys * page_stride16 + src16[c5]));
      }
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };

#pragma unroll
  for (int i = 0; i < DEPTH - 1; ++i) issue(i, i);

  if (q_thread) sm_q[tid - ((NW * 32) - 4)].init(qf);
  __syncthreads();
  QRegs<VARIANT> qr[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) qr[g] = sm_q[g];

  uint32_t rd_off[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) rd_off[g] = lane * 64 + (((g + (lane >> 1)) & 3) << 4);
  float* const out_row = p.scores + (size_t)(b * p.Hq + h) * p.stride + (size_t)first * kPage;
  int use_slot = 0, fill_slot = DEPTH - 1;
  for (int i = 0; i < my_pairs; ++i) {
    cp_async_wait<DEPTH - 2>();  // pair i has landed (this thread's copies)
    __syncwarp();                     // ... and every other lane's
    const int pg0 = (warp + i * NW) * 2;
    const uint8_t* stage = ring + use_slot * kWarpStageBytes;
    const int pgl = lane >> 4, tl = lane & 15;
    const int ntok = sm_ntok[pg0 + pgl];
    const bool present = sm_phys[pg0 + pgl] >= 0;
    const uint4 sz = *reinterpret_cast<const uint4*>(stage + 2048 + lane * 16);
    const uint32_t szw[4] = {sz.x, sz.y, sz.z, sz.w};
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 w = *reinterpret_cast<const uint4*>(stage + rd_off[g]);
      const float2 szf = __half22float2(*reinterpret_cast<const __half2*>(&szw[g]));
      acc = fmaf(szf.x, qr[g].dot(w), acc);
      acc = fmaf(szf.y, qr[g].qsum, acc);
    }
    __syncwarp();      // all lanes are done reading the slot that the next issue overwrites
    issue(i + DEPTH - 1, fill_slot);
    use_slot = (use_slot + 1 == DEPTH) ? 0 : use_slot + 1;
    fill_slot = (fill_slot + 1 == DEPTH) ? 0 : fill_slot + 1;
    // a page whose table entry was out of range scores -inf in all sixteen slots (ntok is 0 there)
    if (pg0 + pgl < n_here) out_row[(pg0 + pgl) * kPage + tl] = (present && tl < ntok) ? acc * p.sm_scale : -INFINITY;
  }
  cp_async_wait<0>();
}

// ---- warp-private rings fed by bulk asynchronous copies (TMA) -------------------------------------
// The scheme of the kernel above with the copy engine doing the moving: a stage is two whole slabs
// (2 x 1280 bytes, each one contiguous in HBM and 16-byte aligned), fetched by two cp.async.bulk
// instructions that lane 0 issues and that complete on the stage's own mbarrier (transaction
// bytes); the warp's lanes wait on that barrier (bounded), consume the stage, meet at __syncwarp and
// lane 0 re-arms the barrier and refills the slot.  No block-wide barrier, no producer warp, the
// same bytes in flight per SM as with 16-byte cp.async copies (rings of the same depth and size).
// A bulk copy lands the slab as it lies in HBM, so a lane cannot own a token (the four 16-byte
// chunks of a token would sit in the same banks for every other lane); four lanes share a token
// instead, lane (token, group) reads the group's 16 code bytes and its {scale, min}, and two
// shuffles add the groups up.  Only this GPU's own HBM is read, by plain (single-destination) bulk copies.
template <typename T, int VARIANT, int NW, int DEPTH, int PPB>
__global__ void __launch_bounds__(NW * 32, (220 * 1024) / (NW * DEPTH * kWarpStageBytes + 2048))
estimate_int4_bulk_warp_kernel(const EstParams p) {
  extern __shared__ __align__(128) uint8_t sm_ring[];  // NW * DEPTH * kWarpStageBytes
  __shared__ __align__(8) uint64_t sm_bar[NW][DEPTH];
  __shared__ int sm_phys[PPB + 1];
  __shared__ int sm_ntok[PPB + 1];
  __shared__ QRegs<VARIANT> sm_q[4];

  const int row = blockIdx.y;
  const bool has_cand = p.cand_pages != nullptr;
  int b, kvh, h;
  if (has_cand) {
    b = row / p.Hq;
    h = row % p.Hq;
    kvh = h / (p.Hq / p.Hkv);
  } else {  // one query head per KV head
    b = row / p.Hkv;
    kvh = row % p.Hkv;
    h = kvh;
  }
  pdl_wait();  // candidate lists (and maybe q, the page table) come from the kernel before; nothing is read earlier
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = has_cand ? min(p.cand_npages[b * p.Hq + h], p.max_k) : n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * PPB;
  if (first >= n_pages) return;
  const int n_here = min(PPB, n_pages - first);

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  if (tid <= PPB) {
    int phys = -1, ntok = 0;
    if (tid < n_here) {
      const int seq_page = has_cand ? p.cand_pages[(size_t)(b * p.Hq + h) * p.max_k + first + tid] : first + tid;
      if (seq_page >= 0 && seq_page < n_seq_pages) {
        phys = p.indices[page_base + seq_page];
        if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      }
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      ntok = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
    sm_phys[tid] = phys;
    sm_ntok[tid] = phys < 0 ? 0 : ntok;
  }
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) mbar_init(&sm_bar[warp][d], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid >= NW * 32 - 4) {
    float qf[32];
    load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h)) * kD +
                        (tid - (NW * 32 - 4)) * kGroup, qf);
    sm_q[tid - (NW * 32 - 4)].init(qf);
  }
  __syncthreads();

  uint8_t* const ring = sm_ring + (size_t)warp * DEPTH * kWarpStageBytes;
  const int n_pairs = (n_here + 1) >> 1;
  const int my_pairs = (n_pairs > warp) ? (n_pairs - warp + NW - 1) / NW : 0;
  const uint8_t* const k4_head = p.k4 + (size_t)kvh * kSlab;
  const size_t page_stride = (size_t)p.Hkv * kSlab;

  // lane 0: arm the slot's barrier with the bytes that will arrive, then start the copies
  uint32_t armed = 0;  // bit d: slot d has been armed and not yet consumed (the same in every lane)
  auto issue = [&](int i, int slot) {
    if (i < my_pairs) {
      armed |= 1u << slot;
      if (lane == 0) {
        const int pg0 = (warp + i * NW) * 2;
        const int phys0 = sm_phys[pg0], phys1 = sm_phys[pg0 + 1];  // missing pages hold -1
        uint8_t* const dst = ring + slot * kWarpStageBytes;
        mbar_arrive_expect_tx(&sm_bar[warp][slot], (phys0 >= 0 ? kSlab : 0) + (phys1 >= 0 ? kSlab : 0));
        if (phys0 >= 0) bulk_copy_g2s(dst, k4_head + (size_t)phys0 * page_stride, kSlab, &sm_bar[warp][slot]);
        if (phys1 >= 0) bulk_copy_g2s(dst + kSlab, k4_head + (size_t)phys1 * page_stride, kSlab, &sm_bar[warp][slot]);
      }
    }
  };
#pragma unroll
  for (int i = 0; i < DEPTH - 1; ++i) issue(i, i);

  const int grp = lane & 3, tok8 = lane >> 2;
  const QRegs<VARIANT> qr = sm_q[grp];
  float* const out_row = p.scores + (size_t)(b * p.Hq + h) * p.stride + (size_t)first * kPage + tok8;
  int use_slot = 0, fill_slot = DEPTH - 1;
  uint32_t phase = 0;  // bit d: parity of the phase of slot d that is waited for next
  bool alive = true;
  for (int i = 0; i < my_pairs && alive; ++i) {
    // the whole warp goes on or gives up together
    if (!__all_sync(0xffffffffu, mbar_wait(&sm_bar[warp][use_slot], (phase >> use_slot) & 1u))) {
      if (lane == 0) raise_flag(p.status, TWL_FLAG_WAIT_LIMIT);
      alive = false;  // give up on this warp's pages; the drain below still waits for what is in flight
      break;
    }
    phase ^= 1u << use_slot;
    armed &= ~(1u << use_slot);
    const int pg0 = (warp + i * NW) * 2;
    const uint8_t* stage = ring + use_slot * kWarpStageBytes;
#pragma unroll
    for (int s4 = 0; s4 < 4; ++s4) {  // half a page (8 tokens) per step
      const int pgl = s4 >> 1, half = s4 & 1;
      const int pg = pg0 + pgl;
      const uint8_t* slab = stage + pgl * kSlab;
      const uint4 w = *reinterpret_cast<const uint4*>(slab + half * 512 + lane * 16);
      const uint32_t sz = *reinterpret_cast<const uint32_t*>(slab + kSlabCodes + half * 128 + lane * 4);
      const float2 szf = __half22float2(*reinterpret_cast<const __half2*>(&sz));
      float part = fmaf(szf.x, qr.dot(w), szf.y * qr.qsum);
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      if (grp == 0 && pg < n_here) {
        const int tk = half * 8 + tok8;
        out_row[pg * kPage + half * 8] = (tk < sm_ntok[pg]) ? part * p.sm_scale : -INFINITY;
      }
    }
    __syncwarp();  // every lane is done reading the slot that the next issue overwrites
    issue(i + DEPTH - 1, fill_slot);
    use_slot = (use_slot + 1 == DEPTH) ? 0 : use_slot + 1;
    fill_slot = (fill_slot + 1 == DEPTH) ? 0 : fill_slot + 1;
  }
  if (!alive && lane == 0) {
    // copies may still be writing into the ring: wait (bounded) for every slot that was armed and not consumed
    for (int d = 0; d < DEPTH; ++d)
      if (armed & (1u << d)) mbar_wait(&sm_bar[warp][d], (phase >> d) & 1u);
  }
}

// The same streaming scheme for a KV head shared by G query heads (every page is a candidate).
// The codes of a token are unpacked once and used for all G heads; q does not fit in registers G
// times, so each head's converted q sits in shared memory and is read with broadcast loads.
template <typename T, int G>
__global__ void __launch_bounds__(kEstThreads)
estimate_int4_warp_group_kernel(const EstParams p) {
  constexpr int VARIANT = VAR_DP4A;
  extern __shared__ __align__(128) uint8_t sm_ring[];  // kEstWarps * kRingDepth * kWarpStageBytes
  __shared__ int sm_phys[kWarpPagesPerBlock];
  __shared__ int sm_ntok[kWarpPagesPerBlock];
  __shared__ __align__(16) QRegs<VARIANT> sm_q[G][4];

  const int row = blockIdx.y;
  constexpr bool has_cand = false;
  const int b = row / p.Hkv, kvh = row % p.Hkv;
  const int h = kvh * G;  // first query head of the group
  pdl_wait();  // candidate lists (and maybe q, the page table) come from the kernel before; nothing is read earlier
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = has_cand ? min(p.cand_npages[b * p.Hq + h], p.max_k) : n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * kWarpPagesPerBlock;
  if (first >= n_pages) return;
  const int n_here = min(kWarpPagesPerBlock, n_pages - first);

  const int tid = threadIdx.x;
  // four threads fetch q now and convert it later, after the first copies are on their way
  const bool q_thread = tid >= kEstThreads - 4 * G;
  const int qj = tid - (kEstThreads - 4 * G);  // head qj/4 of the group, channel group qj%4
  float qf[32];
  if (q_thread)
    load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h + (qj >> 2))) * kD +
                        (qj & 3) * kGroup, qf);
  if (tid < kWarpPagesPerBlock) {
    int phys = -1, ntok = 0;
    if (tid < n_here) {
      const int seq_page = has_cand ? p.cand_pages[(size_t)(b * p.Hq + h) * p.max_k + first + tid] : first + tid;
      if (seq_page >= 0 && seq_page < n_seq_pages) {
        phys = p.indices[page_base + seq_page];
        if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      }
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      ntok = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
    sm_phys[tid] = phys;
    sm_ntok[tid] = phys < 0 ? 0 : ntok;
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  uint8_t* const ring = sm_ring + (size_t)warp * kRingDepth * kWarpStageBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const int n_pairs = (n_here + 1) >> 1;
  const int my_pairs = (n_pairs > warp) ? (n_pairs - warp + kEstWarps - 1) / kEstWarps : 0;

  // Per-lane constants of the five 16-byte copies of a stage: chunk c = c5*32+lane of the pair,
  // i.e. page c/80 and chunk r = c%80 of its slab (0..63 codes, 64..79 scale/min).
  uint32_t src16[5], dst_off[5];
  bool second[5];
#pragma unroll
  for (int c5 = 0; c5 < 5; ++c5) {
    const int c = c5 * 32 + lane;
    const int pgl = c >= 80 ? 1 : 0;
    const int r = c - pgl * 80;
    second[c5] = pgl != 0;
    src16[c5] = r;
    if (r < 64) {
      const int t = pgl * 16 + (r >> 2), g = r & 3;
      dst_off[c5] = t * 64 + (((g + (t >> 1)) & 3) << 4);
    } else {
      dst_off[c5] = 2048 + (pgl * 16 + (r - 64)) * 16;
    }
  }
  const uint4* const k4_head16 = reinterpret_cast<const uint4*>(p.k4 + (size_t)kvh * kSlab);
  const uint32_t page_stride16 = (uint32_t)(p.Hkv * (kSlab / 16));

  // issue the copies of this warp's i-th pair into the given ring slot
  auto issue = [&](int i, int slot) {
    if (i < my_pairs) {
      const int pg0 = (warp + i * kEstWarps) * 2;
      const uint32_t dst0 = ring_u32 + slot * kWarpStageBytes;
      const int phys0 = sm_phys[pg0], phys1 = sm_phys[pg0 + 1];  // missing pages hold -1
#pragma unroll
      for (int c5 = 0; c5 < 5; ++c5) {
        const int phys = second[c5] ? phys1 : phys0;
        if (phys >= 0)
          cp_async16(dst0 + dst_off[c5], k4_head16 + ((size_t)phys * page_stride16 + src16[c5]));
      }
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };

#pragma unroll
  for (int i = 0; i < kRingDepth - 1; ++i) issue(i, i);

  if (q_thread) sm_q[qj >> 2][qj & 3].init(qf);
  __syncthreads();

  uint32_t rd_off[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) rd_off[g] = lane * 64 + (((g + (lane >> 1)) & 3) << 4);
  float* const out_row = p.scores + (size_t)(b * p.Hq + h) * p.stride + (size_t)first * kPage;
  int use_slot = 0, fill_slot = kRingDepth - 1;
  for (int i = 0; i < my_pairs; ++i) {
    cp_async_wait<kRingDepth - 2>();  // pair i has landed (this thread's copies)
    __syncwarp();                     // ... and every other lane's
    const int pg0 = (warp + i * kEstWarps) * 2;
    const uint8_t* stage = ring + use_slot * kWarpStageBytes;
    const int pgl = lane >> 4, tl = lane & 15;
    const int ntok = sm_ntok[pg0 + pgl];
    const bool present = sm_phys[pg0 + pgl] >= 0;
    const uint4 sz = *reinterpret_cast<const uint4*>(stage + 2048 + lane * 16);
    const uint32_t szw[4] = {sz.x, sz.y, sz.z, sz.w};
    float acc[G];
#pragma unroll
    for (int hh = 0; hh < G; ++hh) acc[hh] = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 w = *reinterpret_cast<const uint4*>(stage + rd_off[g]);
      const float2 szf = __half22float2(*reinterpret_cast<const __half2*>(&szw[g]));
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
      uint32_t even[4], odd16[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        even[j] = ws[j] & 0x0F0F0F0Fu;
        odd16[j] = ws[j] & 0xF0F0F0F0u;
      }
#pragma unroll
      for (int hh = 0; hh < G; ++hh) {
        // same address in every lane: broadcast reads, as four 16-byte loads and one 8-byte load
        // (word-wise reads made the shared-memory pipe the limit: 72 % busy at G = 4)
        const uint4* qp = reinterpret_cast<const uint4*>(&sm_q[hh][g]);
        const uint4 qhe = qp[0], qho = qp[1], qle = qp[2], qlo = qp[3];
        const float2 inv_sum = *reinterpret_cast<const float2*>(qp + 4);  // {inv, qsum}
        const uint32_t ahe[4] = {qhe.x, qhe.y, qhe.z, qhe.w}, aho[4] = {qho.x, qho.y, qho.z, qho.w};
        const uint32_t ale[4] = {qle.x, qle.y, qle.z, qle.w}, alo[4] = {qlo.x, qlo.y, qlo.z, qlo.w};
        int he = 0, ho = 0;
        uint32_t le = 0, lo = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          he = dp4a_u8_s8(even[j], ahe[j], he);
          ho = dp4a_u8_s8(odd16[j], aho[j], ho);
          le = dp4a_u8_u8(even[j], ale[j], le);
          lo = dp4a_u8_u8(odd16[j], alo[j], lo);
        }
        const int tot = (he + (ho >> 4)) * 256 + (int)(le + (lo >> 4));
        const float dot = (__int_as_float(0x4B400000 + tot) - 12582912.f) * inv_sum.x;
        acc[hh] = fmaf(szf.x, dot, acc[hh]);
        acc[hh] = fmaf(szf.y, inv_sum.y, acc[hh]);
      }
    }
    __syncwarp();      // all lanes are done reading the slot that the next issue overwrites
    issue(i + kRingDepth - 1, fill_slot);
    use_slot = (use_slot + 1 == kRingDepth) ? 0 : use_slot + 1;
    fill_slot = (fill_slot + 1 == kRingDepth) ? 0 : fill_slot + 1;
    if (pg0 + pgl < n_here) {
#pragma unroll
      for (int hh = 0; hh < G; ++hh)
        out_row[(size_t)hh * p.stride + (pg0 + pgl) * kPage + tl] =
            (present && tl < ntok) ? acc[hh] * p.sm_scale : -INFINITY;
    }
  }
  cp_async_wait<0>();
}

// ---- query-head groups on the tensor cores ---------------------------------------------------------
// The same warp-private rings, but a staged page (16 tokens) is scored against the whole group with
// m16n8k16 tiles: A = the page's codes of one 32-channel quantisation group, turned into fp16 in
// registers, B = the group's queries for those channels, fp32 accumulators; then
// score += scale * acc + min * sum(q) per (token, group) as in the other kernels.  The work per
// staged byte no longer grows with the number of query heads.
//
// Lane 4*g + t owns tokens g and g+8 of the page and word t of their 16-byte group chunk: eight
// nibbles, channels 8t..8t+7 of the group.  Two codes at a time are or-ed into the mantissas of a
// pair of fp16 numbers - bits 0-3 under 0x6400 give 1024 + c, bits 4-7 under 0x5400 give 64 + c, the
// same again after one shift by 8 - and one exact subtraction each brings them back to c.  (fp16
// takes a nibble at two bit positions, bf16 only at one; that is one shift per word instead of
// three, and the logic unit is what bounds this kernel.)  The k-slots of a tile thus hold channels
// in the order the nibbles come out; B is built once per block in the same order.
// B is fp16 whatever the model dtype: q is scaled by a power of two that puts the group's largest
// |q| into [128, 256) - exact, undone together with the softmax scale - so a bf16 q converts to fp16
// without rounding unless an element is 2^22 times smaller than the largest one.
// Reads of the ring are conflict-free: the eight tokens of a quarter warp's request sit in eight
// different 16-byte bank groups (the chunk rotation of the copy).
__device__ __forceinline__ void unpack_codes_f16(uint32_t w, uint32_t (&r)[4]) {
  const __half2 b1024 = __half2half2(__ushort_as_half(0x6400));
  const __half2 b64 = __half2half2(__ushort_as_half(0x5400));
  const uint32_t w8 = w >> 8;
  uint32_t u0 = (w & 0x000F000Fu) | 0x64006400u, u1 = (w & 0x00F000F0u) | 0x54005400u;
  uint32_t u2 = (w8 & 0x000F000Fu) | 0x64006400u, u3 = (w8 & 0x00F000F0u) | 0x54005400u;
  const __half2 c0 = __hsub2(*reinterpret_cast<__half2*>(&u0), b1024);  // channels (0, 4) of the word's eight
  const __half2 c1 = __hsub2(*reinterpret_cast<__half2*>(&u1), b64);    // (1, 5)
  const __half2 c2 = __hsub2(*reinterpret_cast<__half2*>(&u2), b1024);  // (2, 6)
  const __half2 c3 = __hsub2(*reinterpret_cast<__half2*>(&u3), b64);    // (3, 7)
  r[0] = *reinterpret_cast<const uint32_t*>(&c0);
  r[1] = *reinterpret_cast<const uint32_t*>(&c1);
  r[2] = *reinterpret_cast<const uint32_t*>(&c2);
  r[3] = *reinterpret_cast<const uint32_t*>(&c3);
}

template <typename T, int G>
__global__ void __launch_bounds__(kEstThreads, 2)
estimate_int4_mma_group_kernel(const EstParams p) {
  static_assert(G >= 2 && G <= 8, "one n8 tile holds the group");
  extern __shared__ __align__(128) uint8_t sm_ring[];  // kEstWarps * kRingDepth * kWarpStageBytes
  __shared__ int sm_phys[kWarpPagesPerBlock + 1];
  __shared__ int sm_ntok[kWarpPagesPerBlock + 1];

  const int row = blockIdx.y;
  const int b = row / p.Hkv, kvh = row % p.Hkv;
  const int h = kvh * G;  // first query head of the group
  pdl_wait();  // q and the page table may come from the kernel before; scores may still be read by an older one
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * kWarpPagesPerBlock;
  if (first >= n_pages) return;
  const int n_here = min(kWarpPagesPerBlock, n_pages - first);

  const int tid = threadIdx.x;
  if (tid <= kWarpPagesPerBlock) {  // one entry more than pages: the partner of an odd last page
    int phys = -1, ntok = 0;
    if (tid < n_here) {
      const int seq_page = first + tid;
      phys = p.indices[page_base + seq_page];
      if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      ntok = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
    sm_phys[tid] = phys;
    sm_ntok[tid] = phys < 0 ? 0 : ntok;  // 0 tokens: every slot of the page scores -inf
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;
  uint8_t* const ring = sm_ring + (size_t)warp * kRingDepth * kWarpStageBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const int n_pairs = (n_here + 1) >> 1;
  const int my_pairs = (n_pairs > warp) ? (n_pairs - warp + kEstWarps - 1) / kEstWarps : 0;

  // Per-lane constants of the five 16-byte copies of a stage: chunk c = c5*32+lane of the pair,
  // i.e. page c/80 and chunk r = c%80 of its slab (0..63 codes, 64..79 scale/min).  Which page a
  // copy belongs to is fixed for four of the five (chunks 0..63 first page, 96..159 second) and
  // depends on the lane only for the third.
  uint32_t src_off[5], dst_off[5];
#pragma unroll
  for (int c5 = 0; c5 < 5; ++c5) {
    const int c = c5 * 32 + lane;
    const int pgl = c >= 80 ? 1 : 0;
    const int r = c - pgl * 80;
    src_off[c5] = r * 16;
    if (r < 64) {
      const int tk = pgl * 16 + (r >> 2), g4 = r & 3;
      dst_off[c5] = tk * 64 + (((g4 + (tk >> 1)) & 3) << 4);
    } else {
      dst_off[c5] = 2048 + (pgl * 16 + (r - 64)) * 16;
    }
  }
  const bool third_is_second = lane >= 16;
  const uint8_t* const k4_head = p.k4 + (size_t)kvh * kSlab;
  const size_t page_stride = (size_t)p.Hkv * kSlab;

  // Absent pages (table entry out of range, partner of an odd last page) copy the slab of physical
  // page 0, which is always mapped; their scores are never used.
  auto issue = [&](int i, int slot) {
    if (i < my_pairs) {
      const int pg0 = (warp + i * kEstWarps) * 2;
      const uint32_t dst0 = ring_u32 + slot * kWarpStageBytes;
      const uint8_t* const s0 = k4_head + (size_t)max(sm_phys[pg0], 0) * page_stride;
      const uint8_t* const s1 = k4_head + (size_t)max(sm_phys[pg0 + 1], 0) * page_stride;
      const uint8_t* const s2 = third_is_second ? s1 : s0;
      cp_async16(dst0 + dst_off[0], s0 + src_off[0]);
      cp_async16(dst0 + dst_off[1], s0 + src_off[1]);
      cp_async16(dst0 + dst_off[2], s2 + src_off[2]);
      cp_async16(dst0 + dst_off[3], s1 + src_off[3]);
      cp_async16(dst0 + dst_off[4], s1 + src_off[4]);
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };

#pragma unroll
  for (int i = 0; i < kRingDepth - 1; ++i) issue(i, i);

  // B fragments (head gq of the group, this lane's channels 8t..8t+7 of every quantisation group)
  // and the channel sums of heads 2t and 2t+1, whose scores this lane ends up owning
  uint32_t bq[4][4];
  float qs0[4], qs1[4];
  float out_scale;
  {
    const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)(b * p.Hq + h + (gq < G ? gq : 0)) * kD;
    float qf[4][8];
    float amax = 0.f;
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow) + 4 * grp + t);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = Elem<T>::to_f2(u[k]);
        qf[grp][2 * k] = gq < G ? f.x : 0.f;
        qf[grp][2 * k + 1] = gq < G ? f.y : 0.f;
        amax = fmaxf(amax, fmaxf(fabsf(qf[grp][2 * k]), fabsf(qf[grp][2 * k + 1])));
      }
    }
    amax = warp_max(amax);  // over every head and channel of the group
    int e = (amax > 0.f && amax < INFINITY) ? (7 - ilogbf(amax)) : 0;  // amax * 2^e in [128, 256)
    e = max(-100, min(100, e));
    const float up = ldexpf(1.f, e);
    out_scale = p.sm_scale * ldexpf(1.f, -e);
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      float sum = 0.f;
      __half hq[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        hq[k] = __float2half_rn(qf[grp][k] * up);
        sum += __half2float(hq[k]);  // the sum of what the tiles multiply with
      }
      // elements e0..e7 = channels 8t..8t+7; the tiles want the pairs (e0,e4) (e1,e5) (e2,e6) (e3,e7)
#pragma unroll
      for (int k = 0; k < 4; ++k)
        bq[grp][k] = (uint32_t)__half_as_ushort(hq[k]) | ((uint32_t)__half_as_ushort(hq[k + 4]) << 16);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // sum of q over the group's 32 channels, head gq
      qs0[grp] = __shfl_sync(0xffffffffu, sum, (2 * t) * 4);
      qs1[grp] = __shfl_sync(0xffffffffu, sum, (2 * t + 1) * 4);
    }
  }

  // byte offsets, inside a stage, of this lane's code word of token gq for each quantisation group
  // (tokens gq+8, 16+gq, 24+gq follow at +512, +1024, +1536: the rotation repeats every eight tokens)
  uint32_t code_off[4];
#pragma unroll
  for (int grp = 0; grp < 4; ++grp) code_off[grp] = gq * 64 + (((grp + (gq >> 1)) & 3) << 4) + t * 4;
  const uint32_t sz_off = 2048 + gq * 16;  // {scale, min} x 4 groups of token gq; +128 per eight tokens

  float* const out0 = p.scores + (size_t)(b * p.Hq + h + 2 * t) * p.stride + (size_t)first * kPage + gq;
  const bool own0 = 2 * t < G, own1 = 2 * t + 1 < G;
  const uint8_t* stage = ring;
  int fill_slot = kRingDepth - 1;
  for (int i = 0; i < my_pairs; ++i) {
    cp_async_wait<kRingDepth - 2>();  // pair i has landed (this thread's copies)
    __syncwarp();                     // ... and every other lane's
    float res[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {  // one page = one m16 tile
      const uint4 sza = *reinterpret_cast<const uint4*>(stage + sz_off + mt * 256);
      const uint4 szb = *reinterpret_cast<const uint4*>(stage + sz_off + mt * 256 + 128);
      const uint32_t sa[4] = {sza.x, sza.y, sza.z, sza.w}, sb[4] = {szb.x, szb.y, szb.z, szb.w};
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const uint32_t wa = *reinterpret_cast<const uint32_t*>(stage + code_off[grp] + mt * 1024);
        const uint32_t wb = *reinterpret_cast<const uint32_t*>(stage + code_off[grp] + mt * 1024 + 512);
        uint32_t ca[4], cb[4];
        unpack_codes_f16(wa, ca);
        unpack_codes_f16(wb, cb);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        MmaTile<__half>::run(acc, ca[0], cb[0], ca[1], cb[1], bq[grp][0], bq[grp][1]);
        MmaTile<__half>::run(acc, ca[2], cb[2], ca[3], cb[3], bq[grp][2], bq[grp][3]);
        const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&sa[grp]));  // {scale, min}
        const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&sb[grp]));
        r0 = fmaf(fa.x, acc[0], fmaf(fa.y, qs0[grp], r0));
        r1 = fmaf(fa.x, acc[1], fmaf(fa.y, qs1[grp], r1));
        r2 = fmaf(fb.x, acc[2], fmaf(fb.y, qs0[grp], r2));
        r3 = fmaf(fb.x, acc[3], fmaf(fb.y, qs1[grp], r3));
      }
      res[mt][0] = r0; res[mt][1] = r1; res[mt][2] = r2; res[mt][3] = r3;
    }
    __syncwarp();      // all lanes are done reading the slot that the next issue overwrites
    issue(i + kRingDepth - 1, fill_slot);
    fill_slot = (fill_slot + 1 == kRingDepth) ? 0 : fill_slot + 1;
    stage = (stage + kWarpStageBytes == ring + kRingDepth * kWarpStageBytes) ? ring : stage + kWarpStageBytes;
    const int pg0 = (warp + i * kEstWarps) * 2;
    if (own0) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int pg = pg0 + mt;
        if (pg < n_here) {
          const int ntok = sm_ntok[pg];  // 0 for a page whose table entry was out of range
          float* const o0 = out0 + pg * kPage;
          o0[0] = gq < ntok ? res[mt][0] * out_scale : -INFINITY;
          o0[8] = gq + 8 < ntok ? res[mt][2] * out_scale : -INFINITY;
          if (own1) {
            o0[p.stride] = gq < ntok ? res[mt][1] * out_scale : -INFINITY;
            o0[p.stride + 8] = gq + 8 < ntok ? res[mt][3] * out_scale : -INFINITY;
          }
        }
      }
    }
  }
  cp_async_wait<0>();
}

// ---- the same on the integer tensor-core path --------------------------------------------------
// m16n8k32 tiles of 8-bit integers: one tile spans exactly one 32-channel quantisation group, and a
// code word turns into two operand registers with two masks and one shift (the 16-bit tiles above
// spend nine instructions on it, and the logic unit is what bounds that kernel).  q is what the
// single-head kernel uses: per head, q_d ~= (256*hi_d + lo_d) * 2^-e with |256*hi + lo| < 2^13, hi a
// signed and lo an unsigned byte - two tiles per (page, group), one against the hi bytes and one
// against the lo bytes, both exact in 32-bit integers.  The lo tile starts from the bit pattern of
// 1.5 * 2^23, so that hi*256 + lo, read as a float, is 12582912 + the integer dot product (exact
// below 2^22), and one exact subtraction leaves the dot product.
//
// Lane 4*g + t owns tokens g and g+8 of the page and word t of their 16-byte group chunk, as above:
// the low nibbles of the word (channels 8t, 8t+2, 8t+4, 8t+6) fill the k-slots 4t..4t+3, the high
// nibbles (the odd channels) the k-slots 16+4t..16+4t+3; B holds head g's bytes in the same order.
struct ImmaTile {
  // d = a (u8, 16x32) * b (8-bit, 32x8) + c, 32-bit integers
  static __device__ __forceinline__ void run_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1, int c) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
  }
  static __device__ __forceinline__ void run_u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1, int c) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
  }
};

template <typename T, int G, int NW, int DEPTH, int NBLK>
__global__ void __launch_bounds__(NW * 32, NBLK)
estimate_int4_imma_group_kernel(const EstParams p) {
  constexpr int kPagesHere = NW * 16;  // eight ring stages of two pages per warp
  static_assert(G >= 2 && G <= 8, "one n8 tile holds the group");
  extern __shared__ __align__(128) uint8_t sm_ring[];  // NW * DEPTH * kWarpStageBytes
  __shared__ int sm_phys[kPagesHere + 1];
  __shared__ int sm_ntok[kPagesHere + 1];

  const int row = blockIdx.y;
  const int b = row / p.Hkv, kvh = row % p.Hkv;
  const int h = kvh * G;  // first query head of the group
  pdl_wait();  // q and the page table may come from the kernel before; scores may still be read by an older one
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * kPagesHere;
  if (first >= n_pages) return;
  const int n_here = min(kPagesHere, n_pages - first);

  const int tid = threadIdx.x;
  if (tid <= kPagesHere) {  // one entry more than pages: the partner of an odd last page
    int phys = -1, ntok = 0;
    if (tid < n_here) {
      const int seq_page = first + tid;
      phys = p.indices[page_base + seq_page];
      if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      ntok = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
    sm_phys[tid] = phys;
    sm_ntok[tid] = phys < 0 ? 0 : ntok;  // 0 tokens: every slot of the page scores -inf
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;
  uint8_t* const ring = sm_ring + (size_t)warp * DEPTH * kWarpStageBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const int n_pairs = (n_here + 1) >> 1;
  const int my_pairs = (n_pairs > warp) ? (n_pairs - warp + NW - 1) / NW : 0;

  // the five 16-byte copies of a stage, as in the 16-bit tile kernel
  uint32_t src_off[5], dst_off[5];
#pragma unroll
  for (int c5 = 0; c5 < 5; ++c5) {
    const int c = c5 * 32 + lane;
    const int pgl = c >= 80 ? 1 : 0;
    const int r = c - pgl * 80;
    src_off[c5] = r * 16;
    if (r < 64) {
      const int tk = pgl * 16 + (r >> 2), g4 = r & 3;
      dst_off[c5] = tk * 64 + (((g4 + (tk >> 1)) & 3) << 4);
    } else {
      dst_off[c5] = 2048 + (pgl * 16 + (r - 64)) * 16;
    }
  }
  const bool third_is_second = lane >= 16;
  const uint8_t* const k4_head = p.k4 + (size_t)kvh * kSlab;
  const size_t page_stride = (size_t)p.Hkv * kSlab;

  auto issue = [&](int i, int slot) {
    if (i < my_pairs) {
      const int pg0 = (warp + i * NW) * 2;
      const uint32_t dst0 = ring_u32 + slot * kWarpStageBytes;
      const uint8_t* const s0 = k4_head + (size_t)max(sm_phys[pg0], 0) * page_stride;
      const uint8_t* const s1 = k4_head + (size_t)max(sm_phys[pg0 + 1], 0) * page_stride;
      const uint8_t* const s2 = third_is_second ? s1 : s0;
      cp_async16(dst0 + dst_off[0], s0 + src_off[0]);
      cp_async16(dst0 + dst_off[1], s0 + src_off[1]);
      cp_async16(dst0 + dst_off[2], s2 + src_off[2]);
      cp_async16(dst0 + dst_off[3], s1 + src_off[3]);
      cp_async16(dst0 + dst_off[4], s1 + src_off[4]);
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };

#pragma unroll
  for (int i = 0; i < DEPTH - 1; ++i) issue(i, i);

  // B fragments of head gq (this lane's channels 8t..8t+7 of every group: even ones, then odd
  // ones; hi and lo bytes), and of heads 2t and 2t+1, whose scores this lane ends up owning, the
  // sums of the integers over each group's channels and the factor that undoes the scaling
  uint32_t bh[4][2], bl[4][2];
  float qs0[4], qs1[4];
  float out_scale0, out_scale1;
  {
    const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)(b * p.Hq + h + (gq < G ? gq : 0)) * kD;
    float qf[4][8];
    float amax = 0.f;
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow) + 4 * grp + t);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = Elem<T>::to_f2(u[k]);
        qf[grp][2 * k] = gq < G ? f.x : 0.f;
        qf[grp][2 * k + 1] = gq < G ? f.y : 0.f;
        amax = fmaxf(amax, fmaxf(fabsf(qf[grp][2 * k]), fabsf(qf[grp][2 * k + 1])));
      }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));  // over the head's 128 channels
    int e = (amax > 0.f && amax < INFINITY) ? (12 - ilogbf(amax)) : 0;  // amax * 2^e in [2^12, 2^13)
    e = max(-100, min(100, e));
    const float up = ldexpf(1.f, e);
    const float undo = p.sm_scale * ldexpf(1.f, -e);
    out_scale0 = __shfl_sync(0xffffffffu, undo, (2 * t) * 4);
    out_scale1 = __shfl_sync(0xffffffffu, undo, (2 * t + 1) * 4);
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      int sum = 0;
      uint32_t he = 0, ho = 0, le = 0, lo = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int a = __float2int_rn(qf[grp][2 * k] * up);      // channel 8t + 2k
        const int c = __float2int_rn(qf[grp][2 * k + 1] * up);  // channel 8t + 2k + 1
        sum += a + c;
        he |= (uint32_t)((a >> 8) & 0xFF) << (8 * k);
        le |= (uint32_t)(a & 0xFF) << (8 * k);
        ho |= (uint32_t)((c >> 8) & 0xFF) << (8 * k);
        lo |= (uint32_t)(c & 0xFF) << (8 * k);
      }
      bh[grp][0] = he; bh[grp][1] = ho;
      bl[grp][0] = le; bl[grp][1] = lo;
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // over the group's 32 channels, head gq
      qs0[grp] = (float)__shfl_sync(0xffffffffu, sum, (2 * t) * 4);
      qs1[grp] = (float)__shfl_sync(0xffffffffu, sum, (2 * t + 1) * 4);
    }
  }

  uint32_t code_off[4];
#pragma unroll
  for (int grp = 0; grp < 4; ++grp) code_off[grp] = gq * 64 + (((grp + (gq >> 1)) & 3) << 4) + t * 4;
  const uint32_t sz_off = 2048 + gq * 16;  // {scale, min} x 4 groups of token gq; +128 per eight tokens

  float* const out0 = p.scores + (size_t)(b * p.Hq + h + 2 * t) * p.stride + (size_t)first * kPage + gq;
  const bool own0 = 2 * t < G, own1 = 2 * t + 1 < G;
  const uint8_t* stage = ring;
  int fill_slot = DEPTH - 1;
  constexpr int kMagicBits = 0x4B400000;   // 1.5 * 2^23 as a float
  constexpr float kMagic = 12582912.f;
  for (int i = 0; i < my_pairs; ++i) {
    cp_async_wait<DEPTH - 2>();  // pair i has landed (this thread's copies)
    __syncwarp();                     // ... and every other lane's
    float res[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {  // one page = one m16 tile per group
      const uint4 sza = *reinterpret_cast<const uint4*>(stage + sz_off + mt * 256);
      const uint4 szb = *reinterpret_cast<const uint4*>(stage + sz_off + mt * 256 + 128);
      const uint32_t sa[4] = {sza.x, sza.y, sza.z, sza.w}, sb[4] = {szb.x, szb.y, szb.z, szb.w};
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const uint32_t wa = *reinterpret_cast<const uint32_t*>(stage + code_off[grp] + mt * 1024);
        const uint32_t wb = *reinterpret_cast<const uint32_t*>(stage + code_off[grp] + mt * 1024 + 512);
        const uint32_t a0 = wa & 0x0F0F0F0Fu, a2 = (wa >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wb & 0x0F0F0F0Fu, a3 = (wb >> 4) & 0x0F0F0F0Fu;
        int dl[4], dh[4];
        ImmaTile::run_u8(dl, a0, a1, a2, a3, bl[grp][0], bl[grp][1], kMagicBits);
        ImmaTile::run_s8(dh, a0, a1, a2, a3, bh[grp][0], bh[grp][1], 0);
        const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&sa[grp]));  // {scale, min}
        const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&sb[grp]));
        r0 = fmaf(fa.x, __int_as_float(dh[0] * 256 + dl[0]) - kMagic, fmaf(fa.y, qs0[grp], r0));
        r1 = fmaf(fa.x, __int_as_float(dh[1] * 256 + dl[1]) - kMagic, fmaf(fa.y, qs1[grp], r1));
        r2 = fmaf(fb.x, __int_as_float(dh[2] * 256 + dl[2]) - kMagic, fmaf(fb.y, qs0[grp], r2));
        r3 = fmaf(fb.x, __int_as_float(dh[3] * 256 + dl[3]) - kMagic, fmaf(fb.y, qs1[grp], r3));
      }
      res[mt][0] = r0; res[mt][1] = r1; res[mt][2] = r2; res[mt][3] = r3;
    }
    __syncwarp();      // all lanes are done reading the slot that the next issue overwrites
    issue(i + DEPTH - 1, fill_slot);
    fill_slot = (fill_slot + 1 == DEPTH) ? 0 : fill_slot + 1;
    stage = (stage + kWarpStageBytes == ring + DEPTH * kWarpStageBytes) ? ring : stage + kWarpStageBytes;
    const int pg0 = (warp + i * NW) * 2;
    if (pg0 + 1 < n_here && sm_ntok[pg0] == kPage && sm_ntok[pg0 + 1] == kPage) {
      // two whole pages (all but the last stage of a sequence): nothing to mask
      if (own0) {
        float* const o0 = out0 + pg0 * kPage;
        o0[0] = res[0][0] * out_scale0;
        o0[8] = res[0][2] * out_scale0;
        o0[kPage] = res[1][0] * out_scale0;
        o0[kPage + 8] = res[1][2] * out_scale0;
        if (own1) {
          float* const o1 = o0 + p.stride;
          o1[0] = res[0][1] * out_scale1;
          o1[8] = res[0][3] * out_scale1;
          o1[kPage] = res[1][1] * out_scale1;
          o1[kPage + 8] = res[1][3] * out_scale1;
        }
      }
    } else if (own0) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int pg = pg0 + mt;
        if (pg < n_here) {
          const int ntok = sm_ntok[pg];  // 0 for a page whose table entry was out of range
          float* const o0 = out0 + pg * kPage;
          o0[0] = gq < ntok ? res[mt][0] * out_scale0 : -INFINITY;
          o0[8] = gq + 8 < ntok ? res[mt][2] * out_scale0 : -INFINITY;
          if (own1) {
            o0[p.stride] = gq < ntok ? res[mt][1] * out_scale1 : -INFINITY;
            o0[p.stride + 8] = gq + 8 < ntok ? res[mt][3] * out_scale1 : -INFINITY;
          }
        }
      }
    }
  }
  cp_async_wait<0>();
}

// ---- groups of up to four query heads: both digits of q in one integer tile --------------------
// With G <= 4 the eight columns of a m16n8k32 tile hold the hi digits of the G heads (columns 0..3)
// and their lo digits (columns 4..7): q_d ~= (256*hi_d + lo_d) * 2^-e with lo in [-128, 127] and
// |hi| <= 127, both signed bytes (q rounded to 15 bits), so one tile per (page, group) does what
// the kernel above needs two for.  Lanes t = 0, 1 of a quad then own hi-digit columns and lanes t = 2, 3 the lo-digit columns
// of the same heads; each lane sums scale * dot over the page's four groups for its own columns,
// and the two digits meet once per page (one exchange across the quad) instead of once per group:
// the lane with the hi digits finishes token g, its partner token g + 8, and each stores its own.
// The term sum_groups min * (sum of the group's q integers) is a 16 x 8 x 8 product of its own
// (tokens x {group, half of the sum} x heads): one 16-bit float tile per page, whose result
// initialises the hi lanes' sums.  The {scale, min} pairs of the slab are its A operand as they
// lie (min duplicated into both halves); the sums are split into a 16-bit float and the exact
// remainder, both divided by 256 so that 256 * hi + lo restores them.
struct HmmaK8 {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.f));
  }
};

template <typename T, int G, int NW, int DEPTH, int NBLK>
__global__ void __launch_bounds__(NW * 32, NBLK)
estimate_int4_imma_digits_kernel(const EstParams p) {
  constexpr int kPagesHere = NW * 16;  // eight ring stages of two pages per warp
  static_assert(G >= 2 && G <= 4, "hi and lo digits of the group share one n8 tile");
  extern __shared__ __align__(128) uint8_t sm_ring[];  // NW * DEPTH * kWarpStageBytes: a ring of two-page stages per warp
  __shared__ int sm_phys[kPagesHere + 1];
  __shared__ int sm_ntok[kPagesHere + 1];

  const int row = blockIdx.y;
  const int b = row / p.Hkv, kvh = row % p.Hkv;
  const int h = kvh * G;  // first query head of the group
  pdl_wait();  // q and the page table may come from the kernel before; scores may still be read by an older one
  const int page_base = p.indptr[b];
  const int n_seq_pages = p.indptr[b + 1] - page_base;
  int n_pages = n_seq_pages;
  if (n_pages > p.stride / kPage) {
    n_pages = p.stride / kPage;
    if (threadIdx.x == 0 && blockIdx.x == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
  }
  const int first = blockIdx.x * kPagesHere;
  if (first >= n_pages) return;
  const int n_here = min(kPagesHere, n_pages - first);

  const int tid = threadIdx.x;
  if (tid <= kPagesHere) {  // one entry more than pages: the partner of an odd last page
    int phys = -1, ntok = 0;
    if (tid < n_here) {
      const int seq_page = first + tid;
      phys = p.indices[page_base + seq_page];
      if (phys < 0 || phys >= p.num_pages_total) phys = -1;
      if (phys < 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      ntok = (seq_page == n_seq_pages - 1) ? p.last_len[b] : kPage;
    }
    sm_phys[tid] = phys;
    sm_ntok[tid] = phys < 0 ? 0 : ntok;  // 0 tokens: every slot of the page scores -inf
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, t = lane & 3;
  uint8_t* const ring = sm_ring + (size_t)warp * DEPTH * kWarpStageBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const int n_pairs = (n_here + 1) >> 1;
  const int my_pairs = (n_pairs > warp) ? (n_pairs - warp + NW - 1) / NW : 0;

  // the five 16-byte copies of a stage, as in the kernels above
  uint32_t src_off[5], dst_off[5];
#pragma unroll
  for (int c5 = 0; c5 < 5; ++c5) {
    const int c = c5 * 32 + lane;
    const int pgl = c >= 80 ? 1 : 0;
    const int r = c - pgl * 80;
    src_off[c5] = r * 16;
    if (r < 64) {
      const int tk = pgl * 16 + (r >> 2), g4 = r & 3;
      dst_off[c5] = tk * 64 + (((g4 + (tk >> 1)) & 3) << 4);
    } else {
      dst_off[c5] = 2048 + (pgl * 16 + (r - 64)) * 16;
    }
  }
  const bool third_is_second = lane >= 16;
  const uint8_t* const k4_head = p.k4 + (size_t)kvh * kSlab;
  const size_t page_stride = (size_t)p.Hkv * kSlab;

  auto issue = [&](int i, int slot) {
    if (i < my_pairs) {
      const int pg0 = (warp + i * NW) * 2;
      const uint32_t dst0 = ring_u32 + slot * kWarpStageBytes;
      const uint8_t* const s0 = k4_head + (size_t)max(sm_phys[pg0], 0) * page_stride;
      const uint8_t* const s1 = k4_head + (size_t)max(sm_phys[pg0 + 1], 0) * page_stride;
      const uint8_t* const s2 = third_is_second ? s1 : s0;
      cp_async16(dst0 + dst_off[0], s0 + src_off[0]);
      cp_async16(dst0 + dst_off[1], s0 + src_off[1]);
      cp_async16(dst0 + dst_off[2], s2 + src_off[2]);
      cp_async16(dst0 + dst_off[3], s1 + src_off[3]);
      cp_async16(dst0 + dst_off[4], s1 + src_off[4]);
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };

#pragma unroll
  for (int i = 0; i < DEPTH - 1; ++i) issue(i, i);

  // Column gq of the tile: the hi digits of head gq (gq < 4) or the lo digits of head gq - 4, this
  // lane's channels 8t..8t+7 of every group (even ones, then odd ones).  Column gq of the min tile:
  // head gq's group sums (rows 2t, 2t+1: group t's sum as a 16-bit float and the remainder).
  uint32_t bd[4][2];
  uint32_t bmin;
  float c_own_a, c_own_b, c_x_a, c_x_b;
  const bool hi_lane = t < 2;
  {
    const int hh = gq & 3;
    const bool valid = hh < G;
    const bool lo_digit = gq >= 4;
    const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)(b * p.Hq + h + (valid ? hh : 0)) * kD;
    float qf[4][8];
    float amax = 0.f;
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow) + 4 * grp + t);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = Elem<T>::to_f2(u[k]);
        qf[grp][2 * k] = valid ? f.x : 0.f;
        qf[grp][2 * k + 1] = valid ? f.y : 0.f;
        amax = fmaxf(amax, fmaxf(fabsf(qf[grp][2 * k]), fabsf(qf[grp][2 * k + 1])));
      }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));  // over the head's 128 channels
    // 15 bits where the kernel above has 13: each digit has a tile column of its own here, so both digit
    // sums stay below 2^16 whatever the digits.  amax * 2^e in [2^14, 2^15), one bit less when the hi
    // digit of the largest element would not fit a signed byte (256 * 127 + 127 = 32639).
    int e = (amax > 0.f && amax < INFINITY) ? (14 - ilogbf(amax)) : 0;
    e = max(-100, min(100, e));
    if (amax * ldexpf(1.f, e) > 32639.f) e -= 1;
    const float up = ldexpf(1.f, e);
    const float undo = p.sm_scale * ldexpf(1.f, -e);
    const float os_a = __shfl_sync(0xffffffffu, undo, (2 * (t & 1)) * 4);      // head 2(t&1)
    const float os_b = __shfl_sync(0xffffffffu, undo, (2 * (t & 1) + 1) * 4);  // head 2(t&1) + 1
    c_own_a = hi_lane ? 256.f * os_a : os_a;
    c_x_a = hi_lane ? os_a : 256.f * os_a;
    c_own_b = hi_lane ? 256.f * os_b : os_b;
    c_x_b = hi_lane ? os_b : 256.f * os_b;
    int gsum[4];
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      int sum = 0;
      uint32_t ev = 0, od = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int a = __float2int_rn(qf[grp][2 * k] * up);      // channel 8t + 2k
        const int c = __float2int_rn(qf[grp][2 * k + 1] * up);  // channel 8t + 2k + 1
        sum += a + c;
        const int ah = (a + 128) >> 8, ch = (c + 128) >> 8;     // a = 256 * ah + al, al in [-128, 127]
        const int da = lo_digit ? a - (ah << 8) : ah;
        const int dc = lo_digit ? c - (ch << 8) : ch;
        ev |= (uint32_t)(da & 0xFF) << (8 * k);
        od |= (uint32_t)(dc & 0xFF) << (8 * k);
      }
      bd[grp][0] = ev; bd[grp][1] = od;
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // over the group's 32 channels, head gq & 3
      gsum[grp] = sum;
    }
    const int mine = t == 0 ? gsum[0] : t == 1 ? gsum[1] : t == 2 ? gsum[2] : gsum[3];
    const float sf = (float)mine * (1.f / 256.f);      // |sum| < 2^20: exact
    const __half s_hi = __float2half_rn(sf);
    const __half s_lo = __float2half_rn(sf - __half2float(s_hi));  // a multiple of 2^-8, at most 1: exact
    const __half2 pair = __halves2half2(s_hi, s_lo);
    bmin = (gq < G) ? *reinterpret_cast<const uint32_t*>(&pair) : 0u;
  }

  // ldmatrix row addresses: matrix lane >> 3 = {tokens 0-7, tokens 8-15} x {group 2j, group 2j + 1};
  // the lane then holds word t of token gq (and of token gq + 8) of both groups' 16-byte pieces
  uint32_t lm_off[2];
  {
    const int mat = lane >> 3, tok = (lane & 7) + 8 * (mat & 1);
#pragma unroll
    for (int j = 0; j < 2; ++j) lm_off[j] = tok * 64 + (((2 * j + (mat >> 1) + (tok >> 1)) & 3) << 4);
  }
  const uint32_t sz_off = 2048 + gq * 16;  // {scale, min} x 4 groups of token gq; +128 per eight tokens

  const int tk_own = gq + (hi_lane ? 0 : 8);  // the token of a page that this lane finishes and stores
  float* const out_a = p.scores + (size_t)(b * p.Hq + h + 2 * (t & 1)) * p.stride + (size_t)first * kPage + tk_own;
  const bool own_a = 2 * (t & 1) < G, own_b = 2 * (t & 1) + 1 < G;
  uint32_t stage_off = 0;
  int fill_slot = DEPTH - 1;
  constexpr int kMagicBits = 0x4B400000;   // 1.5 * 2^23 as a float
  constexpr float kMagic = 12582912.f;
  for (int i = 0; i < my_pairs; ++i) {
    cp_async_wait<DEPTH - 2>();  // pair i has landed (this thread's copies)
    __syncwarp();                     // ... and every other lane's
    const uint8_t* const stage = ring + stage_off;
    const uint32_t stage_u32 = ring_u32 + stage_off;
    float res[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {  // one page = one m16 tile per group
      const uint4 sza = *reinterpret_cast<const uint4*>(stage + sz_off + mt * 256);
      const uint4 szb = *reinterpret_cast<const uint4*>(stage + sz_off + mt * 256 + 128);
      const uint32_t ma = *reinterpret_cast<const uint32_t*>(stage + sz_off + mt * 256 + t * 4);
      const uint32_t mb = *reinterpret_cast<const uint32_t*>(stage + sz_off + mt * 256 + 128 + t * 4);
      float r[4];
      HmmaK8::run(r, __byte_perm(ma, 0, 0x3232), __byte_perm(mb, 0, 0x3232), bmin);
      const uint32_t sa[4] = {sza.x, sza.y, sza.z, sza.w}, sb[4] = {szb.x, szb.y, szb.z, szb.w};
      uint32_t w[2][4];  // per pair of groups: {token gq, token gq+8} x {group 2j, group 2j+1}
#pragma unroll
      for (int j = 0; j < 2; ++j)
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(w[j][0]), "=r"(w[j][1]), "=r"(w[j][2]), "=r"(w[j][3])
                     : "r"(stage_u32 + lm_off[j] + mt * 1024));
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        const uint32_t wa = w[grp >> 1][2 * (grp & 1)], wb = w[grp >> 1][2 * (grp & 1) + 1];
        const uint32_t a0 = wa & 0x0F0F0F0Fu, a2 = (wa >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wb & 0x0F0F0F0Fu, a3 = (wb >> 4) & 0x0F0F0F0Fu;
        int d[4];
        ImmaTile::run_s8(d, a0, a1, a2, a3, bd[grp][0], bd[grp][1], kMagicBits);
        const float s0 = __low2float(*reinterpret_cast<const __half2*>(&sa[grp]));  // scale of token gq
        const float s8 = __low2float(*reinterpret_cast<const __half2*>(&sb[grp]));  // ... of token gq + 8
        r[0] = fmaf(s0, __int_as_float(d[0]) - kMagic, r[0]);
        r[1] = fmaf(s0, __int_as_float(d[1]) - kMagic, r[1]);
        r[2] = fmaf(s8, __int_as_float(d[2]) - kMagic, r[2]);
        r[3] = fmaf(s8, __int_as_float(d[3]) - kMagic, r[3]);
      }
      // the hi lane finishes token gq with the partner's lo sums, the lo lane token gq + 8 with the partner's hi sums
      const float x0 = __shfl_xor_sync(0xffffffffu, hi_lane ? r[2] : r[0], 2);
      const float x1 = __shfl_xor_sync(0xffffffffu, hi_lane ? r[3] : r[1], 2);
      res[mt][0] = fmaf(hi_lane ? r[0] : r[2], c_own_a, x0 * c_x_a);
      res[mt][1] = fmaf(hi_lane ? r[1] : r[3], c_own_b, x1 * c_x_b);
    }
    __syncwarp();      // all lanes are done reading the slot that the next issue overwrites
    issue(i + DEPTH - 1, fill_slot);
    fill_slot = (fill_slot + 1 == DEPTH) ? 0 : fill_slot + 1;
    stage_off = (stage_off + kWarpStageBytes == DEPTH * kWarpStageBytes) ? 0 : stage_off + kWarpStageBytes;
    const int pg0 = (warp + i * NW) * 2;
    if (pg0 + 1 < n_here && sm_ntok[pg0] == kPage && sm_ntok[pg0 + 1] == kPage) {
      // two whole pages (all but the last stage of a sequence): nothing to mask
      if (own_a) {
        float* const o = out_a + pg0 * kPage;
        o[0] = res[0][0];
        o[kPage] = res[1][0];
        if (own_b) {
          o[p.stride] = res[0][1];
          o[p.stride + kPage] = res[1][1];
        }
      }
    } else if (own_a) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int pg = pg0 + mt;
        if (pg < n_here) {
          const bool live = tk_own < sm_ntok[pg];  // 0 tokens for a page whose table entry was out of range
          float* const o = out_a + pg * kPage;
          o[0] = live ? res[mt][0] : -INFINITY;
          if (own_b) o[p.stride] = live ? res[mt][1] : -INFINITY;
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <typename T, int G, int NW, int DEPTH, int NBLK>
static int launch_two_tiles(const EstParams& p, int rows, int max_row_pages, cudaStream_t st) {
  constexpr int kBytes = NW * DEPTH * kWarpStageBytes;
  auto kern = estimate_int4_imma_group_kernel<T, G, NW, DEPTH, NBLK>;
  TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
  dim3 grid((max_row_pages + NW * 16 - 1) / (NW * 16), rows);
  TWL_CUDA_TRY(launch_chain(kern, grid, dim3(NW * 32), kBytes, st, p));
  return TWL_OK;
}

template <typename T, int G, int NW, int DEPTH, int NBLK>
static int launch_digits(const EstParams& p, int rows, int max_row_pages, cudaStream_t st) {
  constexpr int kBytes = NW * DEPTH * kWarpStageBytes;
  auto kern = estimate_int4_imma_digits_kernel<T, G, NW, DEPTH, NBLK>;
  TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
  dim3 grid((max_row_pages + NW * 16 - 1) / (NW * 16), rows);
  TWL_CUDA_TRY(launch_chain(kern, grid, dim3(NW * 32), kBytes, st, p));
  return TWL_OK;
}

template <typename T, int G, int VARIANT>
static int launch_one(const EstParams& p, int rows, int max_row_pages, bool ldg, cudaStream_t st) {
  if (rows > 65535) return TWL_ERR_TOO_LARGE;
  if (ldg) {
    dim3 grid((max_row_pages + kPagesPerBlock - 1) / kPagesPerBlock, rows);
    estimate_int4_kernel<T, G, VARIANT><<<grid, kEstThreads, 0, st>>>(p);
  } else if (G > 1 && G <= 4 && VARIANT == VAR_DP4A && !p.force_ring && !p.simt_group && !p.f16_tiles && !p.two_tiles) {
    // Block shape: the kernel wants warps, not ring depth.  Config 2 (856 MB of slabs, 2048 rows), warps x ring
    // stages x blocks per SM: 8 x 5 x 2 (16 warps per SM, 110 registers) 178.5 us; 4 x 5 x 4 170.4; 10 x 4 x 2
    // 185.2; 12 x 3 x 2 168.2; 8 x 3 x 3 (24 warps, 80 registers) 163.8-165.8; 2 x 3 x 12 162.9; 4 x 3 x 6 162.5;
    // 8 x 2 x 4 and 4 x 2 x 8 (32 warps, 64 registers, spills) 182.4 / 177.8.
    // TWL_EST_DIGITS_SHAPE = 1..4 picks one of the others, for measurement.
    constexpr int GG = (G > 1 && G <= 4) ? G : 2;
    static const int shape = [] { const char* e = getenv("TWL_EST_DIGITS_SHAPE"); return e ? atoi(e) : 0; }();
    int rc = TWL_OK;
    switch (shape) {
      case 1: rc = launch_digits<T, GG, 8, 5, 2>(p, rows, max_row_pages, st); break;
      case 2: rc = launch_digits<T, GG, 8, 3, 3>(p, rows, max_row_pages, st); break;
      case 3: rc = launch_digits<T, GG, 2, 3, 12>(p, rows, max_row_pages, st); break;
      case 4: rc = launch_digits<T, GG, 4, 5, 4>(p, rows, max_row_pages, st); break;
      default: rc = launch_digits<T, GG, 4, 3, 6>(p, rows, max_row_pages, st); break;
    }
    if (rc != TWL_OK) return rc;
  } else if (G > 1 && VARIANT == VAR_DP4A && !p.force_ring && !p.simt_group && !p.f16_tiles) {
    // Block shape (warps x ring stages x blocks per SM), 64 sequences x 8 KV heads x 8 query heads, 856 MB of
    // slabs: 8 x 5 x 2 (113 registers) 205 us; 8 x 3 x 3 and 4 x 3 x 6 (80 registers) 203 / 199; 4 x 4 x 5
    // (96 registers, 20 warps per SM) 191.  Groups of 8 run the last one; the smaller groups, which reach this
    // kernel only as a measurement variant, keep the shape their profile was taken with.
    // TWL_EST_TILES_SHAPE = 1..4 picks a shape, for measurement.
    constexpr int GG = G > 1 ? G : 2;
    static const int shape = [] { const char* e = getenv("TWL_EST_TILES_SHAPE"); return e ? atoi(e) : 0; }();
    int rc = TWL_OK;
    switch (shape != 0 ? shape : (GG == 8 ? 3 : 4)) {
      case 1: rc = launch_two_tiles<T, GG, 8, 3, 3>(p, rows, max_row_pages, st); break;
      case 2: rc = launch_two_tiles<T, GG, 4, 3, 6>(p, rows, max_row_pages, st); break;
      case 3: rc = launch_two_tiles<T, GG, 4, 4, 5>(p, rows, max_row_pages, st); break;
      default: rc = launch_two_tiles<T, GG, 8, 5, 2>(p, rows, max_row_pages, st); break;
    }
    if (rc != TWL_OK) return rc;
  } else if (G > 1 && VARIANT == VAR_DP4A && !p.force_ring && !p.simt_group) {
    constexpr int kBytes = kEstWarps * kRingDepth * kWarpStageBytes;
    auto kern = estimate_int4_mma_group_kernel<T, (G > 1 ? G : 2)>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    dim3 grid((max_row_pages + kWarpPagesPerBlock - 1) / kWarpPagesPerBlock, rows);
    TWL_CUDA_TRY(launch_chain(kern, grid, dim3(kEstThreads), kBytes, st, p));
  } else if (G > 1 && VARIANT == VAR_DP4A && !p.force_ring) {
    constexpr int kBytes = kEstWarps * kRingDepth * kWarpStageBytes;
    auto kern = estimate_int4_warp_group_kernel<T, G>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    dim3 grid((max_row_pages + kWarpPagesPerBlock - 1) / kWarpPagesPerBlock, rows);
    TWL_CUDA_TRY(launch_chain(kern, grid, dim3(kEstThreads), kBytes, st, p));
  } else if (G == 1 && p.bulk_warp) {
    // warp-private rings fed by bulk copies: the same block shape and bytes in flight as the default
    constexpr int kWarps = 2, kPages = 32;
    constexpr int kBytes = kWarps * kRingDepth * kWarpStageBytes;
    dim3 grid((max_row_pages + kPages - 1) / kPages, rows);
    auto kern = estimate_int4_bulk_warp_kernel<T, VARIANT, kWarps, kRingDepth, kPages>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    TWL_CUDA_TRY(launch_chain(kern, grid, dim3(kWarps * 32), kBytes, st, p));
  } else if (G == 1 && !p.force_ring) {
    // Small blocks: 16 warps and the same bytes in flight per SM whatever the block size, but the
    // blocks' set-up phases spread out more.  Per step of config 1: 8 warps x 128 pages 5.45 ms,
    // 4 x 64 5.38, 2 x 32 5.32, 1 x 16 5.34 (16 pages = 8 ring stages per warp in every case).
    constexpr int kWarps = 2, kPages = 32;
    constexpr int kBytes = kWarps * kRingDepth * kWarpStageBytes;
    dim3 grid((max_row_pages + kPages - 1) / kPages, rows);
    auto kern = estimate_int4_warp_kernel<T, VARIANT, kWarps, kRingDepth, kPages>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    TWL_CUDA_TRY(launch_chain(kern, grid, dim3(kWarps * 32), kBytes, st, p));
  } else {
    constexpr int kRingBytes = kStages * kStagePages * kSlab;
    auto kern = estimate_int4_tma_kernel<T, G, VARIANT>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes));
    dim3 grid((max_row_pages + p.pages_per_block - 1) / p.pages_per_block, rows);
    kern<<<grid, kTmaThreads, kRingBytes, st>>>(p);
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

template <typename T, int VARIANT>
static int launch_variant(const EstParams& p, bool has_cand, int max_row_pages, bool ldg,
                          cudaStream_t st) {
  if (has_cand) return launch_one<T, 1, VARIANT>(p, p.B * p.Hq, max_row_pages, ldg, st);
  const int g = p.Hq / p.Hkv;
  switch (g) {
    case 1: return launch_one<T, 1, VARIANT>(p, p.B * p.Hkv, max_row_pages, ldg, st);
    case 2: return launch_one<T, 2, VARIANT>(p, p.B * p.Hkv, max_row_pages, ldg, st);
    case 4: return launch_one<T, 4, VARIANT>(p, p.B * p.Hkv, max_row_pages, ldg, st);
    case 8: return launch_one<T, 8, VARIANT>(p, p.B * p.Hkv, max_row_pages, ldg, st);
    default: return TWL_ERR_UNSUPPORTED;
  }
}

template <typename T>
static int launch_dtype(const EstParams& p, bool has_cand, int max_row_pages, int variant,
                        cudaStream_t st) {
  // +16: direct global loads; +128: the block-wide bulk-copy ring even for a single query head
  const_cast<EstParams&>(p).force_ring = (variant & 128) != 0;
  const_cast<EstParams&>(p).simt_group = (variant & 32) != 0;  // +32: integer-dot kernel for query-head groups
  const_cast<EstParams&>(p).bulk_warp = (variant & 64) != 0;   // +64: warp-private rings fed by bulk copies
  const_cast<EstParams&>(p).f16_tiles = (variant & 256) != 0;  // +256: 16-bit float tiles for query-head groups
  const_cast<EstParams&>(p).two_tiles = (variant & 512) != 0;  // +512: hi and lo digits in two integer tiles even for groups of 2 or 4
  const bool ldg = (variant & 16) != 0;
  switch (variant & 15) {
    case VAR_F32: return launch_variant<T, VAR_F32>(p, has_cand, max_row_pages, ldg, st);
    case VAR_H2: return launch_variant<T, VAR_H2>(p, has_cand, max_row_pages, ldg, st);
    case 0:
    case VAR_DP4A: return launch_variant<T, VAR_DP4A>(p, has_cand, max_row_pages, ldg, st);
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
  p.pages_per_block = kTmaPagesPerBlockDefault;  // of the bulk-copy ring variant
  // rows never hold more pages than the score row has room for
  const int max_row_pages = has_cand ? max_k : score_stride / kPage;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) return launch_dtype<__half>(p, has_cand, max_row_pages, variant, st);
  if (dtype == TWL_BF16) return launch_dtype<__nv_bfloat16>(p, has_cand, max_row_pages, variant, st);
  return TWL_ERR_UNSUPPORTED;
}
