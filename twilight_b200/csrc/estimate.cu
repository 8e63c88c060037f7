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
constexpr int kTmaPagesPerBlock = 128;               // 160 KiB of INT4 cache per block
constexpr int kTmaThreads = kEstThreads + 32;        // 8 consumer warps + 1 producer warp
constexpr uint32_t kWaitLimit = 1u << 22;

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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
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
  __shared__ int sm_phys[kTmaPagesPerBlock];
  __shared__ int sm_ntok[kTmaPagesPerBlock];
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
  const int first = blockIdx.x * kTmaPagesPerBlock;
  if (first >= n_pages) return;
  const int n_here = min(kTmaPagesPerBlock, n_pages - first);
  const int n_stages_total = (n_here + kStagePages - 1) / kStagePages;

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
  } else if (tid >= kEstThreads - 4 * G && tid < kEstThreads) {
    const int j = tid - (kEstThreads - 4 * G);
    const int g = j >> 2, grp_j = j & 3;
    float qf[32];
    load_q_group<T>(reinterpret_cast<const T*>(p.q) + ((size_t)(b * p.Hq + h0 + g)) * kD + grp_j * kGroup, qf);
    sm_q[g][grp_j].init(qf);
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
      if (!ok) {
        raise_flag(p.status, TWL_FLAG_WAIT_LIMIT);
        // drain: every stage issued so far completes its transaction count sooner or later
        for (int st = max(0, issued - kStages); st < issued; ++st)
          mbar_wait(&sm_full[st % kStages], (st / kStages) & 1);
      }
    }
    return;
  }

  // ---- consumers ----
  const int grp = lane & 3, tok_in_step = lane >> 2;
  QRegs<VARIANT> qr[G];
#pragma unroll
  for (int g = 0; g < G; ++g) qr[g] = sm_q[g][grp];

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
      const int slot_out = (first + pg) * kPage + half * 8 + tok_in_step;
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
          p.scores[(size_t)(b * p.Hq + h0 + g) * p.stride + slot_out] = v;
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm_empty[slot]);
  }
}

template <typename T, int G, int VARIANT>
static int launch_one(const EstParams& p, int rows, int max_row_pages, bool ldg, cudaStream_t st) {
  if (rows > 65535) return TWL_ERR_TOO_LARGE;
  if (ldg) {
    dim3 grid((max_row_pages + kPagesPerBlock - 1) / kPagesPerBlock, rows);
    estimate_int4_kernel<T, G, VARIANT><<<grid, kEstThreads, 0, st>>>(p);
  } else {
    constexpr int kRingBytes = kStages * kStagePages * kSlab;
    auto kern = estimate_int4_tma_kernel<T, G, VARIANT>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes));
    dim3 grid((max_row_pages + kTmaPagesPerBlock - 1) / kTmaPagesPerBlock, rows);
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
  const bool ldg = (variant & 16) != 0;  // +16: direct global loads instead of the staged ring
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
  // rows never hold more pages than the score row has room for
  const int max_row_pages = has_cand ? max_k : score_stride / kPage;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) return launch_dtype<__half>(p, has_cand, max_row_pages, variant, st);
  if (dtype == TWL_BF16) return launch_dtype<__nv_bfloat16>(p, has_cand, max_row_pages, variant, st);
  return TWL_ERR_UNSUPPORTED;
}
