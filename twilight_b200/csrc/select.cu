// Selector: Quest page scores from stored (min,max) page metadata, then top-k pages.
//
// Stands in for quest_selector of twilight/pyimpl/quest.py:17-122.  The reference rebuilds
// the per-page channel maxima of sign(q)*K from the whole K cache on every step
// (quest.py:37-74); here the channel-wise min and max of every page are kept as metadata and
//   score(page) = sum_d max(q_d*kmax_d, q_d*kmin_d)            (== |q| . max_t sign(q)*K_t)
// is evaluated in fp32.  The page count kept is quest.py:93-98; ties at the last kept score
// go to the lower page number (torch.topk, quest.py:99, leaves them unspecified).
#include <cstdlib>

#include "common.cuh"

namespace twl {

constexpr int kSelThreads = 256;
constexpr int kSelPagesPerBlock = 256;  // 128 KiB of metadata per block (64 / 128 / 512 pages: 103 / 95 / 96 us against 91 us on config 1)

struct ScoreParams {
  const void* q;
  const void* kmeta;
  const int32_t* indptr;
  const int32_t* indices;
  float* page_scores;
  int32_t* status;
  int B, Hq, Hkv, num_pages_total, max_pages;
  // fused selection (counters != nullptr): the block that finishes a row's scores last also
  // picks the row's best pages
  int32_t* counters;     // [B*Hkv], zero on entry, left zero
  int32_t* cand_pages;   // [B][Hq][max_k]
  int32_t* cand_npages;  // [B][Hq]
  int token_budget, max_k;
};

struct TopkScratch {
  int hist[256];
  int wsum[33];
  uint32_t prefix;
  int krem;
};
__device__ void topk_row(const float* src, int n, int k, int32_t* out, uint32_t* keys, TopkScratch& sc);

// Eight lanes share a page: lane `sub` reads 16-byte pieces sub and sub+8 of the 256-byte min
// row and of the max row (channels 8*sub..8*sub+7 and 64+8*sub..), so a warp step covers four
// pages = 2 KiB contiguous per page pair of rows.  G query heads share the loaded metadata.
// A single head per row is all loads: five blocks per SM (48 registers) beat four (56) and six (42)
// by 1-2 %.
template <typename T, int G>
__global__ void __launch_bounds__(kSelThreads, G == 1 ? 5 : 1)
quest_page_scores_kernel(const ScoreParams p) {
  // blocks that run side by side take the same pages of different KV heads: their 512-byte slabs
  // are neighbours inside one 512*H_kv-byte page record, which keeps DRAM rows open
  const int row = blockIdx.x;  // (b, kv head), kv head fastest
  const int b = row / p.Hkv, kvh = row % p.Hkv;
  // This is the first kernel of a layer pass: q and the page table may have been written by the
  // kernel launched just before it (a projection, a cache append), so nothing is read before the
  // wait.  Every block waits, so that this grid never completes before the one before it.
  pdl_wait();
  const int page_base = p.indptr[b];
  const int n_pages = min(p.indptr[b + 1] - page_base, p.max_pages);
  const int first = blockIdx.y * kSelPagesPerBlock;
  if (first >= n_pages) {
    if (p.counters != nullptr && n_pages <= 0 && blockIdx.y == 0 && threadIdx.x < G)
      p.cand_npages[b * p.Hq + kvh * G + threadIdx.x] = 0;
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, pg_in_step = lane >> 3;
  const int h0 = kvh * G;

  // Query heads of the group: in registers for small groups; for 4 or more heads the registers
  // would cost too much occupancy, so q (as fp32) sits in shared memory and each head's 16 values
  // are fetched per page with four 128-bit loads (the 8 lanes of a page read 8 distinct pieces).
  constexpr bool kQInSmem = G > 2;
  __shared__ __align__(16) float sm_qf[kQInSmem ? G : 1][kD];
  float qf[kQInSmem ? 1 : G][16];
  if (kQInSmem) {
    for (int i = threadIdx.x; i < G * kD; i += kSelThreads)
      sm_qf[i / kD][i % kD] = Elem<T>::to_f(reinterpret_cast<const T*>(p.q)[(size_t)(b * p.Hq + h0) * kD + i]);
  } else {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)(b * p.Hq + h0 + g) * kD;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow) + sub + 8 * part);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = Elem<T>::to_f2(u[k]);
          qf[g][8 * part + 2 * k] = f.x;
          qf[g][8 * part + 2 * k + 1] = f.y;
        }
      }
    }
  }

  // physical page ids of the block's pages go to shared memory first, so that the streaming loop
  // has no dependent index loads
  __shared__ int sm_phys[kSelPagesPerBlock];
  const int n_here = min(kSelPagesPerBlock, n_pages - first);
  for (int i = threadIdx.x; i < kSelPagesPerBlock; i += kSelThreads) {
    int phys = -1;
    if (i < n_here) {
      phys = p.indices[page_base + first + i];
      if (phys < 0 || phys >= p.num_pages_total) {
        phys = -1;
        raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      }
    }
    sm_phys[i] = phys;
  }
  __syncthreads();

  if constexpr (kQInSmem) {
    // A warp takes four pages per step (8 lanes per page), 32 pages apart from its next step.
    // With a group in shared memory the shared-memory reads of q bound the kernel (four 16-byte
    // reads per head and step: 65 % of the shared-memory pipe at G = 8), so two steps are loaded
    // together and every q vector that is fetched is used for both.
    constexpr int kStep = (kSelThreads / 32) * 4;
    constexpr int kPair = 2;
    for (int l0 = warp * 4; l0 < n_here; l0 += kPair * kStep) {
      uint4 mn[kPair][2], mx[kPair][2];
      bool ok[kPair], live[kPair];
#pragma unroll
      for (int u = 0; u < kPair; ++u) {
        const int l = l0 + u * kStep + pg_in_step;
        live[u] = l < n_here;
        const int phys = live[u] ? sm_phys[l] : -1;
        ok[u] = phys >= 0;
        if (ok[u]) {
          const T* slab = reinterpret_cast<const T*>(p.kmeta) + ((size_t)phys * p.Hkv + kvh) * 2 * kD;
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            mn[u][part] = ldg_stream_u4(reinterpret_cast<const uint4*>(slab) + sub + 8 * part);
            mx[u][part] = ldg_stream_u4(reinterpret_cast<const uint4*>(slab + kD) + sub + 8 * part);
          }
        }
      }
      // per channel {centre, half-width} of the page's range: max(q*hi, q*lo) =
      // q*(hi+lo)/2 + |q|*(hi-lo)/2 for hi >= lo, i.e. two FMAs per head instead of two products,
      // a max and an add
      float va[kPair][16], vb[kPair][16];
#pragma unroll
      for (int u = 0; u < kPair; ++u) {
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          const uint32_t un[4] = {mn[u][part].x, mn[u][part].y, mn[u][part].z, mn[u][part].w};
          const uint32_t ux[4] = {mx[u][part].x, mx[u][part].y, mx[u][part].z, mx[u][part].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 lo = ok[u] ? Elem<T>::to_f2(un[k]) : make_float2(0.f, 0.f);
            const float2 hi = ok[u] ? Elem<T>::to_f2(ux[k]) : make_float2(0.f, 0.f);
            va[u][8 * part + 2 * k] = 0.5f * (hi.x + lo.x); va[u][8 * part + 2 * k + 1] = 0.5f * (hi.y + lo.y);
            vb[u][8 * part + 2 * k] = 0.5f * (hi.x - lo.x); vb[u][8 * part + 2 * k + 1] = 0.5f * (hi.y - lo.y);
          }
        }
      }
      float acc[kPair][G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float qv[16];
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          const float4 a = *reinterpret_cast<const float4*>(&sm_qf[g][64 * part + 8 * sub]);
          const float4 c = *reinterpret_cast<const float4*>(&sm_qf[g][64 * part + 8 * sub + 4]);
          qv[8 * part + 0] = a.x; qv[8 * part + 1] = a.y; qv[8 * part + 2] = a.z; qv[8 * part + 3] = a.w;
          qv[8 * part + 4] = c.x; qv[8 * part + 5] = c.y; qv[8 * part + 6] = c.z; qv[8 * part + 7] = c.w;
        }
#pragma unroll
        for (int u = 0; u < kPair; ++u) {
          float t = 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            t = fmaf(qv[i], va[u][i], t);
            t = fmaf(fabsf(qv[i]), vb[u][i], t);
          }
          acc[u][g] = t;
        }
      }
#pragma unroll
      for (int u = 0; u < kPair; ++u) {
        const int lp = first + l0 + u * kStep + pg_in_step;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float t = acc[u][g];
          t += __shfl_xor_sync(0xffffffffu, t, 1);
          t += __shfl_xor_sync(0xffffffffu, t, 2);
          t += __shfl_xor_sync(0xffffffffu, t, 4);
          if (live[u] && (g & 7) == sub)
            p.page_scores[(size_t)(b * p.Hq + h0 + g) * p.max_pages + lp] = ok[u] ? t : -INFINITY;
        }
      }
    }
  } else {
    constexpr int kU = 1;  // page quads in flight per warp (2 was measured slower)
    for (int l0 = warp * 4; l0 < n_here; l0 += (kSelThreads / 32) * 4 * kU) {
      uint4 mn[kU][2], mx[kU][2];
      bool ok[kU], live[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int l = l0 + u * (kSelThreads / 32) * 4 + pg_in_step;
        live[u] = l < n_here;
        const int phys = live[u] ? sm_phys[l] : -1;
        ok[u] = phys >= 0;
        if (ok[u]) {
          const T* slab = reinterpret_cast<const T*>(p.kmeta) + ((size_t)phys * p.Hkv + kvh) * 2 * kD;
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            mn[u][part] = ldg_stream_u4(reinterpret_cast<const uint4*>(slab) + sub + 8 * part);
            mx[u][part] = ldg_stream_u4(reinterpret_cast<const uint4*>(slab + kD) + sub + 8 * part);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int lp = first + l0 + u * (kSelThreads / 32) * 4 + pg_in_step;
        float acc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) acc[g] = 0.f;
        if (ok[u]) {
          float lo16[16], hi16[16];
#pragma unroll
          for (int part = 0; part < 2; ++part) {
            const uint32_t un[4] = {mn[u][part].x, mn[u][part].y, mn[u][part].z, mn[u][part].w};
            const uint32_t ux[4] = {mx[u][part].x, mx[u][part].y, mx[u][part].z, mx[u][part].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 lo = Elem<T>::to_f2(un[k]), hi = Elem<T>::to_f2(ux[k]);
              lo16[8 * part + 2 * k] = lo.x; lo16[8 * part + 2 * k + 1] = lo.y;
              hi16[8 * part + 2 * k] = hi.x; hi16[8 * part + 2 * k + 1] = hi.y;
            }
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float qv[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) qv[i] = qf[g][i];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[g] += fmaxf(qv[i] * hi16[i], qv[i] * lo16[i]);
          }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 1);
          acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 2);
          acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], 4);
          if (live[u] && (g & 7) == sub)
            p.page_scores[(size_t)(b * p.Hq + h0 + g) * p.max_pages + lp] = ok[u] ? acc[g] : -INFINITY;
        }
      }
    }
  }
  if (p.counters == nullptr) return;
  // ---- fused selection: last block of the row to arrive (ticket; nobody waits) ----
  extern __shared__ __align__(16) uint32_t dyn_keys[];  // max_pages keys
  __shared__ TopkScratch sc;
  __shared__ int sm_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int n_blocks = (n_pages + kSelPagesPerBlock - 1) / kSelPagesPerBlock;
    const int ticket = atomicAdd(&p.counters[row], 1);
    sm_last = (ticket == n_blocks - 1);
    if (sm_last) p.counters[row] = 0;  // ready for the next call
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  int k = max(1, p.token_budget / kPage) + ((p.token_budget % kPage) != 0 ? 1 : 0);  // quest.py:93-95
  k = min(min(k, n_pages), p.max_k);                                                 // quest.py:98
  for (int g = 0; g < G; ++g) {
    const int qrow = b * p.Hq + h0 + g;
    int32_t* out = p.cand_pages + (size_t)qrow * p.max_k;
    if (threadIdx.x == 0) p.cand_npages[qrow] = k;
    if (k == n_pages) {
      for (int i = threadIdx.x; i < n_pages; i += kSelThreads) out[i] = i;
    } else if (k > 0) {
      topk_row(p.page_scores + (size_t)qrow * p.max_pages, n_pages, k, out, dyn_keys, sc);
    }
  }
}

// ---- query-head groups of 4 or 8: the scores as a tensor-core contraction -----------------------
// sum_d max(q_d*hi_d, q_d*lo_d) = sum_d (min(q_d,0)*lo_d + max(q_d,0)*hi_d) because hi >= lo, i.e.
//   score[page][head] = sum_k A[page][k] * B[k][head],   k = 0..255,
// where row `page` of A is the 512-byte metadata slab exactly as it lies in memory ([min | max],
// model dtype) and B = [min(q,0) ; max(q,0)] is exact in the model dtype.  A warp takes 16 pages
// per step: lane 4*g + t reads the 16-byte pieces t, t+4, .., t+28 of the slabs of pages g and g+8
// straight into the A fragments of sixteen m16n8k16 tiles (two per piece) (the channel-to-slot assignment this
// gives is applied to B as well), accumulates in fp32 and owns the scores of pages g, g+8 for
// heads 2t, 2t+1.  With four heads the upper four columns of B are zero.
// NW warps per block, PPB pages per block: a warp should stream many steps per block it belongs
// to, because a block's set-up (page table look-ups, a barrier) moves no metadata.
// PIPE: two steps of loads in flight per warp instead of one (193 registers instead of 120).
// HPB: KV heads per block.  With HPB > 1 the block's warps take HPB neighbouring KV heads of the same
// pages (warp w: head w % HPB), so the HPB slabs of a page record - HPB * 512 contiguous bytes - are
// fetched by one SM at about the same time.  Scattered 512-byte reads over a metadata array of a
// gigabyte or more are bound by address translation, not by DRAM (128 sequences x 4096 shuffled pages x
// 4 KV heads, 1.07 GB: 344 us against 170 us with consecutive physical pages, while the same bytes
// as four launches over 268 MB arrays take 4 x 50 us); sharing a page record among the warps of a
// block divides the translations per byte by HPB.
template <typename T, int G, int NW, int PPB, bool PIPE, int HPB = 1>
__global__ void __launch_bounds__(NW * 32, (PIPE ? 256 : 512) / (NW * 32))
quest_page_scores_mma_kernel(const ScoreParams p) {
  static_assert(G == 4 || G == 8, "one n8 tile holds the group");
  static_assert(NW % HPB == 0, "whole warps per KV head");
  constexpr int kThreads = NW * 32;
  const int row = blockIdx.x;  // (b, group of HPB kv heads), kv heads fastest
  const int b = row / (p.Hkv / HPB);
  const int kvh = (row % (p.Hkv / HPB)) * HPB + (int)(threadIdx.x >> 5) % HPB;
  pdl_wait();  // q and the page table may come from the kernel launched just before
  const int page_base = p.indptr[b];
  const int n_pages = min(p.indptr[b + 1] - page_base, p.max_pages);
  const int first = blockIdx.y * PPB;
  if (first >= n_pages) return;
  const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) / HPB;  // this head's warps: 0 .. NW / HPB - 1
  const int g = lane >> 2, t = lane & 3;
  const int h0 = kvh * G;

  // B fragments of head g.  The slab is 32 pieces of 16 bytes (16 of minima, 16 of maxima); this
  // lane holds pieces t, t+4, .., t+28 of it, so its B pieces are those of [min(q,0) | max(q,0)]
  uint32_t bq[8][4];
  {
    const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)(b * p.Hq + h0 + (g < G ? g : 0)) * kD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow) + 4 * c + t);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // a 16-bit float is negative iff its sign bit is set; -0 and +0 both give a zero product
        const uint32_t lo_neg = (u[k] & 0x00008000u) ? 0x0000ffffu : 0u;
        const uint32_t hi_neg = (u[k] & 0x80000000u) ? 0xffff0000u : 0u;
        const uint32_t neg = lo_neg | hi_neg;
        bq[c][k] = (g < G) ? (u[k] & neg) : 0u;       // min(q,0): pairs with the page minima
        bq[4 + c][k] = (g < G) ? (u[k] & ~neg) : 0u;  // max(q,0): pairs with the page maxima
      }
    }
  }

  __shared__ int sm_phys[PPB];
  const int n_here = min(PPB, n_pages - first);
  for (int i = threadIdx.x; i < PPB; i += kThreads) {
    int phys = -1;
    if (i < n_here) {
      phys = p.indices[page_base + first + i];
      if (phys < 0 || phys >= p.num_pages_total) {
        phys = -1;
        raise_flag(p.status, TWL_FLAG_BAD_INDEX);
      }
    }
    sm_phys[i] = phys;
  }
  __syncthreads();

  const uint4* const meta16 = reinterpret_cast<const uint4*>(p.kmeta);
  const size_t slab16 = 2 * kD * sizeof(T) / 16;  // 32 pieces per (page, kv-head) slab
  struct Step {
    uint4 va[8], vb[8];
    int pa, pb;
  };
  auto load_step = [&](Step& s, int l0) {
    const int la = l0 + g, lb = l0 + g + 8;
    s.pa = la < n_here ? sm_phys[la] : -1;
    s.pb = lb < n_here ? sm_phys[lb] : -1;
    // absent pages read the slab of physical page 0 (always mapped); their scores are not used
    const uint4* sa = meta16 + ((size_t)max(s.pa, 0) * p.Hkv + kvh) * slab16 + t;
    const uint4* sb = meta16 + ((size_t)max(s.pb, 0) * p.Hkv + kvh) * slab16 + t;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      s.va[c] = ldg_stream_u4(sa + 4 * c);
      s.vb[c] = ldg_stream_u4(sb + 4 * c);
    }
  };
  auto finish_step = [&](const Step& s, int l0) {
    const int la = l0 + g, lb = l0 + g + 8;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      MmaTile<T>::run(acc, s.va[c].x, s.vb[c].x, s.va[c].y, s.vb[c].y, bq[c][0], bq[c][1]);
      MmaTile<T>::run(acc, s.va[c].z, s.vb[c].z, s.va[c].w, s.vb[c].w, bq[c][2], bq[c][3]);
    }
    if (2 * t < G) {
      float* const o0 = p.page_scores + (size_t)(b * p.Hq + h0 + 2 * t) * p.max_pages + first;
      float* const o1 = o0 + p.max_pages;
      if (la < n_here) {
        o0[la] = s.pa >= 0 ? acc[0] : -INFINITY;
        o1[la] = s.pa >= 0 ? acc[1] : -INFINITY;
      }
      if (lb < n_here) {
        o0[lb] = s.pb >= 0 ? acc[2] : -INFINITY;
        o1[lb] = s.pb >= 0 ? acc[3] : -INFINITY;
      }
    }
  };
  constexpr int kStride = (NW / HPB) * 16;
  if constexpr (PIPE) {
    // two register sets: the loads of the next step are in flight while this one is multiplied
    Step s0, s1;
    int l0 = warp * 16;
    if (l0 < n_here) load_step(s0, l0);
    while (l0 < n_here) {
      const int l1 = l0 + kStride, l2 = l1 + kStride;
      if (l1 < n_here) load_step(s1, l1);
      finish_step(s0, l0);
      if (l2 < n_here) load_step(s0, l2);
      if (l1 < n_here) finish_step(s1, l1);
      l0 = l2;
    }
  } else {
    for (int l0 = warp * 16; l0 < n_here; l0 += kStride) {
      Step s0;
      load_step(s0, l0);
      finish_step(s0, l0);
    }
  }
}

// ---- top-k pages of one (batch, query head) row ---------------------------------------------
__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  if (u == 0x80000000u) u = 0u;  // -0 ties with +0, as it does for a comparison of the floats
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float <=> larger key
}

constexpr int kTopkThreads = 256;
static_assert(kTopkThreads == kSelThreads, "the fused tail runs the selection with the scoring block");

// Keeps the k best of src[0..n) (k < n) and writes their positions, ascending, to out[0..k).
// Called by a whole block of kTopkThreads threads; keys: n words of shared memory.  Scores are
// read through L2 because other blocks may have written them.
__device__ void topk_row(const float* src, int n, int k, int32_t* out, uint32_t* keys, TopkScratch& sc) {
  int (&hist)[256] = sc.hist;
  int (&wsum)[33] = sc.wsum;
  uint32_t& sh_prefix = sc.prefix;
  int& sh_krem = sc.krem;
  // keys, and the smallest and the largest of them: the leading bits they share need no pass
  uint32_t kmin = 0xFFFFFFFFu, kmax = 0u;
  for (int i = threadIdx.x; i < n; i += kTopkThreads) {
    const uint32_t key = order_key(__ldcg(src + i));
    keys[i] = key;
    kmin = min(kmin, key);
    kmax = max(kmax, key);
  }
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  if ((threadIdx.x & 31) == 0) {
    wsum[threadIdx.x >> 5] = (int)kmin;
    wsum[8 + (threadIdx.x >> 5)] = (int)kmax;
  }
  __syncthreads();
  {
    constexpr int kW = kTopkThreads / 32;
    const int lane = threadIdx.x & 31;
    kmin = __reduce_min_sync(0xffffffffu, lane < kW ? (uint32_t)wsum[lane] : 0xFFFFFFFFu);
    kmax = __reduce_max_sync(0xffffffffu, lane < kW ? (uint32_t)wsum[8 + lane] : 0u);
  }
  // MSB-first radix select of the k-th largest key, up to 8 bits per pass, starting below the
  // leading bits that all keys share (page scores of one row often lie within a few octaves: the
  // sign and most exponent bits are common then, and the select takes three passes instead of four;
  // 25.1 -> 22.9 us on 1024 rows x 4096 pages)
  int top = 32 - __clz(kmin ^ kmax);  // bits still undetermined: keys agree above bit `top`
  if (threadIdx.x == 0) {
    sh_prefix = top < 32 ? (kmax >> top) << top : 0u;
    sh_krem = k;
  }
  __syncthreads();  // wsum is free again; prefix and krem are set
  while (top > 0) {
    const int width = min(8, top), shift = top - width;
    const uint32_t mask = top < 32 ? 0xFFFFFFFFu << top : 0u, dmask = (1u << width) - 1u;
    hist[threadIdx.x] = 0;  // kTopkThreads == 256 bins
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    // (plain per-lane adds: letting a warp whose keys share a bin add once - by a vote, or by
    // __match_any_sync groups - was slower, 14.8 and 18.8 against 12.7 us on 512 rows x 2048 pages)
    for (int i = threadIdx.x; i < n; i += kTopkThreads) {
      const uint32_t key = keys[i];
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & dmask], 1);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // lane l owns bins 255-8l .. 248-8l (descending); find where the running count reaches k
      const int lane = threadIdx.x;
      const int krem = sh_krem;  // read by every lane before the scan's shuffles, written after
      int local = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) local += hist[255 - 8 * lane - j];
      int inc = local;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      const int before = inc - local;
      if (before < krem && krem <= inc) {
        int run = before;
        for (int j = 0; j < 8; ++j) {
          const int bin = 255 - 8 * lane - j;
          if (run + hist[bin] >= krem) {
            sh_prefix = prefix | ((uint32_t)bin << shift);
            sh_krem = krem - run;
            break;
          }
          run += hist[bin];
        }
      }
    }
    top = shift;
    __syncthreads();
  }
  const uint32_t thr = sh_prefix;  // k-th largest key
  const int take_eq = sh_krem;     // how many keys equal to it are kept (lowest pages first)
  // ordered compaction, 4 consecutive pages per thread per tile
  int base_gt = 0, base_eq = 0;
  for (int t0 = 0; t0 < n; t0 += kTopkThreads * 4) {
    const int i0 = t0 + threadIdx.x * 4;
    int gt[4], eq[4], cg = 0, ce = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool in = i0 + j < n;
      const uint32_t key = in ? keys[i0 + j] : 0u;
      gt[j] = in && key > thr;
      eq[j] = in && key == thr;
      cg += gt[j];
      ce += eq[j];
    }
    int total;
    const int packed = block_excl_scan<kTopkThreads>(cg | (ce << 16), &total, wsum);
    int ng = base_gt + (packed & 0xFFFF), ne = base_eq + (packed >> 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (gt[j]) {
        out[ng + min(ne, take_eq)] = i0 + j;
        ++ng;
      } else if (eq[j]) {
        if (ne < take_eq) out[ng + ne] = i0 + j;
        ++ne;
      }
    }
    base_gt += total & 0xFFFF;
    base_eq += total >> 16;
  }
}

struct TopkParams {
  const float* page_scores;
  const int32_t* indptr;
  int32_t* cand_pages;
  int32_t* cand_npages;
  int max_pages, Hq, token_budget, max_k;
};

__global__ void __launch_bounds__(kTopkThreads)
quest_topk_pages_kernel(const TopkParams p) {
  extern __shared__ __align__(16) uint32_t keys[];  // max_pages keys
  __shared__ TopkScratch sc;
  pdl_release();  // the estimator's blocks may move in and set up while this small grid works
  const int row = blockIdx.x, b = row / p.Hq;
  pdl_wait();  // the page scores come from the kernel launched just before; nothing is read earlier
  const int n = min(p.indptr[b + 1] - p.indptr[b], p.max_pages);
  int k = max(1, p.token_budget / kPage) + ((p.token_budget % kPage) != 0 ? 1 : 0);  // quest.py:93-95
  k = min(min(k, n), p.max_k);                                                       // quest.py:98
  int32_t* out = p.cand_pages + (size_t)row * p.max_k;
  if (threadIdx.x == 0) p.cand_npages[row] = k;
  if (k <= 0) return;
  if (k == n) {  // every page is kept
    for (int i = threadIdx.x; i < n; i += kTopkThreads) out[i] = i;
    return;
  }
  const float* page_scores = p.page_scores;
  const int max_pages = p.max_pages;
  topk_row(page_scores + (size_t)row * max_pages, n, k, out, keys, sc);
}

template <typename T, int G>
static int launch_scores(const ScoreParams& p, cudaStream_t st) {
  const int rows = p.B * p.Hkv;
  const int chunks = (p.max_pages + kSelPagesPerBlock - 1) / kSelPagesPerBlock;
  if (chunks > 65535) return TWL_ERR_TOO_LARGE;
  dim3 grid(rows, chunks);
  const size_t smem = p.counters ? (size_t)p.max_pages * sizeof(uint32_t) : 0;
  if (smem > 48 * 1024)
    TWL_CUDA_TRY(cudaFuncSetAttribute(quest_page_scores_kernel<T, G>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024 * 4));
  TWL_CUDA_TRY(launch_chain(quest_page_scores_kernel<T, G>, grid, dim3(kSelThreads), smem, st, p));
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

template <typename T, int G, int NW, int PPB, bool PIPE, int HPB = 1>
static int launch_scores_mma_shape(const ScoreParams& p, cudaStream_t st) {
  const int rows = p.B * (p.Hkv / HPB);
  const int chunks = (p.max_pages + PPB - 1) / PPB;
  if (chunks > 65535) return TWL_ERR_TOO_LARGE;
  TWL_CUDA_TRY(launch_chain(quest_page_scores_mma_kernel<T, G, NW, PPB, PIPE, HPB>, dim3(rows, chunks), dim3(NW * 32), 0, st, p));
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

template <typename T, int G>
static int launch_scores_mma(const ScoreParams& p, cudaStream_t st) {
  // Two warps per block, one step (8 KiB) of loads in flight per warp, 120 registers: eight blocks =
  // 16 warps per SM.  Measured on one KV head x 128 sequences x 4096 pages (268 MB of metadata,
  // 17 MB of scores written): 49.7 us with 256 pages per block, 51.8 with 512, 50.3 with four warps
  // x 512 pages, 51.6 with eight warps x 256 pages.  Two steps in flight per warp need 193
  // registers, so an SM holds half the warps: 55.6 us whatever the block shape (1, 2 or 8 warps x
  // 128..512 pages) - this kernel wants warps, not bytes in flight per warp.  Staging the slabs
  // through a shared-memory ring (whole-slab cp.async copies, ldmatrix fragments) was slower (60-68
  // us) and is not kept; neither is a one-wave grid whose blocks walk the (row, page run) items
  // (58.9 us with runs of 128 pages, 59.9 us with 256).  Pages per block: 256 while that still
  // fills the GPU once, else 128 so that small problems spread out.
  // TWL_SCORES_MMA_SHAPE (for measurement): 1 = 8 warps x 256 pages, 5 = 2 x 512, 6 = 4 x 512, all
  // with one step in flight; 7 = 2 x 512 with two steps in flight; 8 = one KV head per block even when
  // the GPU holds several.
  static const int forced = [] {
    const char* e = getenv("TWL_SCORES_MMA_SHAPE");
    return e ? atoi(e) : 0;
  }();
  if (forced == 1) return launch_scores_mma_shape<T, G, 8, 256, false>(p, st);
  if (forced == 5) return launch_scores_mma_shape<T, G, 2, 512, false>(p, st);
  if (forced == 6) return launch_scores_mma_shape<T, G, 4, 512, false>(p, st);
  if (forced == 7) return launch_scores_mma_shape<T, G, 2, 512, true>(p, st);
  // Several KV heads per GPU: the warps of a block take neighbouring heads of the same 128 pages (the same
  // 8 steps per warp as two warps sharing 256 pages).  TWL_SCORES_MMA_SHAPE=8 keeps one head per block.
  if (forced != 8) {
    if (p.Hkv % 4 == 0) return launch_scores_mma_shape<T, G, 4, 128, false, 4>(p, st);
    if (p.Hkv % 2 == 0) return launch_scores_mma_shape<T, G, 2, 128, false, 2>(p, st);
  }
  const long rows = (long)p.B * p.Hkv, one_wave = 8L * num_sms();
  if (rows * ((p.max_pages + 255) / 256) >= one_wave) return launch_scores_mma_shape<T, G, 2, 256, false>(p, st);
  return launch_scores_mma_shape<T, G, 2, 128, false>(p, st);
}

template <typename T>
static int launch_scores_g(const ScoreParams& p, cudaStream_t st) {
  // Groups of four and eight query heads go to the tensor-core kernel (the per-head FMA form is
  // bound by shared-memory reads of q there); TWL_SCORES_SIMT=1 keeps the FMA form for comparison.
  static const bool simt = [] {
    const char* e = getenv("TWL_SCORES_SIMT");
    return e && e[0] == '1';
  }();
  if (p.counters == nullptr && !simt) {
    if (p.Hq / p.Hkv == 4) return launch_scores_mma<T, 4>(p, st);
    if (p.Hq / p.Hkv == 8) return launch_scores_mma<T, 8>(p, st);
  }
  switch (p.Hq / p.Hkv) {
    case 1: return launch_scores<T, 1>(p, st);
    case 2: return launch_scores<T, 2>(p, st);
    case 4: return launch_scores<T, 4>(p, st);
    case 8: return launch_scores<T, 8>(p, st);
    default: return TWL_ERR_UNSUPPORTED;
  }
}

}  // namespace twl

extern "C" int twl_quest_page_scores(const void* q, int dtype, const void* kmeta,
                                     const int32_t* kv_indptr, const int32_t* kv_indices,
                                     int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                     int32_t num_pages_total, float* page_scores,
                                     int32_t max_pages, int32_t* status, void* stream) {
  using namespace twl;
  if (!q || !kmeta || !kv_indptr || !kv_indices || !page_scores) return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_pages_total <= 0 ||
      max_pages <= 0 || num_q_heads % num_kv_heads != 0)
    return TWL_ERR_BAD_ARG;
  if (!aligned(q, 16) || !aligned(kmeta, 16)) return TWL_ERR_MISALIGNED;
  ScoreParams p;
  p.q = q; p.kmeta = kmeta; p.indptr = kv_indptr; p.indices = kv_indices;
  p.page_scores = page_scores; p.status = status; p.B = batch; p.Hq = num_q_heads;
  p.Hkv = num_kv_heads; p.num_pages_total = num_pages_total; p.max_pages = max_pages;
  p.counters = nullptr; p.cand_pages = nullptr; p.cand_npages = nullptr; p.token_budget = 0; p.max_k = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) return launch_scores_g<__half>(p, st);
  if (dtype == TWL_BF16) return launch_scores_g<__nv_bfloat16>(p, st);
  return TWL_ERR_UNSUPPORTED;
}

extern "C" int twl_quest_select(const void* q, int dtype, const void* kmeta,
                                const int32_t* kv_indptr, const int32_t* kv_indices, int32_t batch,
                                int32_t num_q_heads, int32_t num_kv_heads, int32_t num_pages_total,
                                int32_t token_budget, float* page_scores, int32_t max_pages,
                                int32_t* cand_pages, int32_t* cand_npages, int32_t max_k,
                                int32_t* counters, int32_t* status, void* stream) {
  using namespace twl;
  if (!q || !kmeta || !kv_indptr || !kv_indices || !page_scores || !cand_pages || !cand_npages ||
      !counters)
    return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_pages_total <= 0 ||
      max_pages <= 0 || max_k <= 0 || token_budget < 0 || num_q_heads % num_kv_heads != 0)
    return TWL_ERR_BAD_ARG;
  if (max_pages > 48 * 1024) return TWL_ERR_TOO_LARGE;  // keys of a row live in shared memory
  if (!aligned(q, 16) || !aligned(kmeta, 16)) return TWL_ERR_MISALIGNED;
  ScoreParams p;
  p.q = q; p.kmeta = kmeta; p.indptr = kv_indptr; p.indices = kv_indices;
  p.page_scores = page_scores; p.status = status; p.B = batch; p.Hq = num_q_heads;
  p.Hkv = num_kv_heads; p.num_pages_total = num_pages_total; p.max_pages = max_pages;
  p.counters = counters; p.cand_pages = cand_pages; p.cand_npages = cand_npages;
  p.token_budget = token_budget; p.max_k = max_k;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) return launch_scores_g<__half>(p, st);
  if (dtype == TWL_BF16) return launch_scores_g<__nv_bfloat16>(p, st);
  return TWL_ERR_UNSUPPORTED;
}

extern "C" int twl_quest_topk_pages(const float* page_scores, int32_t max_pages,
                                    const int32_t* kv_indptr, int32_t batch, int32_t num_q_heads,
                                    int32_t token_budget, int32_t* cand_pages,
                                    int32_t* cand_npages, int32_t max_k, void* stream) {
  using namespace twl;
  if (!page_scores || !kv_indptr || !cand_pages || !cand_npages) return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_q_heads <= 0 || max_pages <= 0 || max_k <= 0 || token_budget < 0)
    return TWL_ERR_BAD_ARG;
  if (max_pages > 48 * 1024) return TWL_ERR_TOO_LARGE;  // keys of a row live in shared memory
  const size_t smem = (size_t)max_pages * sizeof(uint32_t);
  TWL_CUDA_TRY(cudaFuncSetAttribute(quest_topk_pages_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024 * 4));
  TopkParams tp;
  tp.page_scores = page_scores; tp.indptr = kv_indptr; tp.cand_pages = cand_pages;
  tp.cand_npages = cand_npages; tp.max_pages = max_pages; tp.Hq = num_q_heads;
  tp.token_budget = token_budget; tp.max_k = max_k;
  TWL_CUDA_TRY(launch_chain(quest_topk_pages_kernel, dim3(batch * num_q_heads), dim3(kTopkThreads), smem,
                            reinterpret_cast<cudaStream_t>(stream), tp));
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}
