// Kernel #3: sparse paged decode attention over the pruned token lists.
//
// Stands in for twilight/pyimpl/attention.py:188-190 (exact q.k logits, here only for the
// kept tokens) and :298-306 (masked fp32 softmax, P.V).  The reference computes the dense
// [L] row and masks it; here a row's cost is its budget.
//
// Budgets differ by orders of magnitude between heads, so work is balanced on the device: the
// kept tokens of a (batch, query head) row are cut into chunks of `chunk` tokens, every block
// first prefix-sums the rows' chunk counts in shared memory (all blocks compute the same
// tables, nothing is exchanged), and block x then takes item x of every round of grid-size
// items from the flattened (row, chunk) list, in which the full-length chunks of all rows come
// before the rows' last chunks.  The four warps of a block split an item's tokens evenly.
//
// A warp with more than a handful of tokens streams them through a private ring in shared
// memory: 8 tokens per stage (their 256-byte K rows and V rows, fetched with 16-byte
// asynchronous copies), three stages, so two stages are always in flight while one is used and
// the bytes in flight do not depend on how the compiler schedules loads.  Token -> K/V row
// lookups (index list, page table) run a 32-token group ahead of the copies.  Four lanes share
// a token: lane (t, part) multiplies 32 channels of q (chunks part, part+4, part+8, part+12 of
// eight channels) with its token's K, two shuffles finish the dot product, and the same lane
// accumulates its token's V into 32 private accumulators, which are added across the eight
// tokens once per item.  Odd tokens store their chunks with bit 2 of the chunk number flipped,
// which makes the 16-byte reads of a quarter warp hit eight different bank groups.  Softmax is
// online (running max shared by the warp, per-lane partial sums).
// A warp with at most four tokens (budgets of a few tokens are the common case after pruning)
// reads them straight into registers instead.
// Warps merge through shared memory; chunks of a row merge through the caller's workspace, and
// the block that finishes a row's last chunk (an atomic ticket, nobody waits) writes the output.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace twl {

constexpr int kAttThreads = 128;
constexpr int kAttWarps = kAttThreads / 32;
constexpr int kMaxChunksPerRow = 32;     // partial slots per row in the workspace
constexpr int kAttStageTokens = 8;
constexpr int kAttStageBytes = kAttStageTokens * 2 * kD * 2;  // K rows, then V rows: 4 KiB
constexpr int kAttStages = 3;
constexpr int kAttRingBytes = kAttWarps * kAttStages * kAttStageBytes;  // 48 KiB per block
constexpr int kAttBlocksPerSM = 4;       // what the ring leaves room for
constexpr int kAttMaxRows = 64 * 1024;   // schedule tables (1.25 bytes a row) next to the ring
constexpr float kNegBig = -3.0e38f;      // finite stand-in for -inf so that exp(m_old-m_new) is defined

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
  float* part_ml;     // [rows][kMaxChunksPerRow][2]
  float* part_o;      // [rows][kMaxChunksPerRow][128]
  int32_t* status;
  const float* weights;  // [rows][index_stride] softmax weights of the kept tokens, or nullptr
  int32_t* group_flags;  // [batch*Hkv] 1 = the (sequence, KV head) row is served by the group kernel; or nullptr
  int index_stride, rows, Hq, Hkv, num_pages_total, chunk;
  int group_skip_rows;  // group kernel: do not fetch token rows that no head of the group keeps
  int group_chunk_pages;  // group kernel: pages of the longest chunk of a sequence of max_seq_pages pages
  int max_seq_pages;      // upper bound of a sequence's page count (the physical page count if nothing better is known)
  float sm_scale;
};

// chunk length actually used for a row: `chunk`, grown so that a row never needs more than
// kMaxChunksPerRow partial slots
__device__ __forceinline__ int row_chunk_len(int budget, int chunk) {
  int len = chunk;
  while ((budget + len - 1) / len > kMaxChunksPerRow) len *= 2;
  return len;
}

// USE_W: the caller supplies un-normalised softmax weights of the kept tokens (attention over
// estimated weights, twilight/pyimpl/attention.py:295-296); K is then not read at all.
template <typename T, bool USE_W = false>
__global__ void __launch_bounds__(kAttThreads, kAttBlocksPerSM)
sparse_decode_attn_kernel(const AttParams p) {
  extern __shared__ __align__(128) unsigned char sm_dyn[];  // the ring, then the schedule table
  // schedule tables: chunk count of every row (one byte each) and, per group of 32 rows, the
  // exclusive prefix sums of the rows' leading (full) chunks and of their last chunks
  const int n_groups = (p.rows + 31) >> 5;
  int* sm_glead = reinterpret_cast<int*>(sm_dyn + kAttRingBytes);
  int* sm_glast = sm_glead + n_groups + 1;
  uint8_t* sm_cnt = reinterpret_cast<uint8_t*>(sm_glast + n_groups + 1);
  __shared__ float sm_m[kAttWarps], sm_l[kAttWarps];
  __shared__ int sm_scan[66];
  __shared__ int sm_ticket;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // a warp's 128 merged output channels sit at the start of its (then idle) part of the ring
  auto warp_out = [&](int w) -> float* {
    return reinterpret_cast<float*>(sm_dyn + w * (kAttStages * kAttStageBytes));
  };
  float* const my_out = warp_out(warp);
  pdl_wait();  // budgets and index lists come from the pruner launched before
  // ---- schedule (identical in every block): a row of n chunks has n-1 leading chunks of full
  // length and one last chunk.  Work items are numbered with all leading chunks first, then all
  // last chunks, so that the long items are dealt out before the short ones ----
  {
    constexpr int kPer = 4;  // consecutive rows per thread and pass: 8 threads cover a group
    int carry_lead = 0, carry_last = 0;
    for (int r0 = 0; r0 < p.rows; r0 += kAttThreads * kPer) {
      int s_lead = 0, s_last = 0;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const int r = r0 + tid * kPer + j;
        if (r < p.rows) {
          const bool grouped = p.group_flags != nullptr && p.group_flags[r / (p.Hq / p.Hkv)] != 0;
          const int bud = grouped ? 0 : min(max(p.budget[r], 0), p.index_stride);
          const int len = row_chunk_len(bud, p.chunk);
          const int n = (bud + len - 1) / len;
          sm_cnt[r] = grouped ? (uint8_t)255 : (uint8_t)n;  // 255: not this kernel's row (row counts stop at 32)
          s_lead += max(n - 1, 0);
          s_last += n > 0 ? 1 : 0;
        }
      }
      int t_lead, t_last, e_lead, e_last;
      block_excl_scan2<kAttThreads>(s_lead, s_last, &e_lead, &e_last, &t_lead, &t_last, sm_scan);
      const int first = r0 + tid * kPer;
      if ((tid & 7) == 0 && first < p.rows) {
        sm_glead[first >> 5] = carry_lead + e_lead;
        sm_glast[first >> 5] = carry_last + e_last;
      }
      carry_lead += t_lead;
      carry_last += t_last;
    }
    if (tid == 0) {
      sm_glead[n_groups] = carry_lead;
      sm_glast[n_groups] = carry_last;
    }
    __syncthreads();
  }
  const int n_lead = sm_glead[n_groups];
  const int n_items = n_lead + sm_glast[n_groups];
  // rows without kept tokens produce zeros (the reference never meets this case)
  for (int r = blockIdx.x * kAttThreads + tid; r < p.rows; r += gridDim.x * kAttThreads) {
    if (sm_cnt[r] == 0) {
      T* o = reinterpret_cast<T*>(p.out) + (size_t)r * kD;
      for (int d = 0; d < kD; ++d) o[d] = Elem<T>::from_f(0.f);
    }
  }

  const T* kbase = reinterpret_cast<const T*>(p.k);
  const T* vbase = reinterpret_cast<const T*>(p.v);
  unsigned char* const my_ring = sm_dyn + warp * (kAttStages * kAttStageBytes);
  const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);

  // block x takes item x of every round of gridDim.x items; odd rounds run backwards, so the
  // blocks that got the long items of one round get the short ones of the next
  for (int base = 0, round = 0; base < n_items; base += gridDim.x, ++round) {
    const int item = base + ((round & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x);
    if (item >= n_items) continue;  // the same for the whole block
    // group of this item: last g with prefix[g] <= position in its list; then the lanes of
    // every warp (all warps do the same) scan the group's 32 rows for the one that holds it
    const bool leading = item < n_lead;
    const int* pref = leading ? sm_glead : sm_glast;
    const int pos = leading ? item : item - n_lead;
    int lo = 0, hi = n_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (pref[mid] <= pos) lo = mid; else hi = mid;
    }
    const int rem = pos - pref[lo];
    const int cand_row = lo * 32 + lane;
    const int n_raw = cand_row < p.rows ? (int)sm_cnt[cand_row] : 0;
    const int n_mine = n_raw == 255 ? 0 : n_raw;
    const int mine = leading ? max(n_mine - 1, 0) : (n_mine > 0 ? 1 : 0);
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, inc - mine <= rem && rem < inc);  // one lane
    const int src = __ffs(hit) - 1;
    const int row = lo * 32 + src;
    const int n_parts = __shfl_sync(0xffffffffu, n_mine, src);
    const int c = leading ? rem - __shfl_sync(0xffffffffu, inc - mine, src) : n_parts - 1;
    const int b = row / p.Hq, h = row % p.Hq;
    const int kvh = h / (p.Hq / p.Hkv);
    const int budget = min(p.budget[row], p.index_stride);
    const int clen = row_chunk_len(budget, p.chunk);
    const int begin = c * clen, end = min(budget, begin + clen);
    const int page_base = p.indptr[b];
    const int n_seq_pages = p.indptr[b + 1] - page_base;
    const int32_t* idx = p.idx + (size_t)row * p.index_stride;
    const T* qrow = reinterpret_cast<const T*>(p.q) + (size_t)row * kD;
    T* out = reinterpret_cast<T*>(p.out) + (size_t)row * kD;

    // this warp's share of the item: whole stages of 8 tokens
    const int per_warp = (((end - begin) + kAttWarps - 1) / kAttWarps + kAttStageTokens - 1) & ~(kAttStageTokens - 1);
    const int w_begin = begin + warp * per_warp;
    const int w_end = min(end, w_begin + per_warp);
    const int n_my = max(w_end - w_begin, 0);

    // token index -> row number inside the K/V page arrays (-1 = nothing to read).  The two
    // dependent loads (index list, page table) are issued a 32-token group apart and their
    // results are looked at a group later still, so the streaming loop never waits on them;
    // bad indices are only remembered and reported after the loop
    bool bad = false;
    auto load_tok = [&](int t) -> int { return (t < w_end) ? idx[t] : -1; };
    auto table = [&](int tok) -> int {
      int ro = -1;
      const int pg = tok >> 4;
      if (tok >= 0 && pg < n_seq_pages) {
        const int phys = p.indices[page_base + pg];
        if (phys >= 0 && phys < p.num_pages_total) ro = (phys * p.Hkv + kvh) * kPage + (tok & 15);
      }
      return ro;
    };

    float m = USE_W ? 0.f : kNegBig, l = 0.f;
    if (n_my == 0) {
#pragma unroll
      for (int d = 0; d < 4; ++d) my_out[lane * 4 + d] = 0.f;
    } else if (!USE_W && n_my <= 4) {
      // ---- a handful of tokens: four rows straight into registers, lane owns 4 channels ----
      float qf[4];
      {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(qrow) + lane);
        const float2 a = Elem<T>::to_f2(u.x), bq = Elem<T>::to_f2(u.y);
        qf[0] = a.x * p.sm_scale; qf[1] = a.y * p.sm_scale;
        qf[2] = bq.x * p.sm_scale; qf[3] = bq.y * p.sm_scale;
      }
      const int ro = table(load_tok(w_begin + lane));  // lanes past the share get -1
      bad = (w_begin + lane < w_end) && ro < 0;
      uint2 k4[4], v4[4];
      int r4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        // absent tokens read row 0 (always mapped) and get weight 0, so the loads carry no branch
        r4[u] = __shfl_sync(0xffffffffu, ro, u);
        const int rc = max(r4[u], 0);
        k4[u] = ldg_stream_u2(kbase + (size_t)rc * kD + lane * 4);
        v4[u] = ldg_stream_u2(vbase + (size_t)rc * kD + lane * 4);
      }
      float sc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 k0 = Elem<T>::to_f2(k4[u].x), k1 = Elem<T>::to_f2(k4[u].y);
        sc[u] = qf[0] * k0.x + qf[1] * k0.y + qf[2] * k1.x + qf[3] * k1.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        sc[u] = (r4[u] >= 0) ? sc[u] : -INFINITY;
        m = fmaxf(m, sc[u]);
      }
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float pu = __expf(sc[u] - m);
        l += pu;
        const float2 v0 = Elem<T>::to_f2(v4[u].x), v1 = Elem<T>::to_f2(v4[u].y);
        acc[0] = fmaf(pu, v0.x, acc[0]);
        acc[1] = fmaf(pu, v0.y, acc[1]);
        acc[2] = fmaf(pu, v1.x, acc[2]);
        acc[3] = fmaf(pu, v1.y, acc[3]);
      }
#pragma unroll
      for (int d = 0; d < 4; ++d) my_out[lane * 4 + d] = acc[d];
    } else {
      // ---- streamed through the ring ----
      const int t8 = lane >> 2, part = lane & 3;
      const int flip = (t8 & 1) << 2;
      float qv[USE_W ? 1 : 32];
      if (!USE_W) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 u = __ldg(reinterpret_cast<const uint4*>(qrow) + part + 4 * j);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = Elem<T>::to_f2(w[i]);
            qv[8 * j + 2 * i] = f.x * p.sm_scale;
            qv[8 * j + 2 * i + 1] = f.y * p.sm_scale;
          }
        }
      }
      float acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.f;
      const int n_stages = (n_my + kAttStageTokens - 1) / kAttStageTokens;
      const float* wrow = USE_W ? p.weights + (size_t)row * p.index_stride : nullptr;
      // lane i of a group resolves token w_begin + 32*group + i (and, USE_W, loads its weight)
      int ro_cur = -1, ro_next = table(load_tok(w_begin + lane));
      int tok_next = load_tok(w_begin + 32 + lane);
      float w_cur = 0.f, w_next = 0.f;
      if (USE_W) w_next = (w_begin + lane < w_end) ? wrow[w_begin + lane] : 0.f;
      unsigned valid = 0;           // 8 bits per ring slot: which tokens of the stage count
      float pw0 = 0.f, pw1 = 0.f, pw2 = 0.f;  // USE_W: this lane's token weight, per ring slot
      int issue_j = 0, issue_slot = 0;
      auto issue = [&]() {
        // stage issue_j -> slot issue_slot
        if (issue_j < n_stages) {
          const int sub = issue_j & 3;
          if (sub == 0) {
            const int group = issue_j >> 2;
            ro_cur = ro_next;
            w_cur = w_next;
            bad = bad || ((w_begin + 32 * group + lane < w_end) && ro_cur < 0);
            ro_next = table(tok_next);
            tok_next = load_tok(w_begin + 32 * (group + 2) + lane);
            const int t_next = w_begin + 32 * (group + 1) + lane;
            if (USE_W) w_next = (t_next < w_end) ? wrow[t_next] : 0.f;
          }
          const uint32_t dst = my_ring_s + issue_slot * kAttStageBytes;
          const int cpos = lane & 15;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int tk = 2 * i + (lane >> 4);
            const int rc = max(__shfl_sync(0xffffffffu, ro_cur, sub * 8 + tk), 0);
            const uint32_t off = tk * 256 + ((cpos ^ ((tk & 1) << 2)) << 4);
            if (!USE_W) cp_async16(dst + off, kbase + (size_t)rc * kD + cpos * 8);
            cp_async16(dst + kAttStageTokens * 256 + off, vbase + (size_t)rc * kD + cpos * 8);
          }
          const unsigned vm = (__ballot_sync(0xffffffffu, ro_cur >= 0) >> (sub * 8)) & 0xFFu;
          valid = (valid & ~(0xFFu << (8 * issue_slot))) | (vm << (8 * issue_slot));
          if (USE_W) {
            const float pw = __shfl_sync(0xffffffffu, w_cur, sub * 8 + t8);
            if (issue_slot == 0) pw0 = pw; else if (issue_slot == 1) pw1 = pw; else pw2 = pw;
          }
        }
        cp_async_commit();  // always, so that group counting stays uniform
        ++issue_j;
        issue_slot = (issue_slot + 1 == kAttStages) ? 0 : issue_slot + 1;
      };
#pragma unroll
      for (int s0 = 0; s0 < kAttStages - 1; ++s0) issue();
      int slot = 0;
      for (int k = 0; k < n_stages; ++k) {
        issue();
        cp_async_wait<kAttStages - 1>();  // stage k has landed (this thread's copies)
        __syncwarp();
        const unsigned char* st = my_ring + slot * kAttStageBytes;
        const bool ok = (valid >> (8 * slot + t8)) & 1u;
        float pw;
        if (!USE_W) {
          const uint4* krow = reinterpret_cast<const uint4*>(st + t8 * 256);
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 kv = krow[(part + 4 * j) ^ flip];
            const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = Elem<T>::to_f2(w[i]);
              s = fmaf(qv[8 * j + 2 * i], f.x, s);
              s = fmaf(qv[8 * j + 2 * i + 1], f.y, s);
            }
          }
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          s = ok ? s : -INFINITY;
          float mx = s;
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m, mx);
          const float scale = __expf(m - m_new);
          pw = __expf(s - m_new);
          l = l * scale + pw;
          if (scale != 1.f) {  // warp-uniform: m and m_new are the same in every lane
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] *= scale;
          }
          m = m_new;
        } else {
          pw = slot == 0 ? pw0 : (slot == 1 ? pw1 : pw2);
          pw = ok ? pw : 0.f;
          l += pw;
        }
        const uint4* vrow = reinterpret_cast<const uint4*>(st + kAttStageTokens * 256 + t8 * 256);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 vv = vrow[(part + 4 * j) ^ flip];
          const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = Elem<T>::to_f2(w[i]);
            acc[8 * j + 2 * i] = fmaf(pw, f.x, acc[8 * j + 2 * i]);
            acc[8 * j + 2 * i + 1] = fmaf(pw, f.y, acc[8 * j + 2 * i + 1]);
          }
        }
        __syncwarp();  // every lane is done with the slot before it is refilled
        slot = (slot + 1 == kAttStages) ? 0 : slot + 1;
      }
      cp_async_wait<0>();
      __syncwarp();  // the ring is idle from here on; its first bytes take the warp's result
      // add up the eight tokens' lanes; the four lanes of a token carried the same weight
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
      }
      if (t8 == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int i = 0; i < 8; ++i) my_out[(part + 4 * j) * 8 + i] = acc[8 * j + i];
        }
      }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);

    // merge the warps of this block
    if (lane == 0) {
      sm_m[warp] = m;
      sm_l[warp] = l;
    }
    __syncthreads();
    float bm = kNegBig;
#pragma unroll
    for (int w = 0; w < kAttWarps; ++w) bm = fmaxf(bm, sm_m[w]);
    float bl = 0.f, bo = 0.f;
    const int d = tid;  // thread d owns channel d from here on
#pragma unroll
    for (int w = 0; w < kAttWarps; ++w) {
      const float f = __expf(sm_m[w] - bm);
      bl += f * sm_l[w];
      bo += f * warp_out(w)[d];
    }
    if (n_parts == 1) {
      out[d] = Elem<T>::from_f(bl > 0.f ? bo / bl : 0.f);
    } else {
      // publish this chunk's partial, then take a ticket
      const size_t slot = (size_t)row * kMaxChunksPerRow + c;
      p.part_o[slot * kD + d] = bo;
      if (d == 0) {
        p.part_ml[slot * 2] = bm;
        p.part_ml[slot * 2 + 1] = bl;
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) sm_ticket = atomicAdd(&p.counters[row], 1);
      __syncthreads();
      if (sm_ticket == n_parts - 1) {  // every chunk of the row has been published
        __threadfence();
        float gm = kNegBig;
        for (int cc = 0; cc < n_parts; ++cc)
          gm = fmaxf(gm, __ldcg(&p.part_ml[((size_t)row * kMaxChunksPerRow + cc) * 2]));
        float gl = 0.f, go = 0.f;
        for (int cc = 0; cc < n_parts; ++cc) {
          const size_t s2 = (size_t)row * kMaxChunksPerRow + cc;
          const float f = __expf(__ldcg(&p.part_ml[s2 * 2]) - gm);
          gl += f * __ldcg(&p.part_ml[s2 * 2 + 1]);
          go += f * __ldcg(&p.part_o[s2 * kD + d]);
        }
        out[d] = Elem<T>::from_f(gl > 0.f ? go / gl : 0.f);
        if (tid == 0) p.counters[row] = 0;  // leave the workspace ready for the next call
      }
    }
    __syncthreads();  // shared merge buffers are reused by the next item
  }
}

// ---- query-head groups: the K/V pages of a KV head are read once for all of its query heads ----
//
// When the query heads of a KV head keep, between them, at least as many tokens as the sequence
// has (what dense-ish heads do), fetching every head's tokens separately reads the same K/V rows
// several times.  This kernel serves such (sequence, KV head) rows instead: it walks the pages of a
// chunk of the sequence in which any head of the group kept a token, stages each page once (K and
// V: 8 KiB) in a warp-private ring, and computes all the group's heads on tensor cores:
//   S^T[head][token] = Q K^T      m16n8k16 tiles, A = Q (heads as rows, padded to 16), B = the K page
//   masked per head by the page's kept-token bits, online softmax per head in the accumulator
//   layout, O[head][dim] += P V   A = P rounded to the model dtype (attention.py:302-304), B = the
//   V page read transposed.
// The per-head kept-token bits come from the index lists themselves: they are ascending (the
// pruner writes them so), so a head's tokens inside the chunk are one run of its list, found by a
// 32-way search; every lane turns a piece of the run into page bit masks.  Partial results go
// through the same workspace slots and arrival counters as the per-head kernel's chunks, so the
// merge and the output are the same.  Whether a row is served here is decided on the device from
// the budgets (the host never sees them) and published in group_flags for the per-head kernel,
// which runs afterwards and skips those rows.
// Four warps share a work item (a chunk of 64-256 pages of one sequence and KV head): with two, an
// item lives twice as long and the grid's tail - SMs running out of items - cost 7-9 % (config 2
// 943 -> 877 us, config-4 shard 637 -> 583 us); with eight, a warp gets too few pages to fill its ring
// (1011 us on config 2).
constexpr int kGrpWarps = 4;
constexpr int kGrpThreads = kGrpWarps * 32;
constexpr int kGrpStageBytes = 2 * kPage * kD * 2;                       // K page, then V page: 8 KiB
// ring of a block: `stages` whole-page stages (K page, then V page) per warp, or, with stages == 1,
// three half-stages (one K or V page each) per warp
__host__ __device__ constexpr int grp_ring_bytes(int stages) {
  return stages == 1 ? kGrpWarps * 3 * (kGrpStageBytes / 2) : kGrpWarps * stages * kGrpStageBytes;
}
constexpr int kGrpMaxChunkPages = 256;                                   // pages of one work item
constexpr int kGrpMinChunkPages = 64;

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// First positions of ascending lists whose value is >= a key: search s looks for key[s & 1] in the list
// idx[s >> 1][0..n[s >> 1]).  The warp probes 32 places per step, so three dependent loads settle a
// list of 32768 entries; the NS searches advance in lockstep, their probes of a step in flight
// together, so the whole set costs the latency of one search.
template <int NS>
__device__ __forceinline__ void warp_lower_bounds(const int32_t* const (&idx)[NS / 2], const int (&n)[NS / 2],
                                                  const int (&key)[2], int lane, int (&pos)[NS]) {
  int lo[NS], hi[NS];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    lo[s] = 0;
    hi[s] = n[s >> 1];
  }
  while (true) {
    bool any = false;
    int val[NS], step[NS];
    bool inb[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const bool open = lo[s] < hi[s];  // warp-uniform
      any = any || open;
      step[s] = (hi[s] - lo[s] + 31) >> 5;
      const int q = lo[s] + lane * step[s];
      inb[s] = open && q < hi[s];
      val[s] = inb[s] ? idx[s >> 1][q] : 0;
    }
    if (!any) break;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      if (lo[s] < hi[s]) {
        const bool less = inb[s] && val[s] < key[s & 1];
        const int cnt = __popc(__ballot_sync(0xffffffffu, less));  // the probes below key are a prefix
        if (cnt == 0) {
          hi[s] = lo[s];
        } else {
          const int nlo = lo[s] + (cnt - 1) * step[s] + 1;
          hi[s] = min(hi[s], lo[s] + cnt * step[s]);
          lo[s] = nlo;
        }
      }
    }
  }
#pragma unroll
  for (int s = 0; s < NS; ++s) pos[s] = lo[s];
}

template <typename T, int G, int kGrpStages>
__global__ void __launch_bounds__(kGrpThreads, (kGrpStages == 1 ? 16 : 12) / kGrpWarps)
group_decode_attn_kernel(const AttParams p) {
  static_assert(G == 2 || G == 4 || G == 8, "the group sits in the upper rows of one m16 tile");
  extern __shared__ __align__(128) unsigned char sm_dyn[];  // the rings; later the warps' results
  // behind the rings, sized by the launch for the longest chunk any row can have (cpm pages):
  const int cpm = p.group_chunk_pages;
  int* const sm_uphys = reinterpret_cast<int*>(sm_dyn + grp_ring_bytes(kGrpStages));  // [cpm] where the pages lie
  uint32_t* const sm_mask = reinterpret_cast<uint32_t*>(sm_uphys + cpm);   // [G][cpm / 2] kept-token bits, two pages a word
  uint16_t* const sm_upage = reinterpret_cast<uint16_t*>(sm_mask + G * (cpm / 2));  // [cpm] pages with any kept token
  uint16_t* const sm_ubits = sm_upage + cpm;                               // [cpm] which of their tokens any head keeps
  __shared__ int sm_segcnt[kGrpMaxChunkPages / 32];
  __shared__ int sm_ticket[G];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = blockIdx.x, rkv = blockIdx.y;
  const int b = rkv / p.Hkv, kvh = rkv % p.Hkv;
  const int row0 = b * p.Hq + kvh * G;  // first (batch, query head) row of the group
  pdl_wait();  // budgets and index lists come from the pruner launched before
  const int page_base = p.indptr[b];
  const int pages_b = p.indptr[b + 1] - page_base;
  // served here when the group's heads keep at least one token per token of the sequence
  int bud_l = 0;
  if (lane < G) bud_l = min(max(p.budget[row0 + lane], 0), p.index_stride);
  const int bud_sum = warp_sum_i(bud_l);
  const bool mine = pages_b > 0 && pages_b <= kMaxChunksPerRow * cpm &&
                    (long long)bud_sum >= (long long)pages_b * kPage;
  if (c == 0 && tid == 0) p.group_flags[rkv] = mine ? 1 : 0;
  if (!mine) return;
  int cp = kGrpMinChunkPages;  // pages per chunk: at most kMaxChunksPerRow chunks per row
  while (cp * kMaxChunksPerRow < pages_b) cp *= 2;
  const int n_chunks = (pages_b + cp - 1) / cp;
  if (c >= n_chunks) return;
  const int p0 = c * cp, p1 = min(pages_b, p0 + cp), npg = p1 - p0;

  // ---- Q as the A operand: row g = head g (rows from G on are zero), eight k-steps of 16 channels
  // (fetched first: the loads are under way while the index lists are searched) ----
  const int g = lane >> 2, t = lane & 3;
  uint32_t qa[8][2];
  {
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.q) +
                                                             (size_t)(row0 + (g < G ? g : 0)) * kD);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = g < G ? __ldg(qrow + 8 * ks + t) : 0u;      // channels 16ks + 2t, +1
      qa[ks][1] = g < G ? __ldg(qrow + 8 * ks + 4 + t) : 0u;  // channels 16ks + 8 + 2t, +1
    }
  }

  // ---- kept-token bits of every head for the pages of this chunk ----
  for (int i = tid; i < G * (cpm / 2); i += kGrpThreads) sm_mask[i] = 0u;
  __syncthreads();
  bool bad = false;
  {
    // a warp's heads (warp, warp + kGrpWarps, ...): where the chunk begins and ends in each one's
    // ascending index list, all searches in lockstep
    constexpr int HPW = (G + kGrpWarps - 1) / kGrpWarps;
    const int32_t* lists[HPW];
    int ns[HPW], pos[2 * HPW];
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
      const int hh = warp + j * kGrpWarps;
      lists[j] = p.idx + (size_t)(row0 + (hh < G ? hh : 0)) * p.index_stride;
      ns[j] = __shfl_sync(0xffffffffu, bud_l, hh & 31);
      if (hh >= G) ns[j] = 0;
    }
    const int keys[2] = {p0 * kPage, p1 * kPage};
    warp_lower_bounds<2 * HPW>(lists, ns, keys, lane, pos);
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
      const int hh = warp + j * kGrpWarps;
      if (hh >= G) continue;
      const int32_t* idx = lists[j];
      const int s0 = pos[2 * j], s1 = pos[2 * j + 1];
      if (c == n_chunks - 1 && s1 < ns[j]) bad = true;  // tokens past the last page of the sequence
      // each lane owns a run of whole 16-byte groups of the list (a row of the index array starts on a 64-byte
      // boundary); four groups at a time are in flight before the first is used
      const int a4 = s0 >> 2, e4 = (s1 + 3) >> 2;
      const int per = (e4 - a4 + 31) >> 5;
      const int la = a4 + lane * per, le = min(e4, la + per);
      const int4* const idx4 = reinterpret_cast<const int4*>(idx);
      int cur = -1;
      uint32_t bits = 0;
      for (int i = la; i < le; i += 4) {
        int4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = idx4[min(i + k, le - 1)];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int tk[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            const int at = (i + k) * 4 + m;  // position in the list
            if (i + k < le && at >= s0 && at < s1) {
              const int pg = (tk[m] >> 4) - p0;
              if (pg != cur) {
                if (cur >= 0 && cur < npg) atomicOr(&sm_mask[hh * (cpm / 2) + (cur >> 1)], bits << ((cur & 1) * 16));
                cur = pg;
                bits = 0;
              }
              bits |= 1u << (tk[m] & 15);
            }
          }
        }
      }
      if (cur >= 0 && cur < npg) atomicOr(&sm_mask[hh * (cpm / 2) + (cur >> 1)], bits << ((cur & 1) * 16));
    }
  }
  __syncthreads();
  int n_union;
  // ---- pages with any kept token, and where they lie: every warp takes 32-page segments of the chunk, so that
  // the page-table reads of the whole chunk are in flight together; the segments' counts give their offsets ----
  {
    constexpr int kSegs = kGrpMaxChunkPages / 32, kSegsPerWarp = (kSegs + kGrpWarps - 1) / kGrpWarps;
    static_assert(kSegs % kGrpWarps == 0 && kSegs <= 32, "whole segments per warp; one lane per segment in the scan");
    uint32_t u[kSegsPerWarp];
    int phys[kSegsPerWarp];
    unsigned m[kSegsPerWarp];
#pragma unroll
    for (int k = 0; k < kSegsPerWarp; ++k) {
      const int j = (warp + k * kGrpWarps) * 32 + lane;
      u[k] = 0;
      if (j < npg) {
#pragma unroll
        for (int hh = 0; hh < G; ++hh) u[k] |= (sm_mask[hh * (cpm / 2) + (j >> 1)] >> ((j & 1) * 16)) & 0xFFFFu;
      }
      phys[k] = u[k] != 0 ? p.indices[page_base + p0 + j] : -1;
    }
#pragma unroll
    for (int k = 0; k < kSegsPerWarp; ++k) {
      if (u[k] != 0 && (phys[k] < 0 || phys[k] >= p.num_pages_total)) {
        phys[k] = -1;
        bad = true;
      }
      m[k] = __ballot_sync(0xffffffffu, phys[k] >= 0);
      if (lane == 0) sm_segcnt[warp + k * kGrpWarps] = __popc(m[k]);
    }
    __syncthreads();
    const int cnt_l = lane < kSegs ? sm_segcnt[lane] : 0;
    int inc = cnt_l;  // inclusive prefix sums of the segments' counts
#pragma unroll
    for (int o = 1; o < kSegs; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
#pragma unroll
    for (int k = 0; k < kSegsPerWarp; ++k) {
      const int seg = warp + k * kGrpWarps;
      const int base = __shfl_sync(0xffffffffu, inc - cnt_l, seg & 31);
      if (seg < kSegs && phys[k] >= 0) {
        const int pos = base + __popc(m[k] & ((1u << lane) - 1));
        sm_upage[pos] = (uint16_t)(seg * 32 + lane);
        sm_ubits[pos] = (uint16_t)(p.group_skip_rows ? u[k] : 0xFFFFu);
        sm_uphys[pos] = phys[k];
      }
    }
    n_union = __shfl_sync(0xffffffffu, inc, kSegs - 1);
  }
  __syncthreads();
  if (__any_sync(0xffffffffu, bad) && lane == 0) raise_flag(p.status, TWL_FLAG_BAD_INDEX);

  unsigned char* const my_ring = sm_dyn + warp * (grp_ring_bytes(kGrpStages) / kGrpWarps);
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);
  const int my_n = (n_union > warp) ? (n_union - warp + kGrpWarps - 1) / kGrpWarps : 0;
  const T* const kbase = reinterpret_cast<const T*>(p.k);
  const T* const vbase = reinterpret_cast<const T*>(p.v);
  // a page is 16 token rows of 256 bytes; chunk ch of token row r goes to position ch ^ (r & 7), which
  // keeps the copies and the 8-row matrix reads below free of bank conflicts
  // Token rows that no head keeps are not fetched: their slots keep what an earlier page left there
  // (zeros at first), finite values that the masked softmax multiplies by zero.
  auto issue = [&](int i, int slot) {
    if (i < my_n) {
      const int phys = sm_uphys[warp + i * kGrpWarps];
      const uint32_t ub = sm_ubits[warp + i * kGrpWarps];
      const size_t off = ((size_t)phys * p.Hkv + kvh) * (kPage * kD);
      const unsigned char* ksrc = reinterpret_cast<const unsigned char*>(kbase + off) + lane * 16;
      const unsigned char* vsrc = reinterpret_cast<const unsigned char*>(vbase + off) + lane * 16;
      const uint32_t dst = ring_s + slot * kGrpStageBytes;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int r = 2 * j + (lane >> 4), ch = lane & 15;
        const uint32_t d = r * 256 + ((ch ^ (r & 7)) << 4);
        if ((ub >> r) & 1u) {
          cp_async16(dst + d, ksrc + j * 512);
          cp_async16(dst + kPage * kD * 2 + d, vsrc + j * 512);
        }
      }
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };
  {
    uint4* z = reinterpret_cast<uint4*>(my_ring);
    for (int i = lane; i < grp_ring_bytes(kGrpStages) / kGrpWarps / 16; i += 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncwarp();
  }
  // the n-th half-stage of the warp: the K page (n even) or the V page (n odd) of its page n / 2
  // this lane's eight copies of a page: token rows 2j + (lane >> 4), chunk lane & 15; rows r and r + 8
  // are swizzled alike, so four offsets do
  uint32_t doff[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = 2 * j + (lane >> 4), ch = lane & 15;
    doff[j] = r * 256 + ((ch ^ (r & 7)) << 4);
  }
  auto issue_half = [&](int n, int hslot) {
    const int i = n >> 1;
    if (i < my_n) {
      const int phys = sm_uphys[warp + i * kGrpWarps];
      const uint32_t ub = (uint32_t)sm_ubits[warp + i * kGrpWarps] >> (lane >> 4);  // bit 2j: this lane's row of step j
      const size_t off = ((size_t)phys * p.Hkv + kvh) * (kPage * kD);
      const unsigned char* src = reinterpret_cast<const unsigned char*>(((n & 1) ? vbase : kbase) + off) + lane * 16;
      const uint32_t dst = ring_s + hslot * (kGrpStageBytes / 2);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (ub & (1u << (2 * j))) cp_async16(dst + doff[j & 3] + (j >> 2) * 2048, src + j * 512);
    }
    cp_async_commit();
  };
  if (kGrpStages == 1) {
    issue_half(0, 0);
    issue_half(1, 1);
    issue_half(2, 2);
  } else {
#pragma unroll
    for (int i = 0; i < kGrpStages - 1; ++i) issue(i, i);
  }

  // ldmatrix lane addressing: matrix mi = lane >> 3, row r8 = lane & 7 of it
  const int mi = lane >> 3, r8 = lane & 7;
  // K: matrices (tokens 0-7, chunk 2ks) (tokens 0-7, 2ks+1) (tokens 8-15, 2ks) (tokens 8-15, 2ks+1)
  const int k_tok = r8 + (mi >> 1) * 8, k_sub = mi & 1;
  // V, transposed: (tokens 0-7, chunk 2jj) (tokens 8-15, 2jj) (tokens 0-7, 2jj+1) (tokens 8-15, 2jj+1)
  const int v_tok = r8 + (mi & 1) * 8, v_sub = mi >> 1;

  // O is kept transposed, Oᵀ = Vᵀ·Pᵀ: tile jj holds channels 16jj..16jj+15 as rows and the heads as
  // columns, so every accumulator register is used (this lane: channels 16jj+g and 16jj+8+g of heads
  // 2t and 2t+1).  Pᵀ as the B operand has the layout of the Sᵀ accumulators: nothing is moved.
  float o[8][4];
#pragma unroll
  for (int jj = 0; jj < 8; ++jj) o[jj][0] = o[jj][1] = o[jj][2] = o[jj][3] = 0.f;
  float m_run = kNegBig, l_run = 0.f;  // of head g, over this lane's tokens (columns 2t, 2t+1, 8+2t, 9+2t)
  // Half-stages: K of page i sits in slot 2i mod 3, V in slot (2i+1) mod 3.  Once a page's K fragments
  // are in registers its slot takes V of the next page, once the V fragments are, theirs takes K of
  // the page after the next: two half-stages in flight all the time in 12 KiB per warp.
  int slot = 0, fill = kGrpStages - 1;
  int kslot = 0, vslot = 1;
  for (int i = 0; i < my_n; ++i) {
    uint32_t st;
    if (kGrpStages == 1) {
      cp_async_wait<2>();
      __syncwarp();
      st = ring_s + kslot * (kGrpStageBytes / 2);
    } else {
      cp_async_wait<(kGrpStages >= 2 ? kGrpStages - 2 : 0)>();
      __syncwarp();
      // the slot of the page worked on in the last iteration is refilled before this page is worked
      // on: kGrpStages - 1 pages of the warp are in flight all the time
      issue(i + kGrpStages - 1, fill);
      st = ring_s + slot * kGrpStageBytes;
    }
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      // all fragment loads of the page first, then the tiles: the loads' latencies overlap instead
      // of each one being waited for by the tile that follows it
      uint32_t kb[8][4];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t addr = st + k_tok * 256 + ((((2 * ks + k_sub)) ^ (k_tok & 7)) << 4);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(kb[ks][0]), "=r"(kb[ks][1]), "=r"(kb[ks][2]), "=r"(kb[ks][3])
                     : "r"(addr));
      }
      if (kGrpStages == 1) {
        __syncwarp();  // every lane has its K fragments
        issue_half(2 * i + 3, kslot);
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        MmaTile<T>::run(s0, qa[ks][0], 0u, qa[ks][1], 0u, kb[ks][0], kb[ks][1]);  // tokens 0-7
        MmaTile<T>::run(s1, qa[ks][0], 0u, qa[ks][1], 0u, kb[ks][2], kb[ks][3]);  // tokens 8-15
      }
    }
    const int pg = sm_upage[warp + i * kGrpWarps];
    const uint32_t bits = g < G ? (sm_mask[g * (cpm / 2) + (pg >> 1)] >> ((pg & 1) * 16)) & 0xFFFFu : 0u;
    float x[4];
    x[0] = (bits >> (2 * t)) & 1u ? s0[0] * p.sm_scale : -INFINITY;
    x[1] = (bits >> (2 * t + 1)) & 1u ? s0[1] * p.sm_scale : -INFINITY;
    x[2] = (bits >> (8 + 2 * t)) & 1u ? s1[0] * p.sm_scale : -INFINITY;
    x[3] = (bits >> (9 + 2 * t)) & 1u ? s1[1] * p.sm_scale : -INFINITY;
    float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float alpha = __expf(m_run - m_new);
    float pw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) pw[k] = __expf(x[k] - m_new);
    l_run = l_run * alpha + (pw[0] + pw[1]) + (pw[2] + pw[3]);
    m_run = m_new;
    if (__any_sync(0xffffffffu, alpha != 1.f)) {
      const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * t), al1 = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        o[jj][0] *= al0;
        o[jj][1] *= al1;
        o[jj][2] *= al0;
        o[jj][3] *= al1;
      }
    }
    const uint32_t pa0 = pack_pair<T>(pw[0], pw[1]), pa2 = pack_pair<T>(pw[2], pw[3]);
    uint32_t sv = st + kPage * kD * 2;
    if (kGrpStages == 1) {
      cp_async_wait<2>();
      __syncwarp();
      sv = ring_s + vslot * (kGrpStageBytes / 2);
    }
    {
      uint32_t vb[8][4];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const uint32_t addr = sv + v_tok * 256 + ((((2 * jj + v_sub)) ^ (v_tok & 7)) << 4);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(vb[jj][0]), "=r"(vb[jj][1]), "=r"(vb[jj][2]), "=r"(vb[jj][3])
                     : "r"(addr));
      }
      if (kGrpStages == 1) {
        __syncwarp();  // every lane has its V fragments
        issue_half(2 * i + 4, vslot);
      }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        // A = Vᵀ: (channels 16jj.., tokens 0-7) (16jj+8.., 0-7) (16jj.., 8-15) (16jj+8.., 8-15)
        MmaTile<T>::run(o[jj], vb[jj][0], vb[jj][2], vb[jj][1], vb[jj][3], pa0, pa2);
      }
    }
    __syncwarp();  // every lane is done with the slot before the next iteration refills it
    slot = (slot + 1 == kGrpStages) ? 0 : slot + 1;
    fill = (fill + 1 == kGrpStages) ? 0 : fill + 1;
    kslot = (kslot >= 1) ? kslot - 1 : 2;  // 2(i+1) mod 3
    vslot = (vslot >= 1) ? vslot - 1 : 2;
  }
  cp_async_wait<0>();
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();  // the rings are idle from here on: they take the warps' results

  // ---- merge the warps: per head (max, sum, 128 channels) ----
  float* const res = reinterpret_cast<float*>(sm_dyn);  // [warp][G][130]
  if (2 * t < G) {
    float* const o0 = res + ((size_t)warp * G + 2 * t) * 130;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      o0[16 * jj + g] = o[jj][0];
      o0[16 * jj + 8 + g] = o[jj][2];
      if (2 * t + 1 < G) {
        o0[130 + 16 * jj + g] = o[jj][1];
        o0[130 + 16 * jj + 8 + g] = o[jj][3];
      }
    }
  }
  if (g < G && t == 0) {
    float* const mine_o = res + ((size_t)warp * G + g) * 130;
    mine_o[128] = m_run;
    mine_o[129] = l_run;
  }
  __syncthreads();
  for (int e = tid; e < G * kD; e += kGrpThreads) {
    const int hh = e / kD, d = e % kD;
    float gm = kNegBig;
#pragma unroll
    for (int w = 0; w < kGrpWarps; ++w) gm = fmaxf(gm, res[((size_t)w * G + hh) * 130 + 128]);
    float gl = 0.f, go = 0.f;
#pragma unroll
    for (int w = 0; w < kGrpWarps; ++w) {
      const float* r = res + ((size_t)w * G + hh) * 130;
      const float f = __expf(r[128] - gm);
      gl += f * r[129];
      go += f * r[d];
    }
    const int row = row0 + hh;
    if (n_chunks == 1) {
      reinterpret_cast<T*>(p.out)[(size_t)row * kD + d] = Elem<T>::from_f(gl > 0.f ? go / gl : 0.f);
    } else {
      const size_t ps = (size_t)row * kMaxChunksPerRow + c;
      p.part_o[ps * kD + d] = go;
      if (d == 0) {
        p.part_ml[ps * 2] = gm;
        p.part_ml[ps * 2 + 1] = gl;
      }
    }
  }
  if (n_chunks == 1) return;
  // publish, then one ticket per head; whoever holds the last ticket of a row merges its chunks
  __threadfence();
  __syncthreads();
  if (tid < G) sm_ticket[tid] = atomicAdd(&p.counters[row0 + tid], 1);
  __syncthreads();
  // a warp per head (the heads' tickets agree for the whole block): lane c holds chunk c's (max, sum), the
  // weights go round by shuffles, every lane sums four channels over the chunks (kMaxChunksPerRow <= 32)
  static_assert(kMaxChunksPerRow <= 32, "one lane per chunk");
  for (int hh = warp; hh < G; hh += kGrpWarps) {
    if (sm_ticket[hh] != n_chunks - 1) continue;
    __threadfence();
    const int row = row0 + hh;
    const size_t s_base = (size_t)row * kMaxChunksPerRow;
    float m_c = kNegBig, l_c = 0.f;
    if (lane < n_chunks) {
      m_c = __ldcg(&p.part_ml[(s_base + lane) * 2]);
      l_c = __ldcg(&p.part_ml[(s_base + lane) * 2 + 1]);
    }
    const float gm = warp_max(m_c);
    const float f_c = lane < n_chunks ? __expf(m_c - gm) : 0.f;
    const float gl = warp_sum(f_c * l_c);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* po = reinterpret_cast<const float4*>(p.part_o + s_base * kD) + lane;
    for (int cc = 0; cc < n_chunks; ++cc) {
      const float f = __shfl_sync(0xffffffffu, f_c, cc);
      const float4 v = __ldcg(po + (size_t)cc * (kD / 4));
      acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
    }
    const float inv = gl > 0.f ? 1.f / gl : 0.f;
    T* const o = reinterpret_cast<T*>(p.out) + (size_t)row * kD + lane * 4;
    o[0] = Elem<T>::from_f(acc.x * inv);
    o[1] = Elem<T>::from_f(acc.y * inv);
    o[2] = Elem<T>::from_f(acc.z * inv);
    o[3] = Elem<T>::from_f(acc.w * inv);
    if (lane == 0) p.counters[row] = 0;  // leave the workspace ready for the next call
  }
}

// Launch shared by the entry points.  `chain`: launch with programmatic stream serialization so
// that the kernel's prologue overlaps the tail of the kernel before it.
static int launch_attn(const AttParams& p_in, int dtype, size_t rows, int32_t index_stride, int32_t chunk,
                       bool chain, cudaStream_t st) {
  // TWL_ATTN_FETCH_ALL=1: the group kernel fetches whole pages (for measurement)
  static const bool fetch_all = [] {
    const char* e = getenv("TWL_ATTN_FETCH_ALL");
    return e && e[0] == '1';
  }();
  // TWL_ATTN_GROUP_STAGES=2 / 3: whole-page stages (two or three per warp) in the group kernel's
  // rings instead of three half-stages (for measurement)
  static const int grp_stages = [] {
    const char* e = getenv("TWL_ATTN_GROUP_STAGES");
    return (e && e[0] == '3') ? 3 : (e && e[0] == '2') ? 2 : 1;
  }();
  AttParams p = p_in;
  p.group_skip_rows = fetch_all ? 0 : 1;
  // chunks are 64 * 2^k pages, at most kMaxChunksPerRow a row: the tables behind the rings are sized
  // for the longest sequence the caller announces (sequences longer than that, or than 256 pages a
  // chunk allow, stay with the per-head kernel)
  p.group_chunk_pages = kGrpMinChunkPages;
  while (p.group_chunk_pages < kGrpMaxChunkPages && p.group_chunk_pages * kMaxChunksPerRow < p.max_seq_pages)
    p.group_chunk_pages *= 2;
  // enough blocks to give every row its own block when budgets are small, never more than the
  // machine holds at once (the schedule tables grow with the row count and may cost a block)
  const size_t max_items =
      rows * std::min<size_t>(kMaxChunksPerRow, ((size_t)index_stride + chunk - 1) / chunk);
  const size_t n_groups = (rows + 31) / 32;
  const size_t smem = (kAttRingBytes + 2 * (n_groups + 1) * sizeof(int) + rows + 15) & ~(size_t)15;
  // query-head groups whose heads keep, together, at least the sequence's length in tokens are served
  // by the group kernel (it decides per row on the device and leaves flags for the kernel below)
  if (p.group_flags != nullptr) {
    const int g = p.Hq / p.Hkv;
    const dim3 grid(kMaxChunksPerRow, (unsigned)(rows / g));
    if (grid.y > 65535) return TWL_ERR_TOO_LARGE;
#define TWL_LAUNCH_GRP_S(TYPE, GG, SS)                                                             \
  do {                                                                                             \
    auto kern = group_decode_attn_kernel<TYPE, GG, SS>;                                            \
    const int bytes = grp_ring_bytes(SS) + p.group_chunk_pages * (8 + 2 * GG);                     \
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));  \
    if (chain) {                                                                                   \
      TWL_CUDA_TRY(launch_chain(kern, grid, dim3(kGrpThreads), bytes, st, p));                     \
    } else {                                                                                       \
      kern<<<grid, kGrpThreads, bytes, st>>>(p);                                                   \
    }                                                                                              \
  } while (0)
#define TWL_LAUNCH_GRP(TYPE, GG)                                                                   \
  do {                                                                                             \
    if (grp_stages == 3) TWL_LAUNCH_GRP_S(TYPE, GG, 3);                                            \
    else if (grp_stages == 2) TWL_LAUNCH_GRP_S(TYPE, GG, 2);                                       \
    else TWL_LAUNCH_GRP_S(TYPE, GG, 1);                                                            \
  } while (0)
    if (dtype == TWL_F16) {
      if (g == 2) TWL_LAUNCH_GRP(__half, 2); else if (g == 4) TWL_LAUNCH_GRP(__half, 4); else TWL_LAUNCH_GRP(__half, 8);
    } else if (dtype == TWL_BF16) {
      if (g == 2) TWL_LAUNCH_GRP(__nv_bfloat16, 2); else if (g == 4) TWL_LAUNCH_GRP(__nv_bfloat16, 4); else TWL_LAUNCH_GRP(__nv_bfloat16, 8);
    } else {
      return TWL_ERR_UNSUPPORTED;
    }
#undef TWL_LAUNCH_GRP_S
#undef TWL_LAUNCH_GRP
    TWL_CHECK_LAUNCH();
  }
#define TWL_LAUNCH_ATT(TYPE, W)                                                                    \
  do {                                                                                             \
    auto kern = sparse_decode_attn_kernel<TYPE, W>;                                                \
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
    int per_sm = 0;                                                                                \
    TWL_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kAttThreads, smem)); \
    if (per_sm < 1) return TWL_ERR_TOO_LARGE;                                                      \
    const unsigned grid = (unsigned)std::min<size_t>(max_items, (size_t)num_sms() * per_sm);        \
    if (chain) {                                                                                   \
      TWL_CUDA_TRY(launch_chain(kern, dim3(grid), dim3(kAttThreads), smem, st, p));                \
    } else {                                                                                       \
      kern<<<grid, kAttThreads, smem, st>>>(p);                                                    \
    }                                                                                              \
  } while (0)
  if (dtype == TWL_F16) {
    if (p.weights) TWL_LAUNCH_ATT(__half, true); else TWL_LAUNCH_ATT(__half, false);
  } else if (dtype == TWL_BF16) {
    if (p.weights) TWL_LAUNCH_ATT(__nv_bfloat16, true); else TWL_LAUNCH_ATT(__nv_bfloat16, false);
  } else {
    return TWL_ERR_UNSUPPORTED;
  }
#undef TWL_LAUNCH_ATT
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Groups of 2, 4 or 8 query heads per KV head may be served by the group kernel; TWL_ATTN_GROUP=0
// in the environment keeps everything on the per-head kernel (for measurement).
static bool group_path_enabled(int num_q_heads, int num_kv_heads) {
  static const bool on = [] {
    const char* e = getenv("TWL_ATTN_GROUP");
    return !(e && e[0] == '0');
  }();
  const int g = num_q_heads / num_kv_heads;
  return on && (g == 2 || g == 4 || g == 8);
}

}  // namespace twl

extern "C" size_t twl_sparse_attn_workspace_bytes(int32_t batch, int32_t num_q_heads,
                                                  int32_t index_stride, int32_t chunk) {
  if (batch <= 0 || num_q_heads <= 0 || index_stride <= 0 || chunk <= 0) return 0;
  const size_t rows = (size_t)batch * num_q_heads;
  size_t bytes = twl::align_up(2 * rows * sizeof(int32_t), 256);  // arrival counters, then group flags
  bytes += twl::align_up(rows * twl::kMaxChunksPerRow * 2 * sizeof(float), 256);
  bytes += rows * twl::kMaxChunksPerRow * twl::kD * sizeof(float);
  return bytes;
}

static int attn_entry(const void* q, int dtype, const void* k_pages, const void* v_pages,
                      const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* indices,
                      int32_t index_stride, const int32_t* budget, const float* weights, int32_t batch,
                      int32_t num_q_heads, int32_t num_kv_heads, int32_t num_pages_total,
                      float sm_scale, void* out, void* workspace, size_t workspace_bytes,
                      int32_t chunk, int32_t* status, void* stream, int32_t max_seq_pages = 0) {
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
  // the schedule table lives in shared memory; K/V row numbers are 32-bit
  if (rows > (size_t)kAttMaxRows) return TWL_ERR_TOO_LARGE;
  if ((int64_t)num_pages_total * num_kv_heads * kPage >= (int64_t)1 << 31) return TWL_ERR_TOO_LARGE;
  AttParams p;
  p.q = q; p.k = k_pages; p.v = v_pages; p.indptr = kv_indptr; p.indices = kv_indices;
  p.idx = indices; p.budget = budget; p.out = out; p.status = status; p.weights = weights;
  char* ws = static_cast<char*>(workspace);
  p.counters = reinterpret_cast<int32_t*>(ws);
  // the group kernel reads the index lists in 16-byte pieces
  const bool lists16 = aligned(indices, 16) && index_stride % 4 == 0;
  p.group_flags = (weights == nullptr && lists16 && group_path_enabled(num_q_heads, num_kv_heads)) ? p.counters + rows : nullptr;
  ws += align_up(2 * rows * sizeof(int32_t), 256);
  p.part_ml = reinterpret_cast<float*>(ws);
  ws += align_up(rows * kMaxChunksPerRow * 2 * sizeof(float), 256);
  p.part_o = reinterpret_cast<float*>(ws);
  p.index_stride = index_stride; p.rows = (int)rows; p.Hq = num_q_heads; p.Hkv = num_kv_heads;
  p.num_pages_total = num_pages_total; p.chunk = chunk; p.sm_scale = sm_scale;
  p.max_seq_pages = max_seq_pages > 0 ? std::min(max_seq_pages, num_pages_total) : num_pages_total;
  return launch_attn(p, dtype, rows, index_stride, chunk, true, reinterpret_cast<cudaStream_t>(stream));
}

// For the one-call step, which knows the longest sequence's page count.
namespace twl {
int sparse_decode_attn_bounded(const void* q, int dtype, const void* k_pages, const void* v_pages,
                               const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* indices,
                               int32_t index_stride, const int32_t* budget, const float* weights, int32_t batch,
                               int32_t num_q_heads, int32_t num_kv_heads, int32_t num_pages_total, float sm_scale,
                               void* out, void* workspace, size_t workspace_bytes, int32_t chunk, int32_t* status,
                               void* stream, int32_t max_seq_pages) {
  return attn_entry(q, dtype, k_pages, v_pages, kv_indptr, kv_indices, indices, index_stride, budget, weights,
                    batch, num_q_heads, num_kv_heads, num_pages_total, sm_scale, out, workspace, workspace_bytes,
                    chunk, status, stream, max_seq_pages);
}
}  // namespace twl

extern "C" int twl_sparse_decode_attn(const void* q, int dtype, const void* k_pages,
                                      const void* v_pages, const int32_t* kv_indptr,
                                      const int32_t* kv_indices, const int32_t* indices,
                                      int32_t index_stride, const int32_t* budget, int32_t batch,
                                      int32_t num_q_heads, int32_t num_kv_heads,
                                      int32_t num_pages_total, float sm_scale, void* out,
                                      void* workspace, size_t workspace_bytes, int32_t chunk,
                                      int32_t* status, void* stream) {
  return attn_entry(q, dtype, k_pages, v_pages, kv_indptr, kv_indices, indices, index_stride, budget,
                    nullptr, batch, num_q_heads, num_kv_heads, num_pages_total, sm_scale, out,
                    workspace, workspace_bytes, chunk, status, stream);
}

extern "C" int twl_sparse_decode_attn_weighted(const void* q, int dtype, const void* k_pages,
                                               const void* v_pages, const int32_t* kv_indptr,
                                               const int32_t* kv_indices, const int32_t* indices,
                                               int32_t index_stride, const int32_t* budget,
                                               const float* weights, int32_t batch,
                                               int32_t num_q_heads, int32_t num_kv_heads,
                                               int32_t num_pages_total, float sm_scale, void* out,
                                               void* workspace, size_t workspace_bytes,
                                               int32_t chunk, int32_t* status, void* stream) {
  if (!weights) return TWL_ERR_BAD_ARG;
  return attn_entry(q, dtype, k_pages, v_pages, kv_indptr, kv_indices, indices, index_stride, budget,
                    weights, batch, num_q_heads, num_kv_heads, num_pages_total, sm_scale, out,
                    workspace, workspace_bytes, chunk, status, stream);
}

// ---- the same kernel on library-owned scratch ------------------------------------------------
// Some hosts of this library must not allocate device memory at all once they are up: a serving
// process that has handed every free byte to its own pool, or a plugin that is only ever called
// from inside a loop where cudaMalloc is forbidden by policy.  For them the split-KV scratch of
// the attention kernel lives in the library image itself, sized for at most
// TWL_STATIC_ATTN_MAX_ROWS (batch * query heads) rows.
namespace twl {

constexpr size_t kStaticRows = TWL_STATIC_ATTN_MAX_ROWS;
constexpr size_t kStaticCounterBytes = (2 * kStaticRows * sizeof(int32_t) + 255) / 256 * 256;  // counters, group flags
constexpr size_t kStaticMlBytes = (kStaticRows * kMaxChunksPerRow * 2 * sizeof(float) + 255) / 256 * 256;
constexpr size_t kStaticScratchBytes =
    kStaticCounterBytes + kStaticMlBytes + kStaticRows * kMaxChunksPerRow * kD * sizeof(float);

// One copy per GPU that loads the library, held until the process exits.  In host code this name
// is only a handle for cudaGetSymbolAddress; the device address it returns is what kernels get.
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_attn_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
static int static_scratch_for_current_device(void** out) {
  int dev = -1;
  TWL_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TWL_ERR_UNSUPPORTED;
  void* ptr = __atomic_load_n(&g_static_attn_ptr[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    TWL_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_attn_scratch));
    if (ptr == nullptr) return TWL_ERR_LAUNCH;
    __atomic_store_n(&g_static_attn_ptr[dev], ptr, __ATOMIC_RELEASE);  // same value from any thread
  }
  *out = ptr;
  return TWL_OK;
}

}  // namespace twl

extern "C" int twl_sparse_decode_attn_static(const void* q, int dtype, const void* k_pages,
                                             const void* v_pages, const int32_t* kv_indptr,
                                             const int32_t* kv_indices, const int32_t* indices,
                                             int32_t index_stride, const int32_t* budget,
                                             int32_t batch, int32_t num_q_heads,
                                             int32_t num_kv_heads, int32_t num_pages_total,
                                             float sm_scale, void* out, int32_t chunk,
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
  const size_t rows = (size_t)batch * num_q_heads;
  if (rows > kStaticRows) return TWL_ERR_TOO_LARGE;  // the built-in scratch holds no more rows
  if ((int64_t)num_pages_total * num_kv_heads * kPage >= (int64_t)1 << 31) return TWL_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != TWL_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the arrival counters must start at zero
  TWL_CUDA_TRY(cudaMemsetAsync(scratch, 0, kStaticCounterBytes, st));
  AttParams p;
  p.q = q; p.k = k_pages; p.v = v_pages; p.indptr = kv_indptr; p.indices = kv_indices;
  p.idx = indices; p.budget = budget; p.out = out; p.status = status; p.weights = nullptr;
  char* ws = static_cast<char*>(scratch);
  p.counters = reinterpret_cast<int32_t*>(ws);
  const bool lists16 = aligned(indices, 16) && index_stride % 4 == 0;  // the group kernel reads 16-byte pieces
  p.group_flags = (lists16 && group_path_enabled(num_q_heads, num_kv_heads)) ? p.counters + rows : nullptr;
  p.part_ml = reinterpret_cast<float*>(ws + kStaticCounterBytes);
  p.part_o = reinterpret_cast<float*>(ws + kStaticCounterBytes + kStaticMlBytes);
  p.index_stride = index_stride; p.rows = (int)rows; p.Hq = num_q_heads; p.Hkv = num_kv_heads;
  p.num_pages_total = num_pages_total; p.chunk = chunk; p.sm_scale = sm_scale;
  p.max_seq_pages = num_pages_total;
  return launch_attn(p, dtype, rows, index_stride, chunk, false, st);
}
