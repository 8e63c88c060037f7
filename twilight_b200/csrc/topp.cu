// Kernel #2: top-p pruner.
//
// Two forms share one search routine:
//  * twl_top_p_return_mask_{f32,f16}: the reference operator (dense probabilities in,
//    dense 0/1 mask out), csrc/include/sampling.cuh:119-231.
//  * twl_topp_prune: fp32 softmax over the estimator's scores (twilight/pyimpl/top_p.py:11),
//    the same search, then an ordered compaction into a token index list and a budget
//    (replacing the mask AND/sum of twilight/pyimpl/attention.py:280-285).
//
// The search keeps the reference's decisions: low=0, high=x[0] (attention sink), each round
// mid=(low+high)/2, S=sum{x>mid}, a=min({x>low},high), b=max({x<=high},low), low=mid if
// S>=p else high=min(mid,b), until b-a<=1e-5; kept = x>low.  Unlike the reference, which
// re-reads the row from global memory every round with one 1024-thread block, the row is
// staged once into shared memory (it stays there for all rounds and for the compaction),
// the three reductions of a round are fused into one pass, and a round limit replaces the
// open-ended loop.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace twl {

constexpr int kSearchRoundCap = 128;
constexpr float kSearchEps = 1e-5f;
// floats of a row that fit in shared memory next to the reduction scratch
constexpr int kRowCap = 56 * 1024;
// rows of the fused pruner also need the cut list (a quarter of the row, 6 bytes an entry), whose
// memory the block-wide search then works in
constexpr int kPruneRowCap = 40 * 1024;
// elements of a row that one warp searches on its own (see topp_search_solo)
constexpr int kSoloCap = 1024;
constexpr int kPruneHeaderWords = 352 + kSoloCap;  // reduction scratch, scan scratch, short list

template <typename T>
struct Prec;  // rounding of the search scalars to the probability type, as the reference does
template <>
struct Prec<float> {
  static __device__ __forceinline__ float rnd(float x) { return x; }
  static __device__ __forceinline__ float load(const float* p, size_t i) { return p[i]; }
};
template <>
struct Prec<__half> {
  static __device__ __forceinline__ float rnd(float x) { return __half2float(__float2half_rn(x)); }
  static __device__ __forceinline__ float load(const __half* p, size_t i) { return __half2float(p[i]); }
};
template <>
struct Prec<__nv_bfloat16> {
  static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  static __device__ __forceinline__ float load(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
};

struct Red3 {
  float s, a, b;
};

// Block-wide (sum, min, max) in one barrier.  `buf` holds 3*32 floats and must not be the
// buffer used by the previous call (callers alternate two buffers).
template <int THREADS>
__device__ __forceinline__ Red3 block_red3(float s, float a, float b, float* buf) {
  constexpr int NW = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  s = warp_sum(s);
  a = warp_min(a);
  b = warp_max(b);
  if (lane == 0) {
    buf[warp] = s;
    buf[32 + warp] = a;
    buf[64 + warp] = b;
  }
  __syncthreads();
  float s2 = lane < NW ? buf[lane] : 0.f;
  float a2 = lane < NW ? buf[32 + lane] : INFINITY;
  float b2 = lane < NW ? buf[64 + lane] : -INFINITY;
  Red3 r;
  r.s = warp_sum(s2);
  r.a = warp_min(a2);
  r.b = warp_max(b2);
  return r;
}

// Runs the pivot search over x[0..n) (shared or global memory), returns `low`.
// PT = type whose rounding the scalars follow.  red = 2*96 floats of shared scratch.
template <int THREADS, typename PT, typename F>
__device__ float topp_search(F load, int n, float x0, float p_in, float* red, int32_t* status) {
  const float p = Prec<PT>::rnd(p_in);
  const float eps = Prec<PT>::rnd(kSearchEps);
  float low = 0.f, high = x0;
  int round = 0;
  while (true) {
    const float mid = Prec<PT>::rnd(Prec<PT>::rnd(low + high) * 0.5f);
    float s = 0.f, a = high, b = low;
    for (int i = threadIdx.x; i < n; i += THREADS) {
      const float x = load(i);
      s += (x > mid) ? x : 0.f;
      a = (x > low) ? fminf(a, x) : a;
      b = (x <= high) ? fmaxf(b, x) : b;
    }
    Red3 r = block_red3<THREADS>(s, a, b, red + (round & 1) * 96);
    if (Prec<PT>::rnd(r.s) >= p) {
      low = mid;
    } else {
      high = fminf(mid, r.b);
    }
    ++round;
    if (!(Prec<PT>::rnd(r.b - r.a) > eps)) break;
    if (round >= kSearchRoundCap) {
      if (threadIdx.x == 0) raise_flag(status, TWL_FLAG_ITER_CAP);
      break;
    }
  }
  return low;
}

// The search for fp16 / bf16 probabilities, reproducing the reference's arithmetic for that type
// (TopPReturnMaskKernel<..., DType = half or bfloat16>, csrc/include/sampling.cuh:156-217): p, eps,
// low, high, mid and the stop width live in the type, and so does the mass above the pivot, which
// the reference adds with a 1024-thread block reduction per chunk of 1024*VEC elements (VEC =
// gcd(8, d)): every thread adds its VEC consecutive items (two-wide: the items at even and at odd
// positions in order, side by side, then the two sums; in order when there are fewer than four),
// every warp combines its lanes with a shuffle-down tree (offsets 1, 2, 4, 8, 16), thread 0 adds
// the 32 warp totals in order, and the chunk totals are accumulated in order - each addition
// rounded to the type.  That is the order the block reduction of the CUDA 12.9 toolkit's CUB
// produces for 16-bit floats; it is used here too, so the masks are those of the reference's kernel
// built with that toolkit, bit for bit (checked against it on a GPU).  Needs THREADS == 1024.
// red: 192 floats of shared scratch.
template <int THREADS, typename PT, typename F>
__device__ float topp_search_lowp(F load, int d, float x0, float p_in, float* red, int32_t* status) {
  static_assert(THREADS == 1024, "the order of the additions is that of a 1024-thread block");
  const int tx = threadIdx.x, lane = tx & 31, warp = tx >> 5;
  const int vec = (d & 7) == 0 ? 8 : ((d & 3) == 0 ? 4 : ((d & 1) == 0 ? 2 : 1));  // gcd(16 / sizeof, d)
  const int n_chunks = (d + THREADS * vec - 1) / (THREADS * vec);
  float* const wtot = red + 96;  // 32 warp totals, then the running total
  const float p = Prec<PT>::rnd(p_in);
  const float eps = Prec<PT>::rnd(kSearchEps);
  float low = 0.f, high = x0;
  int round = 0;
  while (true) {
    const float mid = Prec<PT>::rnd(Prec<PT>::rnd(low + high) * 0.5f);
    float a = high, b = low;
    float total = 0.f;  // meaningful in thread 0
    for (int c = 0; c < n_chunks; ++c) {
      const int base = (c * THREADS + tx) * vec;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (base < d) {  // d is a multiple of vec: whole groups
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < vec) {
            const float x = load(base + j);
            a = (x > low) ? fminf(a, x) : a;
            b = (x <= high) ? fmaxf(b, x) : b;
            v[j] = (x > mid) ? x : 0.f;
          }
        }
      }
      // a thread's items: even and odd positions are added up side by side (two-wide additions),
      // then the two sums are added; with fewer than four items, in order
      float ts;
      if (vec == 8) {
        const float ev = Prec<PT>::rnd(Prec<PT>::rnd(Prec<PT>::rnd(v[0] + v[2]) + v[4]) + v[6]);
        const float od = Prec<PT>::rnd(Prec<PT>::rnd(Prec<PT>::rnd(v[1] + v[3]) + v[5]) + v[7]);
        ts = Prec<PT>::rnd(ev + od);
      } else if (vec == 4) {
        ts = Prec<PT>::rnd(Prec<PT>::rnd(v[0] + v[2]) + Prec<PT>::rnd(v[1] + v[3]));
      } else if (vec == 2) {
        ts = Prec<PT>::rnd(v[0] + v[1]);
      } else {
        ts = v[0];
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float other = __shfl_down_sync(0xffffffffu, ts, o);
        if (lane + o < 32) ts = Prec<PT>::rnd(ts + other);
      }
      if (lane == 0) wtot[warp] = ts;
      __syncthreads();
      if (tx == 0) {
        float agg = wtot[0];
        for (int w = 1; w < THREADS / 32; ++w) agg = Prec<PT>::rnd(agg + wtot[w]);
        total = Prec<PT>::rnd(total + agg);
      }
      __syncthreads();  // the warp totals are rewritten by the next chunk
    }
    if (tx == 0) wtot[32] = total;
    const Red3 r = block_red3<THREADS>(0.f, a, b, red);  // its barrier also publishes the total
    const float s = wtot[32];
    if (s >= p) {
      low = mid;
    } else {
      high = fminf(mid, r.b);
    }
    ++round;
    __syncthreads();  // everybody has read the reductions before the next round overwrites them
    if (!(Prec<PT>::rnd(r.b - r.a) > eps)) break;
    if (round >= kSearchRoundCap) {
      if (tx == 0) raise_flag(status, TWL_FLAG_ITER_CAP);
      break;
    }
  }
  return low;
}

// Warp-wide inclusive prefix sum of one int per lane.
__device__ __forceinline__ int warp_incl_scan(int v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Block-wide (sum, sum, min, max) in one barrier; buf holds 4*32 floats.
struct Red4 {
  float z, s, a, b;
};
template <int THREADS>
__device__ __forceinline__ Red4 block_red4(float z, float s, float a, float b, float* buf) {
  constexpr int NW = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  z = warp_sum(z);
  s = warp_sum(s);
  a = warp_min(a);
  b = warp_max(b);
  if (lane == 0) {
    buf[warp] = z;
    buf[32 + warp] = s;
    buf[64 + warp] = a;
    buf[96 + warp] = b;
  }
  __syncthreads();
  Red4 r;
  r.z = warp_sum(lane < NW ? buf[lane] : 0.f);
  r.s = warp_sum(lane < NW ? buf[32 + lane] : 0.f);
  r.a = warp_min(lane < NW ? buf[64 + lane] : INFINITY);
  r.b = warp_max(lane < NW ? buf[96 + lane] : -INFINITY);
  return r;
}

// The cut list of the fused pruner: one private segment per warp, holding values and their
// offsets inside the owning warp's slice of the row (so that the kept tokens can be written
// from the list, in row order, without another pass over the row).
struct SearchList {
  float* vals;
  uint16_t* rel;
  int seg_cap;
};

// Walks the entries col[0], col[32], ... col[32 * (cnt - 1)] of a lane's column, `BATCH` loads at a
// time ahead of the calls of f (which may store to entries already read), so that the loads of a
// batch do not wait for one another.  Missing entries of the last batch read as -1, a value outside
// every window of non-negative numbers.
template <int BATCH, typename F>
__device__ __forceinline__ void walk_column(const float* col, int cnt, F f) {
  for (int j0 = 0; j0 < cnt; j0 += BATCH) {
    float e[BATCH];
#pragma unroll
    for (int k = 0; k < BATCH; ++k) e[k] = (j0 + k < cnt) ? col[32 * (j0 + k)] : -1.f;
#pragma unroll
    for (int k = 0; k < BATCH; ++k) f(e[k]);
  }
}

// Block-wide (sum, min, max) of non-negative values in one barrier, three warp-reduce instructions
// a level.  The minimum and the maximum are taken on the bit patterns, which order like the values.
// The sum is taken in fixed point: every lane's partial sum (fp32) is rounded to a multiple of
// total * 2^-30, `total` being the sum of the whole row (no sum of parts exceeds it), and the
// integers are added - exact, so the result does not depend on the order, at a resolution finer
// than the rounding of an fp32 sum of that many terms.  scale = 2^30 / total, inv_scale = 1 / scale.
// `buf` holds 3*32 words and must not be the buffer used by the previous call.
__device__ __forceinline__ unsigned fix_from(float s, float scale) { return __float2uint_rn(s * scale); }
__device__ __forceinline__ float warp_sum_fix(float s, float scale, float inv_scale) {
  return (float)__reduce_add_sync(0xffffffffu, fix_from(s, scale)) * inv_scale;
}
template <int THREADS>
__device__ __forceinline__ Red3 block_red3_pos(float s, float a, float b, float scale, float inv_scale, float* buf) {
  constexpr int NW = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned* ubuf = reinterpret_cast<unsigned*>(buf);
  const unsigned us = __reduce_add_sync(0xffffffffu, fix_from(s, scale));
  const unsigned ua = __reduce_min_sync(0xffffffffu, __float_as_uint(a));
  const unsigned ub = __reduce_max_sync(0xffffffffu, __float_as_uint(b));
  if (lane == 0) {
    ubuf[warp] = us;
    ubuf[32 + warp] = ua;
    ubuf[64 + warp] = ub;
  }
  __syncthreads();
  Red3 r;
  r.s = (float)__reduce_add_sync(0xffffffffu, lane < NW ? ubuf[lane] : 0u) * inv_scale;
  r.a = __uint_as_float(__reduce_min_sync(0xffffffffu, lane < NW ? ubuf[32 + lane] : 0x7f800000u));
  r.b = __uint_as_float(__reduce_max_sync(0xffffffffu, lane < NW ? ubuf[64 + lane] : 0u));
  return r;
}

// The same search with the row in shared memory and a shrinking working set.
//
// A round needs only the elements of the window (low, high]: S sums x > mid, and every x > high is
// above all later pivots too, so its value can be added once and for all to a running sum; a =
// min{x > low} starts at high and b = max{x <= high} starts at low, so elements outside the window
// never move them.  The window halves with every round.  So each lane copies the window elements
// among the ones it reads (four consecutive slots of every 128 of its warp's slice of the row)
// into a column of its own in the warp's part of `region`, adds what lies above the window to its
// share of the running sum, and from then on walks - and keeps squeezing, in place - that column
// instead of the row.  A warp in which some lane's column overflows stays on the row for this
// round and tries again in the next.  Nothing depends on scheduling: every lane's order is fixed.
// The row itself is left as it is (the compaction reads it afterwards).
//
// Starts from the state (low, high, round) the caller hands over (0, x0, 0 for a fresh search; the
// state at which the short-list search below gave up otherwise).
//   x: n non-negative floats (n % 4 == 0); region: NW * seg_floats floats (seg_floats % 32 == 0);
//   red: 192 words; p, eps in the units of x; total = the sum of x.  Returns low.
template <int THREADS>
__device__ float topp_search_window(const float* x, int n, float* region, int seg_floats, float low, float high,
                                    int round, float p, float eps, float total, float* red, int32_t* status) {
  const float scale = 1073741824.f / total, inv_scale = total * (1.f / 1073741824.f);
  constexpr int NW = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slice = ((n + NW - 1) / NW + 127) & ~127;
  const int begin = warp * slice, end = min(n, begin + slice);
  float* const col = region + warp * seg_floats + lane;  // entry j of this lane: col[32 * j]
  const int lane_cap = seg_floats >> 5;
  bool on_list = false;  // warp-uniform
  int cnt = 0;           // entries in this lane's column
  float s_drop = 0.f;    // this lane's share of the sum of everything dropped above the window
  bool first = round == 0;  // the window of a fresh search's first round is (0, x0]: nearly the whole row
  int flip = 0;          // the two reduction buffers alternate
  while (true) {
    const float mid = (low + high) * 0.5f;
    float s, a = high, b = low;
    if (!on_list) {
      s = 0.f;
      float sd = 0.f;
      int w = 0;
      const bool attempt = !first && lane_cap > 0;
      for (int i0 = begin; i0 < end; i0 += 128) {
        const int i = i0 + lane * 4;
        if (i >= end) continue;
        const float4 v = *reinterpret_cast<const float4*>(x + i);  // n % 4 == 0: whole groups
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const bool gh = e[k] > high;
          const bool keep = (e[k] > low) && !gh;
          s += (e[k] > mid) ? e[k] : 0.f;
          a = keep ? fminf(a, e[k]) : a;
          b = keep ? fmaxf(b, e[k]) : b;
          if (attempt) {
            sd += gh ? e[k] : 0.f;
            if (keep) {
              if (w < lane_cap) col[32 * w] = e[k];
              ++w;
            }
          }
        }
      }
      if (attempt && !__any_sync(0xffffffffu, w > lane_cap)) {
        on_list = true;
        cnt = w;
        s_drop = sd;
      }
    } else {
      s = s_drop;
      float sd = s_drop;
      int w = 0;
      walk_column<4>(col, cnt, [&](float e) {
        const bool gh = e > high;
        const bool keep = (e > low) && !gh;
        s += (e > mid) ? e : 0.f;
        sd += gh ? e : 0.f;
        a = keep ? fminf(a, e) : a;
        b = keep ? fmaxf(b, e) : b;
        if (keep) col[32 * w++] = e;  // w never passes the entries already read
      });
      cnt = w;
      s_drop = sd;
    }
    first = false;
    const Red3 r = block_red3_pos<THREADS>(s, a, b, scale, inv_scale, red + flip * 96);
    flip ^= 1;
    if (r.s >= p) {
      low = mid;
    } else {
      high = fminf(mid, r.b);
    }
    ++round;
    if (!(r.b - r.a > eps)) break;
    if (round >= kSearchRoundCap) {
      if (threadIdx.x == 0) raise_flag(status, TWL_FLAG_ITER_CAP);
      break;
    }
  }
  return low;
}

// The search on a short list, run by ONE warp without any block-wide barrier.
//
// While the row is turned into exponentials, every element above cut = x0 / 256 is collected.  As
// long as low is 0 and the pivot stays at or above the cut, and for good once low has risen to a
// pivot >= cut, a round needs nothing else from the row: S sums elements above the pivot; the
// smallest element above low is the row's smallest positive element (low = 0) or a listed one; the
// largest element not above high is a listed one, or the largest unlisted element `b_rest` while
// low is 0 (afterwards unlisted elements lie below low and cannot win).  Rows whose mass sits in a
// few hundred tokens - the case the pruner exists for - are searched entirely here, at a fraction
// of a microsecond per round instead of a block-wide pass.  When the pivot would drop below the
// cut with low still 0 the warp stops and hands its state (low = 0, high, round) to the block.
// Lane-strided sums in a fixed order.  (Squeezing the list to the window (low, high] as the rounds
// go, as the block-wide search does, made this search slower: its lists shrink only in the last
// rounds, and the bookkeeping doubles the work per element before that.)
struct SoloState {
  float low, high;
  int round, done;
};
__device__ __forceinline__ SoloState topp_search_solo(const float* solo, int n_solo, float x0, float cut,
                                                      float a_pos, float b_rest, float p, float eps,
                                                      float total, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const float scale = 1073741824.f / total, inv_scale = total * (1.f / 1073741824.f);
  SoloState st;
  st.low = 0.f; st.high = x0; st.round = 0; st.done = 0;
  while (true) {
    const float low = st.low, high = st.high;
    const float mid = (low + high) * 0.5f;
    if (low == 0.f && mid < cut) break;  // the block takes over from this state
    float s = 0.f, a = high, b = low;
    for (int i = lane; i < n_solo; i += 32) {
      const float e = solo[i];
      s += (e > mid) ? e : 0.f;
      a = (e > low) ? fminf(a, e) : a;
      b = (e <= high) ? fmaxf(b, e) : b;
    }
    s = warp_sum_fix(s, scale, inv_scale);  // fixed point, as in block_red3_pos
    a = __uint_as_float(__reduce_min_sync(0xffffffffu, __float_as_uint(a)));  // non-negative values
    b = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(b)));
    if (low == 0.f) {
      a = fminf(a, a_pos);   // smallest positive element of the whole row (a_pos <= high always)
      b = fmaxf(b, b_rest);  // largest unlisted element: b_rest <= cut <= mid < high
    }
    if (s >= p) {
      st.low = mid;
    } else {
      st.high = fminf(mid, b);
    }
    ++st.round;
    if (!(b - a > eps)) {
      st.done = 1;
      break;
    }
    if (st.round >= kSearchRoundCap) {
      if (lane == 0) raise_flag(status, TWL_FLAG_ITER_CAP);
      st.done = 1;
      break;
    }
  }
  return st;
}

// The same short-list search run by the whole block: every warp walks its own segment of the cut
// list where it lies (`my_val`, `my_cnt` entries; the list stays as it is, the compaction reads it)
// and a round costs one block-wide reduction.  For blocks that have an SM to themselves - there
// one warp searching alone would leave the other schedulers idle - and for lists of any length.
template <int THREADS>
__device__ SoloState topp_search_cut_list(const float* my_val, int my_cnt, float x0, float cut, float a_pos,
                                          float b_rest, float p, float eps, float total, float* red,
                                          int32_t* status) {
  const int lane = threadIdx.x & 31;
  const float scale = 1073741824.f / total, inv_scale = total * (1.f / 1073741824.f);
  SoloState st;
  st.low = 0.f; st.high = x0; st.round = 0; st.done = 0;
  int flip = 0;
  while (true) {
    const float low = st.low, high = st.high;
    const float mid = (low + high) * 0.5f;
    if (low == 0.f && mid < cut) break;  // the search over the whole row takes over from this state
    float s = 0.f, a = high, b = low;
    for (int i = lane; i < my_cnt; i += 32) {
      const float e = my_val[i];
      s += (e > mid) ? e : 0.f;
      a = (e > low) ? fminf(a, e) : a;
      b = (e <= high) ? fmaxf(b, e) : b;
    }
    Red3 r = block_red3_pos<THREADS>(s, a, b, scale, inv_scale, red + flip * 96);
    flip ^= 1;
    if (low == 0.f) {
      r.a = fminf(r.a, a_pos);
      r.b = fmaxf(r.b, b_rest);
    }
    if (r.s >= p) {
      st.low = mid;
    } else {
      st.high = fminf(mid, r.b);
    }
    ++st.round;
    if (!(r.b - r.a > eps)) {
      st.done = 1;
      break;
    }
    if (st.round >= kSearchRoundCap) {
      if (threadIdx.x == 0) raise_flag(status, TWL_FLAG_ITER_CAP);
      st.done = 1;
      break;
    }
  }
  return st;
}

// ---- dense mask form ------------------------------------------------------------------------
template <int THREADS, typename T, bool IN_SMEM>
__global__ void __launch_bounds__(THREADS)
top_p_mask_kernel(const T* __restrict__ probs, uint8_t* __restrict__ mask,
                  const float* __restrict__ top_p_arr, float top_p_val, uint32_t d,
                  int32_t* status) {
  extern __shared__ __align__(16) float smem[];
  float* red = smem;        // 192 floats
  float* row = smem + 192;  // d floats when IN_SMEM
  const size_t base = (size_t)blockIdx.x * d;
  const float p = top_p_arr ? top_p_arr[blockIdx.x] : top_p_val;
  const T* src = probs + base;
  if (IN_SMEM) {
    for (uint32_t i = threadIdx.x; i < d; i += THREADS) row[i] = Prec<T>::load(src, i);
    __syncthreads();
  }
  const float x0 = IN_SMEM ? row[0] : Prec<T>::load(src, 0);
  float low;
  if constexpr (sizeof(T) == 2) {
    if (IN_SMEM) {
      low = topp_search_lowp<THREADS, T>([&](int i) { return row[i]; }, (int)d, x0, p, red, status);
    } else {
      low = topp_search_lowp<THREADS, T>([&](int i) { return Prec<T>::load(src, i); }, (int)d, x0, p, red, status);
    }
  } else if (IN_SMEM) {
    low = topp_search<THREADS, T>([&](int i) { return row[i]; }, (int)d, x0, p, red, status);
  } else {
    low = topp_search<THREADS, T>([&](int i) { return Prec<T>::load(src, i); }, (int)d, x0, p, red, status);
  }
  uint8_t* dst = mask + base;
  if ((d & 3u) == 0 && ((reinterpret_cast<uintptr_t>(dst) & 3u) == 0)) {
    uint32_t* dst4 = reinterpret_cast<uint32_t*>(dst);
    for (uint32_t i = threadIdx.x; i < d / 4; i += THREADS) {
      uint32_t m = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x = IN_SMEM ? row[4 * i + k] : Prec<T>::load(src, 4 * i + k);
        m |= (x > low ? 1u : 0u) << (8 * k);
      }
      dst4[i] = m;
    }
  } else {
    for (uint32_t i = threadIdx.x; i < d; i += THREADS) {
      const float x = IN_SMEM ? row[i] : Prec<T>::load(src, i);
      dst[i] = x > low ? 1 : 0;
    }
  }
}

template <typename T>
static int launch_mask(const T* probs, uint8_t* mask, const float* top_p_arr, float top_p_val,
                       uint32_t rows, uint32_t d, int32_t* status, cudaStream_t st) {
  constexpr int THREADS = 1024;
  if (d <= (uint32_t)kRowCap) {
    const size_t smem = (192 + (size_t)d) * sizeof(float);
    auto kern = top_p_mask_kernel<THREADS, T, true>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<rows, THREADS, smem, st>>>(probs, mask, top_p_arr, top_p_val, d, status);
  } else {
    auto kern = top_p_mask_kernel<THREADS, T, false>;
    kern<<<rows, THREADS, 192 * sizeof(float), st>>>(probs, mask, top_p_arr, top_p_val, d, status);
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

// ---- fused softmax + search + compaction ---------------------------------------------------
struct PruneParams {
  const float* scores;
  const int32_t* indptr;
  const int32_t* last_len;
  const int32_t* cand_pages;
  const int32_t* cand_npages;
  const float* top_p_arr;
  int32_t* out_indices;
  int32_t* out_budget;
  float* out_threshold;
  float* out_weights;  // [rows][index_stride] un-normalised softmax weight of each kept token, or nullptr
  int32_t* status;
  int stride, max_k, B, Hq, index_stride, row_cap, list_cap, seg_floats;
  int mode;  // 0: softmax + top-p search; 1: keep scores above (score of token 0) - top_p_val
  float top_p_val;
};

template <int THREADS, bool IN_SMEM>
__global__ void __launch_bounds__(THREADS, THREADS == 1024 ? 1 : THREADS == 512 ? 3 : 5)
topp_prune_kernel(const PruneParams p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int NW = THREADS / 32;
  float* red = smem;                                  // 256 words
  int* wsum = reinterpret_cast<int*>(smem + 256);     // 96 ints: 33 of scan scratch, 32 segment counts
  float* solo = smem + 352;                           // kSoloCap values: the short list one warp searches
  float* row = smem + kPruneHeaderWords;              // the row when IN_SMEM, then the cut list / search area
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_release();  // the attention kernel's blocks may move in while this small grid works
  const int r = blockIdx.x;
  const int b = r / p.Hq;
  const bool has_cand = p.cand_pages != nullptr;
  pdl_wait();  // scores and candidate lists come from the kernels launched before; nothing is read earlier
  const int n_seq_pages = p.indptr[b + 1] - p.indptr[b];
  int n_pages = has_cand ? min(p.cand_npages[r], p.max_k) : n_seq_pages;
  n_pages = min(n_pages, p.stride / kPage);
  const int n = n_pages * kPage;  // candidate slots; slots past the sequence end hold -inf
  const int32_t* cand = has_cand ? p.cand_pages + (size_t)r * p.max_k : nullptr;
  const float* src = p.scores + (size_t)r * p.stride;
  if (n == 0) {
    if (threadIdx.x == 0) {
      p.out_budget[r] = 0;
      if (p.out_threshold) {
        p.out_threshold[2 * r] = 0.f;
        p.out_threshold[2 * r + 1] = 0.f;
      }
    }
    return;
  }
  // every warp owns a contiguous slice of the row (whole groups of four slots per lane)
  const int slice = ((n + NW - 1) / NW + 127) & ~127;
  const int s_begin = warp * slice, s_end = min(n, s_begin + slice);
  // pass 1: row maximum (and stage the scores)
  float m = -INFINITY;
  {
    const float4* s4 = reinterpret_cast<const float4*>(src);  // stride and n are multiples of 16
    float4* r4 = reinterpret_cast<float4*>(row);
    // all loads of a row in shared memory are issued before the first is used: a block that has
    // its SM to itself has nothing else to hide their latency behind
    constexpr int kLd = !IN_SMEM ? 4 : THREADS == 1024 ? 10 : 4;
    const int n4 = n / 4;
    for (int i0 = threadIdx.x; i0 < n4; i0 += kLd * THREADS) {
      float4 v[kLd];
#pragma unroll
      for (int k = 0; k < kLd; ++k)
        if (i0 + k * THREADS < n4) v[k] = s4[i0 + k * THREADS];
#pragma unroll
      for (int k = 0; k < kLd; ++k) {
        if (i0 + k * THREADS < n4) {
          if (IN_SMEM) r4[i0 + k * THREADS] = v[k];
          m = fmaxf(fmaxf(m, fmaxf(v[k].x, v[k].y)), fmaxf(v[k].z, v[k].w));
        }
      }
    }
  }
  Red3 r1 = block_red3<THREADS>(0.f, 0.f, m, red);
  m = r1.b;
  __syncthreads();
  const float kLog2e = 1.4426950408889634f;
  const float m2 = m * kLog2e;
  // exp(s-m) = 2^(s*log2e - m*log2e): one FMA and one ex2.approx (2 ulp, subnormal results kept
  // so that "probability > 0" means what it says)
  auto fexp = [&](float sc) -> float {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(fmaf(sc, kLog2e, -m2)));
    return y;
  };
  const bool thresh_mode = p.mode == 1;
  // token 0 of the sequence: slot 0 when page 0 is a candidate, else it is not in the row
  const bool sink_present = has_cand ? (cand[0] == 0) : true;
  const float top_p = p.top_p_arr ? p.top_p_arr[r] : p.top_p_val;
  // x0 and low are in the units of what the row holds at emission time: raw scores in threshold
  // mode, un-normalised exponentials for a row in shared memory (unit = 1/inv_z), probabilities
  // for a row read from global memory
  float x0, low, inv_z = 1.f;
  bool from_list = false;
  int list_cnt = 0;
  SearchList L;
  L.seg_cap = (p.list_cap / NW) & ~3;
  L.vals = row + p.row_cap;
  L.rel = reinterpret_cast<uint16_t*>(L.vals + p.list_cap);
  auto prob = [&](int i) -> float {  // rows in global memory only
    return thresh_mode ? src[i] : fexp(src[i]) * inv_z;
  };
  if (thresh_mode) {
    // twilight/pyimpl/elementwise_threshold.py:15-17: weights > weight[0] - threshold; a token 0
    // outside the candidates holds the dtype's minimum there, so every candidate passes
    x0 = sink_present ? (IN_SMEM ? row[0] : src[0]) : -INFINITY;
    low = sink_present ? x0 - top_p : -INFINITY;
  } else if (IN_SMEM) {
    // pass 2: exponentials in place and their sum.  The search runs on the un-normalised values
    // (p and the stop width scaled by the sum instead of every element divided by it).  The same
    // pass collects every element above x0/256 into the cut list, with the smallest positive
    // element and the largest element that was not collected: what the short-list search needs.
    x0 = sink_present ? fexp(row[0]) : 0.f;
    __syncthreads();  // row[0] is read by everyone before its owner overwrites it
    const float cut = x0 * (1.f / 256.f);
    float z = 0.f, a1 = x0, b1 = 0.f;
    int first_cnt = 0;
    float* const my_val = L.vals + warp * L.seg_cap;
    uint16_t* const my_rel = L.rel + warp * L.seg_cap;
    for (int i0 = s_begin; i0 < s_end; i0 += 128) {
      const int i = i0 + lane * 4;
      float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);  // exp gives 0
      if (i < s_end) v = *reinterpret_cast<const float4*>(row + i);
      v.x = fexp(v.x); v.y = fexp(v.y); v.z = fexp(v.z); v.w = fexp(v.w);
      if (i < s_end) *reinterpret_cast<float4*>(row + i) = v;
      const float e[4] = {v.x, v.y, v.z, v.w};
      z += (v.x + v.y) + (v.z + v.w);
      if (first_cnt > L.seg_cap) continue;  // the list has overflowed: this row goes to the block-wide search
      int c = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        a1 = (e[k] > 0.f) ? fminf(a1, e[k]) : a1;
        b1 = (e[k] <= cut) ? fmaxf(b1, e[k]) : b1;
        c += e[k] > cut ? 1 : 0;
      }
      if (__ballot_sync(0xffffffffu, c > 0) == 0) continue;
      const int inc = warp_incl_scan(c);
      int pos = first_cnt + inc - c;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (e[k] > cut) {
          if (pos < L.seg_cap) {
            my_val[pos] = e[k];
            my_rel[pos] = (uint16_t)(i - s_begin + k);
          }
          ++pos;
        }
      }
      first_cnt += __shfl_sync(0xffffffffu, inc, 31);
    }
    const Red4 r2 = block_red4<THREADS>(z, 0.f, a1, b1, red + 96);  // sum, -, smallest positive, largest uncollected
    inv_z = 1.f / r2.z;
    if (top_p > 1.f) {
      low = 0.f;  // no pruning asked for: keep every candidate with non-zero probability
    } else {
      const float p_z = top_p * r2.z, eps_z = kSearchEps * r2.z;
      int* const seg_cnt = wsum + 40;
      if (lane == 0) seg_cnt[warp] = first_cnt;
      __syncthreads();
      bool fits = true;
      int total = 0, my_off = 0;
#pragma unroll 1
      for (int w = 0; w < NW; ++w) {
        const int cw = seg_cnt[w];
        fits = fits && (cw <= L.seg_cap);
        my_off += w < warp ? cw : 0;
        total += cw;
      }
      float lo0 = 0.f, hi0 = x0;
      int round0 = 0;
      bool done = false;
      if (THREADS == 1024 && fits) {
        // this block has its SM to itself: all warps run the rounds, each on its own segment
        __syncthreads();  // seg_cnt has been read by everyone; red is free
        const SoloState st = topp_search_cut_list<THREADS>(my_val, first_cnt, x0, cut, r2.a, r2.b, p_z, eps_z, r2.z,
                                                           red, p.status);
        lo0 = st.low;
        hi0 = st.high;
        round0 = st.round;
        done = st.done != 0;
      } else if (fits && total <= kSoloCap) {
        // the collected elements side by side, then one warp runs the rounds on them alone
        for (int i = lane; i < first_cnt; i += 32) solo[my_off + i] = my_val[i];
        __syncthreads();
        if (warp == 0) {
          const SoloState st = topp_search_solo(solo, total, x0, cut, r2.a, r2.b, p_z, eps_z, r2.z, p.status);
          if (lane == 0) {
            red[0] = st.low;
            red[1] = st.high;
            red[2] = __int_as_float(st.round);
            red[3] = __int_as_float(st.done);
          }
        }
        __syncthreads();
        lo0 = red[0];
        hi0 = red[1];
        round0 = __float_as_int(red[2]);
        done = __float_as_int(red[3]) != 0;
      }
      __syncthreads();  // seg_cnt and red are reused by the block-wide search
      if (done) {
        // A low that has risen is a pivot >= the collection cut: every element above it is in the
        // list, each warp's segment in row order.  A search that ended with low still 0 (the mass
        // above every pivot stayed below p until the window closed) keeps every positive element,
        // listed or not: those come from the row.
        low = lo0;
        from_list = lo0 > 0.f;
        list_cnt = first_cnt;
      } else {
        // the cut list is dead from here on: its memory is the working area of the block-wide search
        low = topp_search_window<THREADS>(row, n, L.vals, p.seg_floats, lo0, hi0, round0, p_z, eps_z, r2.z, red,
                                          p.status);
      }
    }
  } else {
    float z = 0.f;
    for (int i = threadIdx.x; i < n; i += THREADS) z += fexp(src[i]);
    Red3 r2 = block_red3<THREADS>(z, 0.f, 0.f, red + 96);
    inv_z = 1.f / r2.s;
    __syncthreads();
    x0 = sink_present ? prob(0) : 0.f;
    low = top_p > 1.f ? 0.f : topp_search<THREADS, float>(prob, n, x0, top_p, red, p.status);
  }
  __syncthreads();
  // ordered compaction: the warps count the kept slots of their slices, the counts are
  // prefix-summed once, then each warp writes its tokens in order
  const float out_scale = (IN_SMEM && !thresh_mode) ? inv_z : 1.f;
  int32_t* out = p.out_indices + (size_t)r * p.index_stride;
  float* out_w = p.out_weights ? p.out_weights + (size_t)r * p.index_stride : nullptr;
  int base;
  if (IN_SMEM && from_list) {
    // everything above `low` is in the list, each warp's segment in row order
    const float* my_val = L.vals + warp * L.seg_cap;
    const uint16_t* my_rel = L.rel + warp * L.seg_cap;
    int my_cnt = 0;
    for (int i0 = 0; i0 < list_cnt; i0 += 32) {
      const bool keep = (i0 + lane < list_cnt) && (my_val[i0 + lane] > low);
      my_cnt += __popc(__ballot_sync(0xffffffffu, keep));
    }
    if (lane == 0) wsum[warp] = my_cnt;
    __syncthreads();
    const int inc_w = warp_incl_scan(lane < NW ? wsum[lane] : 0);
    base = __shfl_sync(0xffffffffu, inc_w, NW - 1);
    int off = __shfl_sync(0xffffffffu, inc_w, warp) - my_cnt;
    for (int i0 = 0; i0 < list_cnt; i0 += 32) {
      const bool in = i0 + lane < list_cnt;
      const float e = in ? my_val[i0 + lane] : 0.f;
      const bool keep = in && e > low;
      const unsigned mk = __ballot_sync(0xffffffffu, keep);
      const int pos = off + __popc(mk & ((1u << lane) - 1));
      if (keep && pos < p.index_stride) {
        const int i = s_begin + my_rel[i0 + lane];
        const int page = has_cand ? cand[i / kPage] : (i / kPage);
        out[pos] = page * kPage + (i % kPage);
        if (out_w) out_w[pos] = e * out_scale;
      }
      off += __popc(mk);
    }
  } else if (IN_SMEM) {
    // four consecutive slots per lane (n is a multiple of 16, so groups never straddle the end)
    int my_cnt = 0;
    for (int i0 = s_begin; i0 < s_end; i0 += 128) {
      const int i = i0 + lane * 4;
      if (i < s_end) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        my_cnt += (v.x > low) + (v.y > low) + (v.z > low) + (v.w > low);
      }
    }
    my_cnt = warp_sum_i(my_cnt);
    if (lane == 0) wsum[warp] = my_cnt;
    __syncthreads();
    const int inc_w = warp_incl_scan(lane < NW ? wsum[lane] : 0);
    base = __shfl_sync(0xffffffffu, inc_w, NW - 1);                // kept tokens of the row
    int off = __shfl_sync(0xffffffffu, inc_w, warp) - my_cnt;      // exclusive prefix of this warp
    // a run of 128 slots is first looked at four slots per lane; where it holds kept tokens it is
    // walked again one slot per lane, so that a warp's stores go to consecutive addresses
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int i0 = s_begin; i0 < s_end; i0 += 128) {
      const int i = i0 + lane * 4;
      float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);  // never above any cut
      if (i < s_end) v = *reinterpret_cast<const float4*>(row + i);
      const bool any = (v.x > low) || (v.y > low) || (v.z > low) || (v.w > low);
      if (__ballot_sync(0xffffffffu, any) == 0) continue;
      // (no branches below: the four sub-steps' loads are issued together)
      float e[4];
      int page[4];
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
        const int j = i0 + sub * 32 + lane;
        e[sub] = j < s_end ? row[j] : -INFINITY;
        page[sub] = (has_cand && j < s_end) ? cand[j / kPage] : (j / kPage);
      }
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
        const int j = i0 + sub * 32 + lane;
        const bool keep = e[sub] > low;
        const unsigned mk = __ballot_sync(0xffffffffu, keep);
        const int pos = off + __popc(mk & lt_mask);
        if (keep && pos < p.index_stride) {
          out[pos] = page[sub] * kPage + (j % kPage);
          if (out_w) out_w[pos] = thresh_mode ? fexp(e[sub]) : e[sub] * out_scale;
        }
        off += __popc(mk);
      }
    }
  } else {
    int my_cnt = 0;
    for (int i0 = s_begin; i0 < s_end; i0 += 32) {
      const bool keep = (i0 + lane < s_end) && (prob(i0 + lane) > low);
      my_cnt += __popc(__ballot_sync(0xffffffffu, keep));
    }
    if (lane == 0) wsum[warp] = my_cnt;
    __syncthreads();
    const int inc_w = warp_incl_scan(lane < NW ? wsum[lane] : 0);
    base = __shfl_sync(0xffffffffu, inc_w, NW - 1);
    int off = __shfl_sync(0xffffffffu, inc_w, warp) - my_cnt;
    for (int i0 = s_begin; i0 < s_end; i0 += 32) {
      const int i = i0 + lane;
      const bool keep = (i < s_end) && (prob(i) > low);
      const unsigned mk = __ballot_sync(0xffffffffu, keep);
      const int pos = off + __popc(mk & ((1u << lane) - 1));
      if (keep && pos < p.index_stride) {
        const int page = has_cand ? cand[i / kPage] : (i / kPage);
        out[pos] = page * kPage + (i % kPage);
        if (out_w) out_w[pos] = thresh_mode ? fexp(prob(i)) : prob(i);
      }
      off += __popc(mk);
    }
  }
  if (threadIdx.x == 0) {
    if (base > p.index_stride) raise_flag(p.status, TWL_FLAG_BAD_INDEX);
    p.out_budget[r] = min(base, p.index_stride);
    if (p.out_threshold) {
      p.out_threshold[2 * r] = low * out_scale;
      p.out_threshold[2 * r + 1] = x0 * out_scale;
    }
  }
}

template <int THREADS>
static int launch_prune(const PruneParams& p, int rows, int n_max, cudaStream_t st) {
  if (n_max <= kPruneRowCap) {
    constexpr int NW = THREADS / 32;
    constexpr size_t kSmemMax = 227 * 1024, kPerBlockReserve = 1024;
    PruneParams q = p;
    q.row_cap = (n_max + 3) & ~3;
    q.list_cap = (std::max(q.row_cap / 4, 32 * NW) + 63) & ~63;  // entries: a float and a uint16 each
    const size_t fixed = (kPruneHeaderWords + (size_t)q.row_cap) * sizeof(float);
    const size_t list_bytes = (size_t)q.list_cap * 6;
    // The block-wide search works in the cut list's memory; a block that has its SM to itself
    // anyway gets what is left of the SM's shared memory for it, up to one float per slot of the row.
    const int per_sm = (int)std::min<size_t>(2048 / THREADS, kSmemMax / (fixed + list_bytes + kPerBlockReserve));
    if (per_sm < 1) return TWL_ERR_TOO_LARGE;
    const size_t room = per_sm == 1 ? kSmemMax - kPerBlockReserve - fixed : list_bytes;
    const size_t region = std::max(list_bytes, std::min(room, (size_t)q.row_cap * sizeof(float)));
    q.seg_floats = (int)(region / sizeof(float) / NW) & ~31;
    const size_t smem = (fixed + region + 15) & ~(size_t)15;
    auto kern = topp_prune_kernel<THREADS, true>;
    TWL_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TWL_CUDA_TRY(launch_chain(kern, dim3(rows), dim3(THREADS), smem, st, static_cast<const PruneParams&>(q)));
  } else {
    PruneParams q = p;
    q.seg_floats = 0;
    auto kern = topp_prune_kernel<THREADS, false>;
    TWL_CUDA_TRY(launch_chain(kern, dim3(rows), dim3(THREADS), kPruneHeaderWords * sizeof(float), st,
                              static_cast<const PruneParams&>(q)));
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

}  // namespace twl

extern "C" int twl_top_p_return_mask_f32(const float* probs, uint8_t* mask,
                                         const float* top_p_arr, float top_p_val, uint32_t rows,
                                         uint32_t d, int32_t* status, void* stream) {
  if (!probs || !mask || rows == 0 || d == 0) return TWL_ERR_BAD_ARG;
  if (d > 0x7fffffffu) return TWL_ERR_TOO_LARGE;
  return twl::launch_mask<float>(probs, mask, top_p_arr, top_p_val, rows, d, status,
                                 reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int twl_top_p_return_mask_f16(const void* probs, int dtype, uint8_t* mask,
                                         const float* top_p_arr, float top_p_val, uint32_t rows,
                                         uint32_t d, int32_t* status, void* stream) {
  if (!probs || !mask || rows == 0 || d == 0) return TWL_ERR_BAD_ARG;
  if (d > 0x7fffffffu) return TWL_ERR_TOO_LARGE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16)
    return twl::launch_mask<__half>(static_cast<const __half*>(probs), mask, top_p_arr, top_p_val,
                                    rows, d, status, st);
  if (dtype == TWL_BF16)
    return twl::launch_mask<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(probs), mask,
                                           top_p_arr, top_p_val, rows, d, status, st);
  return TWL_ERR_UNSUPPORTED;
}

namespace twl {
static int run_prune(PruneParams& p, int batch, int num_q_heads, int score_stride, const int32_t* cand_pages,
                     int max_k, cudaStream_t st) {
  const int rows = batch * num_q_heads;
  const int n_max = cand_pages ? (int)std::min<int64_t>((int64_t)max_k * kPage, score_stride)
                               : score_stride;
  // one block per row.  More threads per row shorten a row's latency, but only pay while all rows
  // still run at the same time (3 blocks of 512 threads per SM, 6 of 256): a second wave costs more.
  // (Four blocks of 512 threads fit an SM only at 32 registers a thread; the spills that costs made
  // the pruner slower: 30.9 against 24.6 us on 512 rows of 8192 slots with budgets near 330.)
  const bool one_wave_512 = rows <= 3 * num_sms();
  const bool one_wave_1024 = rows <= num_sms();
  // TWL_PRUNE_THREADS=256|512|1024 forces the block size where the row fits (for measurement)
  static const int forced = [] {
    const char* e = getenv("TWL_PRUNE_THREADS");
    return e ? atoi(e) : 0;
  }();
  if (forced == 256 && n_max <= 8192) return launch_prune<256>(p, rows, n_max, st);
  if (forced == 512 && n_max <= 16384) return launch_prune<512>(p, rows, n_max, st);
  if (forced == 1024) return launch_prune<1024>(p, rows, n_max, st);
  if (n_max <= 2048) return launch_prune<256>(p, rows, n_max, st);
  if (n_max <= 8192) return one_wave_512 ? launch_prune<512>(p, rows, n_max, st) : launch_prune<256>(p, rows, n_max, st);
  if (n_max <= 16384) return one_wave_1024 ? launch_prune<1024>(p, rows, n_max, st) : launch_prune<512>(p, rows, n_max, st);
  return launch_prune<1024>(p, rows, n_max, st);
}

static int prune_entry(int mode, const float* scores, int32_t score_stride, const int32_t* kv_indptr,
                       const int32_t* kv_last_page_len, const int32_t* cand_pages,
                       const int32_t* cand_npages, int32_t max_k, int32_t batch, int32_t num_q_heads,
                       const float* arr, float val, int32_t* out_indices, int32_t index_stride,
                       int32_t* out_budget, float* out_threshold, float* out_weights, int32_t* status,
                       void* stream) {
  if (!scores || !kv_indptr || !out_indices || !out_budget) return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_q_heads <= 0 || score_stride <= 0 || index_stride <= 0)
    return TWL_ERR_BAD_ARG;
  if (score_stride % kPage != 0) return TWL_ERR_BAD_ARG;
  if (cand_pages && (!cand_npages || max_k <= 0)) return TWL_ERR_BAD_ARG;
  if (!aligned(scores, 16)) return TWL_ERR_MISALIGNED;
  PruneParams p;
  p.scores = scores; p.indptr = kv_indptr; p.last_len = kv_last_page_len;
  p.cand_pages = cand_pages; p.cand_npages = cand_npages; p.top_p_arr = arr;
  p.out_indices = out_indices; p.out_budget = out_budget; p.out_threshold = out_threshold;
  p.out_weights = out_weights;
  p.status = status; p.stride = score_stride; p.max_k = max_k; p.B = batch; p.Hq = num_q_heads;
  p.index_stride = index_stride; p.top_p_val = val; p.mode = mode;
  return run_prune(p, batch, num_q_heads, score_stride, cand_pages, max_k,
                   reinterpret_cast<cudaStream_t>(stream));
}
}  // namespace twl

extern "C" int twl_topp_prune(const float* scores, int32_t score_stride,
                              const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                              const int32_t* cand_pages, const int32_t* cand_npages,
                              int32_t max_k, int32_t batch, int32_t num_q_heads,
                              const float* top_p_arr, float top_p_val, int32_t* out_indices,
                              int32_t index_stride, int32_t* out_budget, float* out_threshold,
                              int32_t* status, void* stream) {
  return twl::prune_entry(0, scores, score_stride, kv_indptr, kv_last_page_len, cand_pages, cand_npages,
                          max_k, batch, num_q_heads, top_p_arr, top_p_val, out_indices, index_stride,
                          out_budget, out_threshold, nullptr, status, stream);
}

extern "C" int twl_prune_with_weights(int32_t mode, const float* scores, int32_t score_stride,
                                      const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                      const int32_t* cand_pages, const int32_t* cand_npages,
                                      int32_t max_k, int32_t batch, int32_t num_q_heads,
                                      const float* top_p_arr, float value, int32_t* out_indices,
                                      int32_t index_stride, int32_t* out_budget, float* out_threshold,
                                      float* out_weights, int32_t* status, void* stream) {
  if (mode != 0 && mode != 1) return TWL_ERR_BAD_ARG;
  if (!out_weights) return TWL_ERR_BAD_ARG;
  return twl::prune_entry(mode, scores, score_stride, kv_indptr, kv_last_page_len, cand_pages,
                          cand_npages, max_k, batch, num_q_heads, mode == 0 ? top_p_arr : nullptr, value,
                          out_indices, index_stride, out_budget, out_threshold, out_weights, status,
                          stream);
}

extern "C" int twl_threshold_prune(const float* scores, int32_t score_stride,
                                   const int32_t* kv_indptr, const int32_t* kv_last_page_len,
                                   const int32_t* cand_pages, const int32_t* cand_npages,
                                   int32_t max_k, int32_t batch, int32_t num_q_heads, float threshold,
                                   int32_t* out_indices, int32_t index_stride, int32_t* out_budget,
                                   float* out_threshold, int32_t* status, void* stream) {
  return twl::prune_entry(1, scores, score_stride, kv_indptr, kv_last_page_len, cand_pages, cand_npages,
                          max_k, batch, num_q_heads, nullptr, threshold, out_indices, index_stride,
                          out_budget, out_threshold, nullptr, status, stream);
}
