// Shared device/host helpers for the twilight_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/twilight_b200.h"

namespace twl {

constexpr int kPage = TWL_PAGE_SIZE;        // tokens per page
constexpr int kD = TWL_HEAD_DIM;            // head dimension
constexpr int kGroup = TWL_QUANT_GROUP;     // channels per quantisation group
constexpr int kSlab = TWL_K4_SLAB_BYTES;    // bytes of one INT4 (page, kv-head) slab
constexpr int kSlabCodes = kPage * kD / 2;  // 1024 code bytes, then 256 bytes of scale/min

// Streaming multiprocessors of the current device (queried once per device, then cached).
int num_sms();

// Records the last CUDA launch error for twl_last_cuda_error().
void set_last_cuda_error(cudaError_t e);

#define TWL_CHECK_LAUNCH()                         \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) {                      \
      ::twl::set_last_cuda_error(e__);             \
      return TWL_ERR_LAUNCH;                       \
    }                                              \
  } while (0)

#define TWL_CUDA_TRY(expr)                         \
  do {                                             \
    cudaError_t e__ = (expr);                      \
    if (e__ != cudaSuccess) {                      \
      ::twl::set_last_cuda_error(e__);             \
      return TWL_ERR_LAUNCH;                       \
    }                                              \
  } while (0)

// ---- programmatic dependent launch ---------------------------------------------------------------
// The kernels of a decode step depend on each other in a chain.  Launched with the programmatic
// stream-serialisation attribute, the next kernel of the chain may be set up and may run its own
// prologue (reading q, the page table) while the previous one drains; it calls pdl_wait() before it
// touches anything the previous kernel wrote.  Without the attribute the call does nothing.
// The two small grids in front of a streaming kernel (page top-k, pruner) also release their
// dependents at block start (pdl_release), so the next kernel's blocks are resident and past their
// prologue when the small grid ends: 0.7 % per step.  The streaming kernels and the attention
// kernel do not: their dependents' waiting blocks crowd them (9 % slower when every kernel did it,
// 6 % slower for the attention kernel alone).
bool pdl_enabled();  // TWL_PDL=0 in the environment switches it off

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename Params>
inline cudaError_t launch_chain(void (*kernel)(Params), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t st, const Params& params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, params);
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- element type traits ---------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float2 to_f2(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
  }
};
template <>
struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float2 to_f2(uint32_t u) {
    // bf16 -> fp32 is a 16-bit shift
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
};

// ---- warp / block reductions -------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide exclusive prefix sum of one int per thread; *total gets the block sum.
// wsum: 33 ints of shared scratch.  Ends with a barrier, so it can be called in a loop.
template <int THREADS>
__device__ __forceinline__ int block_excl_scan(int v, int* total, int* wsum) {
  constexpr int NW = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < NW ? wsum[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < NW) wsum[lane] = winc - w;
    if (lane == 31) wsum[32] = winc;
  }
  __syncthreads();
  const int r = wsum[warp] + inc - v;
  *total = wsum[32];
  __syncthreads();
  return r;
}

__device__ __forceinline__ void raise_flag(int32_t* status, int flag) {
  if (status != nullptr) atomicOr(status, flag);
}

// 128-bit read-only global load that does not allocate in L1 (streamed once).
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
// Two block-wide exclusive prefix sums in the same barriers.  wsum: 66 ints of shared scratch.
template <int THREADS>
__device__ __forceinline__ void block_excl_scan2(int a, int b, int* ea, int* eb, int* ta, int* tb, int* wsum) {
  constexpr int NW = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int ia = a, ib = b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int x = __shfl_up_sync(0xffffffffu, ia, o), y = __shfl_up_sync(0xffffffffu, ib, o);
    if (lane >= o) {
      ia += x;
      ib += y;
    }
  }
  if (lane == 31) {
    wsum[warp] = ia;
    wsum[33 + warp] = ib;
  }
  __syncthreads();
  if (warp == 0) {
    const int wa = lane < NW ? wsum[lane] : 0, wb = lane < NW ? wsum[33 + lane] : 0;
    int ja = wa, jb = wb;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, ja, o), y = __shfl_up_sync(0xffffffffu, jb, o);
      if (lane >= o) {
        ja += x;
        jb += y;
      }
    }
    if (lane < NW) {
      wsum[lane] = ja - wa;
      wsum[33 + lane] = jb - wb;
    }
    if (lane == 31) {
      wsum[32] = ja;
      wsum[65] = jb;
    }
  }
  __syncthreads();
  *ea = wsum[warp] + ia - a;
  *eb = wsum[33 + warp] + ib - b;
  *ta = wsum[32];
  *tb = wsum[65];
  __syncthreads();
}

// 16-byte asynchronous copy global -> shared (L2 only), commit and wait of the issuing thread's groups
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint2 ldg_stream_u2(const void* p) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(r.x), "=r"(r.y)
               : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}


// ---- warp-level tensor-core tile: D(16x8, fp32) += A(16x16, row) * B(16x8, col), 16-bit inputs ----
// Lane l = 4*g + t holds A rows g and g+8 (a0/a2: row g, k-slots {2t,2t+1} / {2t+8,2t+9}; a1/a3 the
// same slots of row g+8), B column g (b0: k-slots {2t,2t+1}, b1: {2t+8,2t+9}) and D elements
// (g, 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1).  Which channel sits in which k-slot is free as long
// as A and B agree, which is what lets both operands be taken from memory in 16-byte pieces.
template <typename T>
struct MmaTile;
template <>
struct MmaTile<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <>
struct MmaTile<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// twl_sparse_decode_attn for a caller that knows an upper bound of the sequences' page counts
// (attend.cu; the group kernel sizes its shared-memory tables by it).
int sparse_decode_attn_bounded(const void* q, int dtype, const void* k_pages, const void* v_pages,
                               const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* indices,
                               int32_t index_stride, const int32_t* budget, const float* weights, int32_t batch,
                               int32_t num_q_heads, int32_t num_kv_heads, int32_t num_pages_total, float sm_scale,
                               void* out, void* workspace, size_t workspace_bytes, int32_t chunk, int32_t* status,
                               void* stream, int32_t max_seq_pages);

}  // namespace twl
