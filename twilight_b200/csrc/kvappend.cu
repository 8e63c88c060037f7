// Cache-append side: INT4 K quantiser, page (min,max) metadata, one-token append, and the
// index-list -> dense-mask scatter used by the mask-returning compatibility interface.
//
// The quantiser follows min_max_per_token_quant_kv (twilight/pyimpl/quantize.py:4-13) applied
// to groups of 32 channels, with every intermediate rounded to the cache dtype exactly where
// torch rounds it in the reference (range, scale, x+zero, quotient), so the 4-bit codes are
// the reference's codes.  One deviation: for an fp16 group whose values are all equal the
// reference divides 0 by a scale that its clamp(min=1e-9) rounds to 0 and produces NaN; here
// such a group gets code 0 and scale 0, i.e. it dequantises to its (single) value.
#include "common.cuh"

namespace twl {

template <typename T>
__device__ __forceinline__ float rnd(float x) {
  return Elem<T>::to_f(Elem<T>::from_f(x));
}

// Quantises 32 values (already exact values of type T held as float).  Returns 16 code bytes
// (byte j = channel 2j low nibble, 2j+1 high nibble) and {scale, min} as fp16.
template <typename T>
__device__ __forceinline__ void quantize_group(const float* x, uint32_t* packed /*4 words*/,
                                               __half2* sz) {
  float mx = x[0], mn = x[0];
#pragma unroll
  for (int i = 1; i < 32; ++i) {
    mx = fmaxf(mx, x[i]);
    mn = fminf(mn, x[i]);
  }
  float range = rnd<T>(mx - mn);
  range = fmaxf(range, rnd<T>(1e-9f));
  const float scale = rnd<T>(__fdiv_rn(range, 15.f));
  const float zero = -mn;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t word = 0;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float t = rnd<T>(x[8 * w + n] + zero);
      float u = (scale > 0.f) ? rnd<T>(__fdiv_rn(t, scale)) : 0.f;
      u = fminf(fmaxf(rintf(u), 0.f), 15.f);
      word |= ((uint32_t)(int)u) << (4 * n);
    }
    packed[w] = word;
  }
  *sz = __halves2half2(__float2half_rn(scale), __float2half_rn(mn));
}

// one thread per (token, group) of a slab; 64 threads per slab
template <typename T>
__global__ void __launch_bounds__(256)
quantize_k_pages_kernel(const T* __restrict__ k_pages, uint8_t* __restrict__ k4, int64_t n_slabs) {
  const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t slab = item >> 6;
  if (slab >= n_slabs) return;
  const int tg = (int)(item & 63);  // token*4 + group
  const T* src = k_pages + slab * (kPage * kD) + tg * kGroup;
  float x[32];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + i);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = Elem<T>::to_f2(u[k]);
      x[8 * i + 2 * k] = f.x;
      x[8 * i + 2 * k + 1] = f.y;
    }
  }
  uint32_t packed[4];
  __half2 sz;
  quantize_group<T>(x, packed, &sz);
  uint8_t* dst = k4 + slab * kSlab;
  *reinterpret_cast<uint4*>(dst + tg * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  *reinterpret_cast<__half2*>(dst + kSlabCodes + tg * 4) = sz;
}

// one warp per (sequence page, kv head); lane owns 4 channels
template <typename T>
__global__ void __launch_bounds__(256)
build_page_meta_kernel(const T* __restrict__ k_pages, T* __restrict__ kmeta,
                       const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                       const int32_t* __restrict__ last_len, int Hkv, int num_pages_total) {
  const int row = blockIdx.y;  // (b, kv head)
  const int b = row / Hkv, kvh = row % Hkv;
  const int page_base = indptr[b];
  const int n_pages = indptr[b + 1] - page_base;
  const int lane = threadIdx.x & 31;
  const int lp = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (lp >= n_pages) return;
  const int phys = indices[page_base + lp];
  if (phys < 0 || phys >= num_pages_total) return;
  const int n_tok = (lp == n_pages - 1) ? last_len[b] : kPage;
  const T* src = k_pages + ((size_t)phys * Hkv + kvh) * (kPage * kD);
  float mn[4] = {INFINITY, INFINITY, INFINITY, INFINITY};
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  for (int t = 0; t < n_tok; ++t) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(src + t * kD) + lane);
    const float2 a = Elem<T>::to_f2(v.x), c = Elem<T>::to_f2(v.y);
    const float e[4] = {a.x, a.y, c.x, c.y};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mn[k] = fminf(mn[k], e[k]);
      mx[k] = fmaxf(mx[k], e[k]);
    }
  }
  T* dst = kmeta + ((size_t)phys * Hkv + kvh) * 2 * kD;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    dst[lane * 4 + k] = Elem<T>::from_f(mn[k]);
    dst[kD + lane * 4 + k] = Elem<T>::from_f(mx[k]);
  }
}

// one block of 128 threads per (sequence, kv head): thread = channel, warp = quantisation group
template <typename T>
__global__ void __launch_bounds__(128)
append_kv_kernel(const T* __restrict__ new_k, const T* __restrict__ new_v, T* __restrict__ k_pages,
                 T* __restrict__ v_pages, uint8_t* __restrict__ k4, T* __restrict__ kmeta,
                 const int32_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                 const int32_t* __restrict__ last_len, int Hkv, int num_pages_total,
                 int32_t* status) {
  const int row = blockIdx.x;
  const int b = row / Hkv, kvh = row % Hkv;
  const int n_pages = indptr[b + 1] - indptr[b];
  const int ll = last_len[b];
  if (n_pages <= 0 || ll < 1 || ll > kPage) {
    if (threadIdx.x == 0) raise_flag(status, TWL_FLAG_BAD_INDEX);
    return;
  }
  const int phys = indices[indptr[b] + n_pages - 1];
  if (phys < 0 || phys >= num_pages_total) {
    if (threadIdx.x == 0) raise_flag(status, TWL_FLAG_BAD_INDEX);
    return;
  }
  const int slot = ll - 1;
  const int d = threadIdx.x, lane = d & 31, grp = d >> 5;
  const size_t slab = (size_t)phys * Hkv + kvh;
  const T kx = new_k[(size_t)row * kD + d];
  k_pages[slab * (kPage * kD) + slot * kD + d] = kx;
  v_pages[slab * (kPage * kD) + slot * kD + d] = new_v[(size_t)row * kD + d];
  const float x = Elem<T>::to_f(kx);
  // page metadata: first token of a page starts it, later ones fold in
  if (kmeta != nullptr) {
    T* meta = kmeta + slab * 2 * kD;
    if (slot == 0) {
      meta[d] = kx;
      meta[kD + d] = kx;
    } else {
      meta[d] = Elem<T>::from_f(fminf(Elem<T>::to_f(meta[d]), x));
      meta[kD + d] = Elem<T>::from_f(fmaxf(Elem<T>::to_f(meta[kD + d]), x));
    }
  }
  if (k4 != nullptr) {
    const float mx = warp_max(x), mn = warp_min(x);
    float range = rnd<T>(mx - mn);
    range = fmaxf(range, rnd<T>(1e-9f));
    const float scale = rnd<T>(__fdiv_rn(range, 15.f));
    const float t = rnd<T>(x - mn);
    float u = (scale > 0.f) ? rnd<T>(__fdiv_rn(t, scale)) : 0.f;
    u = fminf(fmaxf(rintf(u), 0.f), 15.f);
    const uint32_t code = (uint32_t)(int)u;
    const uint32_t hi = __shfl_down_sync(0xffffffffu, code, 1);
    uint8_t* dst = k4 + slab * kSlab;
    if ((lane & 1) == 0) dst[slot * 64 + grp * 16 + (lane >> 1)] = (uint8_t)(code | (hi << 4));
    if (lane == 0)
      *reinterpret_cast<__half2*>(dst + kSlabCodes + slot * 16 + grp * 4) =
          __halves2half2(__float2half_rn(scale), __float2half_rn(mn));
  }
}

__global__ void indices_to_mask_kernel(const int32_t* __restrict__ indices, int index_stride,
                                       const int32_t* __restrict__ budget, uint8_t* __restrict__ mask,
                                       int d) {
  const int row = blockIdx.y;
  const int n = min(budget[row], index_stride);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int tok = indices[(size_t)row * index_stride + i];
  if (tok >= 0 && tok < d) mask[(size_t)row * d + tok] = 1;
}

}  // namespace twl

extern "C" int twl_quantize_k_pages(const void* k_pages, int dtype, uint8_t* k4_pages,
                                    int64_t n_slabs, void* stream) {
  using namespace twl;
  if (!k_pages || !k4_pages || n_slabs <= 0) return TWL_ERR_BAD_ARG;
  if (!aligned(k_pages, 16) || !aligned(k4_pages, 16)) return TWL_ERR_MISALIGNED;
  const int64_t items = n_slabs * 64;
  const int64_t blocks = (items + 255) / 256;
  if (blocks > 0x7fffffffLL) return TWL_ERR_TOO_LARGE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) {
    quantize_k_pages_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __half*>(k_pages), k4_pages, n_slabs);
  } else if (dtype == TWL_BF16) {
    quantize_k_pages_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(k_pages), k4_pages, n_slabs);
  } else {
    return TWL_ERR_UNSUPPORTED;
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

extern "C" int twl_build_page_meta(const void* k_pages, int dtype, void* kmeta,
                                   const int32_t* kv_indptr, const int32_t* kv_indices,
                                   const int32_t* kv_last_page_len, int32_t batch,
                                   int32_t num_kv_heads, int32_t num_pages_total,
                                   int32_t max_pages, void* stream) {
  using namespace twl;
  if (!k_pages || !kmeta || !kv_indptr || !kv_indices || !kv_last_page_len) return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_kv_heads <= 0 || num_pages_total <= 0 || max_pages <= 0)
    return TWL_ERR_BAD_ARG;
  if (!aligned(k_pages, 16) || !aligned(kmeta, 16)) return TWL_ERR_MISALIGNED;
  if ((int64_t)batch * num_kv_heads > 65535) return TWL_ERR_TOO_LARGE;
  dim3 grid((max_pages + 7) / 8, batch * num_kv_heads);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == TWL_F16) {
    build_page_meta_kernel<__half><<<grid, 256, 0, st>>>(
        static_cast<const __half*>(k_pages), static_cast<__half*>(kmeta), kv_indptr, kv_indices,
        kv_last_page_len, num_kv_heads, num_pages_total);
  } else if (dtype == TWL_BF16) {
    build_page_meta_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(kmeta), kv_indptr,
        kv_indices, kv_last_page_len, num_kv_heads, num_pages_total);
  } else {
    return TWL_ERR_UNSUPPORTED;
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

extern "C" int twl_append_kv(const void* new_k, const void* new_v, int dtype, void* k_pages,
                             void* v_pages, uint8_t* k4_pages, void* kmeta,
                             const int32_t* kv_indptr, const int32_t* kv_indices,
                             const int32_t* kv_last_page_len, int32_t batch, int32_t num_kv_heads,
                             int32_t num_pages_total, int32_t* status, void* stream) {
  using namespace twl;
  if (!new_k || !new_v || !k_pages || !v_pages || !kv_indptr || !kv_indices || !kv_last_page_len)
    return TWL_ERR_BAD_ARG;
  if (batch <= 0 || num_kv_heads <= 0 || num_pages_total <= 0) return TWL_ERR_BAD_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned rows = (unsigned)batch * num_kv_heads;
  if (dtype == TWL_F16) {
    append_kv_kernel<__half><<<rows, 128, 0, st>>>(
        static_cast<const __half*>(new_k), static_cast<const __half*>(new_v),
        static_cast<__half*>(k_pages), static_cast<__half*>(v_pages), k4_pages,
        static_cast<__half*>(kmeta), kv_indptr, kv_indices, kv_last_page_len, num_kv_heads,
        num_pages_total, status);
  } else if (dtype == TWL_BF16) {
    append_kv_kernel<__nv_bfloat16><<<rows, 128, 0, st>>>(
        static_cast<const __nv_bfloat16*>(new_k), static_cast<const __nv_bfloat16*>(new_v),
        static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages), k4_pages,
        static_cast<__nv_bfloat16*>(kmeta), kv_indptr, kv_indices, kv_last_page_len, num_kv_heads,
        num_pages_total, status);
  } else {
    return TWL_ERR_UNSUPPORTED;
  }
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}

extern "C" int twl_indices_to_mask(const int32_t* indices, int32_t index_stride,
                                   const int32_t* budget, int32_t rows, uint8_t* mask, int32_t d,
                                   void* stream) {
  using namespace twl;
  if (!indices || !budget || !mask || rows <= 0 || index_stride <= 0 || d <= 0)
    return TWL_ERR_BAD_ARG;
  if (rows > 65535) return TWL_ERR_TOO_LARGE;
  dim3 grid((index_stride + 255) / 256, rows);
  indices_to_mask_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      indices, index_stride, budget, mask, d);
  TWL_CHECK_LAUNCH();
  return TWL_OK;
}
