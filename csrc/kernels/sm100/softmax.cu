// Softmax over the last axis, forward and backward, for sm_100a (bf16 or fp32 io, fp32 arithmetic).
//
// The reference composes softmax on CUDA from eight launches (max_keepdim, broadcast, sub, exp, sum_keepdim, broadcast,
// log, sub, then exp: crates/incin-backends/src/cuda/backend.rs:948-964) and its WGSL shader does one workgroup per row
// with a tree reduction (wgpu/shaders/softmax.wgsl:13-92).  Here one launch does a row per warp when the row fits a
// warp's registers (C <= 2048: every element is read from global memory exactly once) and a row per block otherwise
// (three passes over a row that stays in L2).  The backward is dx = y * (dy - sum(dy * y)) with the same two shapes.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "incin_b200.h"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int WARP_ROW_MAX = 2048;        // elements of a row one warp keeps in registers (64 per lane)
constexpr int PER_LANE = WARP_ROW_MAX / 32;

// one row per warp; BWD: a = dy, b = y
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                           long long rows, int C) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* pa = a + row * C;
  float v[PER_LANE];
  if (!BWD) {
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int c = lane + i * 32;
      v[i] = c < C ? ldf(pa, c) : -CUDART_INF_F;
      m = fmaxf(m, v[i]);
    }
    m = warp_max(m);
    if (m == -CUDART_INF_F) m = 0.0f;     // a row of -inf: every exponent is 0, the result is NaN as in the composed form
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      v[i] = __expf(v[i] - m);
      s += v[i];
    }
    s = warp_sum(s);
    const float inv = 1.0f / s;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int c = lane + i * 32;
      if (c < C) stf(out + row * C, c, v[i] * inv);
    }
  } else {
    const T* pb = b + row * C;
    float w[PER_LANE];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int c = lane + i * 32;
      v[i] = c < C ? ldf(pa, c) : 0.0f;
      w[i] = c < C ? ldf(pb, c) : 0.0f;
      s += v[i] * w[i];
    }
    s = warp_sum(s);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int c = lane + i * 32;
      if (c < C) stf(out + row * C, c, w[i] * (v[i] - s));
    }
  }
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = l < nw ? sh[l] : (is_max ? -CUDART_INF_F : 0.0f);
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

// one row per block (any C)
template <typename T, bool BWD>
__global__ void __launch_bounds__(512) softmax_block_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                            long long rows, int C) {
  __shared__ float sh[32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* pa = a + row * C;
    if (!BWD) {
      float m = -CUDART_INF_F;
      for (int c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, ldf(pa, c));
      m = block_reduce(m, true, sh);
      if (m == -CUDART_INF_F) m = 0.0f;
      float s = 0.0f;
      for (int c = threadIdx.x; c < C; c += blockDim.x) s += __expf(ldf(pa, c) - m);
      s = block_reduce(s, false, sh);
      const float inv = 1.0f / s;
      for (int c = threadIdx.x; c < C; c += blockDim.x) stf(out + row * C, c, __expf(ldf(pa, c) - m) * inv);
    } else {
      const T* pb = b + row * C;
      float s = 0.0f;
      for (int c = threadIdx.x; c < C; c += blockDim.x) s += ldf(pa, c) * ldf(pb, c);
      s = block_reduce(s, false, sh);
      for (int c = threadIdx.x; c < C; c += blockDim.x) stf(out + row * C, c, ldf(pb, c) * (ldf(pa, c) - s));
    }
  }
}

template <typename T, bool BWD>
int launch(const void* a, const void* b, void* out, long long rows, int C, cudaStream_t s) {
  if (C <= WARP_ROW_MAX) {
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    softmax_warp_kernel<T, BWD><<<blocks, 256, 0, s>>>((const T*)a, (const T*)b, (T*)out, rows, C);
  } else {
    const unsigned blocks = (unsigned)(rows < 148LL * 8 ? rows : 148LL * 8);
    softmax_block_kernel<T, BWD><<<blocks, 512, 0, s>>>((const T*)a, (const T*)b, (T*)out, rows, C);
  }
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace

extern "C" int incin_softmax_lastdim_fwd(const void* x, void* y, long long rows, int C, int is_bf16, void* stream) {
  if (!x || !y || rows <= 0 || C <= 0) return INCIN_ERR_ARGUMENT;
  return is_bf16 ? launch<__nv_bfloat16, false>(x, nullptr, y, rows, C, (cudaStream_t)stream)
                 : launch<float, false>(x, nullptr, y, rows, C, (cudaStream_t)stream);
}

extern "C" int incin_softmax_lastdim_bwd(const void* dy, const void* y, void* dx, long long rows, int C, int is_bf16, void* stream) {
  if (!dy || !y || !dx || rows <= 0 || C <= 0) return INCIN_ERR_ARGUMENT;
  return is_bf16 ? launch<__nv_bfloat16, true>(dy, y, dx, rows, C, (cudaStream_t)stream)
                 : launch<float, true>(dy, y, dx, rows, C, (cudaStream_t)stream);
}
