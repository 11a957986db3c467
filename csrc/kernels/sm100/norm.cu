// LayerNorm / RMSNorm forward and backward, bf16 in/out with fp32 statistics.
//
// One warp owns one row and walks it with 16-byte loads, so a [8192, 768]
// activation is one pass over HBM (the re-reads of a 1.5 KB row hit L1).  The
// backward pass writes dx (optionally fused with the residual-stream gradient)
// row-wise, and reduces dgamma/dbeta column-wise through a small fp32 scratch
// buffer in a fixed order, so the parameter gradients are deterministic.
//
// The reference has a forward-only CUDA layer_norm with no tape entry
// (crates/incin-backends/src/kernel.rs:1233-1336) and composes RMSNorm from
// six elementwise launches (crates/incin-core/src/nn/rms_norm.rs:88-126).
#include "ptx.cuh"
#include "launch.cuh"
#include "../../include/incin_b200.h"

namespace incin {

constexpr int NORM_WARPS = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ----------------------------------------------------------------------------- forward
template <bool RMS>
__global__ void __launch_bounds__(NORM_WARPS * 32)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, long long rows, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * C;
  __nv_bfloat16* yr = y + row * C;
  const bool vec = (C % 8) == 0;
  float s = 0.f;
  if (!RMS) {
    if (vec) {
      for (int c = lane * 8; c < C; c += 256) {
        float f[8];
        load8(xr + c, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += f[i];
      }
    } else {
      for (int c = lane; c < C; c += 32) s += __bfloat162float(xr[c]);
    }
    s = warp_sum(s);
  }
  const float mean = RMS ? 0.f : s / C;
  float q = 0.f;
  if (vec) {
    for (int c = lane * 8; c < C; c += 256) {
      float f[8];
      load8(xr + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = f[i] - mean;
        q += d * d;
      }
    }
  } else {
    for (int c = lane; c < C; c += 32) {
      const float d = __bfloat162float(xr[c]) - mean;
      q += d * d;
    }
  }
  q = warp_sum(q);
  const float rstd = rsqrtf(q / C + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  if (vec) {
    for (int c = lane * 8; c < C; c += 256) {
      float f[8], g[8], o[8];
      load8(xr + c, f);
      load8(gamma + c, g);
      if (beta) {
        float b[8];
        load8(beta + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (f[i] - mean) * rstd * g[i] + b[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (f[i] - mean) * rstd * g[i];
      }
      store8(yr + c, o);
    }
  } else {
    for (int c = lane; c < C; c += 32) {
      float o = (__bfloat162float(xr[c]) - mean) * rstd * __bfloat162float(gamma[c]);
      if (beta) o += __bfloat162float(beta[c]);
      yr[c] = __float2bfloat16(o);
    }
  }
}

// ----------------------------------------------------------------------------- backward: dx
// LayerNorm: dx = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat))
// RMSNorm  : dx = rstd * (g*dy - xhat * mean(g*dy*xhat)),  xhat = x * rstd
template <bool RMS>
__global__ void __launch_bounds__(NORM_WARPS * 32)
norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                   const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                   __nv_bfloat16* __restrict__ dx, long long rows, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * C;
  const __nv_bfloat16* dyr = dy + row * C;
  const float mean = RMS ? 0.f : mean_in[row];
  const float rstd = rstd_in[row];
  const bool vec = (C % 8) == 0;
  float s1 = 0.f, s2 = 0.f;
  if (vec) {
    for (int c = lane * 8; c < C; c += 256) {
      float f[8], d[8], g[8];
      load8(xr + c, f);
      load8(dyr + c, d);
      load8(gamma + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float gd = g[i] * d[i];
        s1 += gd;
        s2 += gd * (f[i] - mean) * rstd;
      }
    }
  } else {
    for (int c = lane; c < C; c += 32) {
      const float gd = __bfloat162float(gamma[c]) * __bfloat162float(dyr[c]);
      s1 += gd;
      s2 += gd * (__bfloat162float(xr[c]) - mean) * rstd;
    }
  }
  s1 = RMS ? 0.f : warp_sum(s1) / C;
  s2 = warp_sum(s2) / C;
  __nv_bfloat16* dxr = dx + row * C;
  const __nv_bfloat16* addr = dx_add ? dx_add + row * C : nullptr;
  if (vec) {
    for (int c = lane * 8; c < C; c += 256) {
      float f[8], d[8], g[8], o[8];
      load8(xr + c, f);
      load8(dyr + c, d);
      load8(gamma + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rstd * (g[i] * d[i] - s1 - (f[i] - mean) * rstd * s2);
      if (addr) {
        float a[8];
        load8(addr + c, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += a[i];
      }
      store8(dxr + c, o);
    }
  } else {
    for (int c = lane; c < C; c += 32) {
      const float xh = (__bfloat162float(xr[c]) - mean) * rstd;
      float o = rstd * (__bfloat162float(gamma[c]) * __bfloat162float(dyr[c]) - s1 - xh * s2);
      if (addr) o += __bfloat162float(addr[c]);
      dxr[c] = __float2bfloat16(o);
    }
  }
}

// ----------------------------------------------------------------------------- backward: dgamma / dbeta
// Stage 1: block (bx, by) reduces rows [by*rows_per, ...) of 64 columns into scratch[by][{g,b}][C].
// Stage 2: one thread per column sums the `chunks` partials in order and adds into the gradient.
constexpr int PG_COLS = 64;
constexpr int PG_TY = 8;

template <bool RMS>
__global__ void __launch_bounds__(32 * PG_TY)
norm_bwd_param_partial(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                       float* __restrict__ scratch, long long rows, int C, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sg[PG_TY][PG_COLS];
  __shared__ float sb[PG_TY][PG_COLS];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = blockIdx.x * PG_COLS + tx * 2;
  const long long rows_per = (rows + chunks - 1) / chunks;
  const long long r0 = (long long)blockIdx.y * rows_per;
  const long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  float g0 = 0.f, g1 = 0.f, b0 = 0.f, b1 = 0.f;
  if (c0 < C) {
    const bool pair = (c0 + 1 < C) && ((C & 1) == 0);
    for (long long r = r0 + ty; r < r1; r += PG_TY) {
      const float mean = RMS ? 0.f : mean_in[r];
      const float rstd = rstd_in[r];
      float d0, d1 = 0.f, x0, x1 = 0.f;
      if (pair) {
        const float2 dd = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + r * C + c0));
        const float2 xx = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + r * C + c0));
        d0 = dd.x; d1 = dd.y; x0 = xx.x; x1 = xx.y;
      } else {
        d0 = __bfloat162float(dy[r * C + c0]);
        x0 = __bfloat162float(x[r * C + c0]);
        if (c0 + 1 < C) {
          d1 = __bfloat162float(dy[r * C + c0 + 1]);
          x1 = __bfloat162float(x[r * C + c0 + 1]);
        }
      }
      g0 += d0 * (x0 - mean) * rstd;
      g1 += d1 * (x1 - mean) * rstd;
      b0 += d0;
      b1 += d1;
    }
  }
  sg[ty][tx * 2] = g0;
  sg[ty][tx * 2 + 1] = g1;
  sb[ty][tx * 2] = b0;
  sb[ty][tx * 2 + 1] = b1;
  __syncthreads();
  if (ty == 0) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int c = c0 + e;
      if (c < C) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int t = 0; t < PG_TY; ++t) {
          a += sg[t][tx * 2 + e];
          b += sb[t][tx * 2 + e];
        }
        scratch[((long long)blockIdx.y * 2 + 0) * C + c] = a;
        scratch[((long long)blockIdx.y * 2 + 1) * C + c] = b;
      }
    }
  }
}

// 16-byte variant of stage 1: 256 columns per block (32 lanes x 8 columns), 8 row lanes; C % 8 == 0
template <bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_param_partial_vec(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                           float* __restrict__ scratch, long long rows, int C, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sg[8][256];
  __shared__ float sb[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + tx * 8;
  const long long rows_per = (rows + chunks - 1) / chunks;
  const long long r0 = (long long)blockIdx.y * rows_per;
  const long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  float g[8] = {0, 0, 0, 0, 0, 0, 0, 0}, b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < C) {
    for (long long r = r0 + ty; r < r1; r += 8) {
      const float mean = RMS ? 0.f : mean_in[r];
      const float rstd = rstd_in[r];
      float d[8], xv[8];
      load8(dy + r * C + c0, d);
      load8(x + r * C + c0, xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        g[i] += d[i] * (xv[i] - mean) * rstd;
        b[i] += d[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sg[ty][tx * 8 + i] = g[i];
    sb[ty][tx * 8 + i] = b[i];
  }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < C) {
    float a = 0.f, bb = 0.f;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      a += sg[t][threadIdx.x];
      bb += sb[t][threadIdx.x];
    }
    scratch[((long long)blockIdx.y * 2 + 0) * C + c] = a;
    scratch[((long long)blockIdx.y * 2 + 1) * C + c] = bb;
  }
}

// Stage 2: 32 columns x 8 chunk lanes per block.  Each thread adds every 8th partial (independent, coalesced loads),
// then the 8 lanes of a column are combined in a fixed order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256)
norm_bwd_param_final(const float* __restrict__ scratch, float* __restrict__ dgamma, float* __restrict__ dbeta, int C,
                     int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sa[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f;
  if (c < C) {
    for (int k = ty; k < chunks; k += 8) {
      a += scratch[((long long)k * 2 + 0) * C + c];
      b += scratch[((long long)k * 2 + 1) * C + c];
    }
  }
  sa[ty][tx] = a;
  sb[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && c < C) {
#pragma unroll
    for (int t = 1; t < 8; ++t) {
      a += sa[t][tx];
      b += sb[t][tx];
    }
    dgamma[c] += a;
    if (dbeta) dbeta[c] += b;
  }
}

static int param_chunks(long long rows) {
  long long c = (rows + 127) / 128;
  if (c > 64) c = 64;
  if (c < 1) c = 1;
  return (int)c;
}

template <bool RMS>
static int norm_bwd_launch(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                           const void* dx_add, void* dx, float* dgamma, float* dbeta, float* scratch, long long rows,
                           int C, cudaStream_t s) {
  if (rows <= 0 || C <= 0) return INCIN_ERR_ARGUMENT;
  const unsigned blocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
  launch_pdl(norm_bwd_dx_kernel<RMS>, dim3(blocks), dim3(NORM_WARPS * 32), 0, s, 
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd,
      (const __nv_bfloat16*)dx_add, (__nv_bfloat16*)dx, rows, C);
  if (dgamma) {
    if (!scratch) return INCIN_ERR_ARGUMENT;
    const int chunks = param_chunks(rows);
    if ((C % 8) == 0) {
      dim3 grid((C + 255) / 256, chunks);
      launch_pdl(norm_bwd_param_partial_vec<RMS>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean,
                                                           rstd, scratch, rows, C, chunks);
    } else {
      dim3 grid((C + PG_COLS - 1) / PG_COLS, chunks);
      launch_pdl(norm_bwd_param_partial<RMS>, dim3(grid), dim3(32 * PG_TY), 0, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                               mean, rstd, scratch, rows, C, chunks);
    }
    launch_pdl(norm_bwd_param_final, dim3((C + 31) / 32), dim3(256), 0, s, scratch, dgamma, dbeta, C, chunks);
  }
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace incin

using namespace incin;

extern "C" int incin_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                                   float* rstd, long long rows, int C, float eps, void* stream) {
  if (rows <= 0 || C <= 0 || !x || !gamma || !y || !rstd) return INCIN_ERR_ARGUMENT;
  const unsigned blocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
  launch_pdl(norm_fwd_kernel<false>, dim3(blocks), dim3(NORM_WARPS * 32), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, mean, rstd,
      rows, C, eps);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, long long rows, int C,
                                 float eps, void* stream) {
  if (rows <= 0 || C <= 0 || !x || !gamma || !y || !rstd) return INCIN_ERR_ARGUMENT;
  const unsigned blocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
  launch_pdl(norm_fwd_kernel<true>, dim3(blocks), dim3(NORM_WARPS * 32), 0, (cudaStream_t)stream, 
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, nullptr, (__nv_bfloat16*)y, nullptr, rstd, rows, C, eps);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" long long incin_layernorm_bwd_scratch_floats(long long rows, int C) {
  return (long long)param_chunks(rows) * 2 * C;
}

extern "C" int incin_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                                   const float* rstd, const void* dx_add, void* dx, float* dgamma, float* dbeta,
                                   float* scratch, long long rows, int C, void* stream) {
  return norm_bwd_launch<false>(dy, x, gamma, mean, rstd, dx_add, dx, dgamma, dbeta, scratch, rows, C,
                                (cudaStream_t)stream);
}

extern "C" int incin_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd,
                                 const void* dx_add, void* dx, float* dgamma, float* scratch, long long rows, int C,
                                 void* stream) {
  return norm_bwd_launch<true>(dy, x, gamma, nullptr, rstd, dx_add, dx, dgamma, nullptr, scratch, rows, C,
                               (cudaStream_t)stream);
}
