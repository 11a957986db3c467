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

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
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

// Forward for C <= 1024 (C % 8 == 0): the row is read once with all its 16-byte loads in flight and stays packed in
// registers for the mean, the centred variance and the output.
template <bool RMS, int ITER>
__global__ void __launch_bounds__(NORM_WARPS * 32)
norm_fwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                    const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                    float* __restrict__ rstd_out, long long rows, int C, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  uint4 raw[ITER];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = it * 256 + lane * 8;
    raw[it] = c < C ? *reinterpret_cast<const uint4*>(x + row * C + c) : make_uint4(0, 0, 0, 0);
  }
  const float inv_c = 1.f / C;
  float mean = 0.f;
  if (!RMS) {
    float s = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      float f[8];
      unpack8(raw[it], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += f[i];
    }
    mean = warp_sum(s) * inv_c;
  }
  float q = 0.f;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    if (it * 256 + lane * 8 < C) {
      float f[8];
      unpack8(raw[it], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = f[i] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) * inv_c + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int c = it * 256 + lane * 8;
    if (c < C) {
      float f[8], g[8], o[8];
      unpack8(raw[it], f);
      load8(gamma + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (f[i] - mean) * rstd * g[i];
      if (beta) {
        float b[8];
        load8(beta + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += b[i];
      }
      store8(y + row * C + c, o);
    }
  }
}

template <bool RMS>
static void norm_fwd_launch(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                            long long rows, int C, float eps, cudaStream_t s) {
  const unsigned blocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
  auto go = [&](auto kern) {
    launch_pdl(kern, dim3(blocks), dim3(NORM_WARPS * 32), 0, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma,
               (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, mean, rstd, rows, C, eps);
  };
  if ((C % 8) == 0 && C <= 1024) {
    const int iters = (C + 255) / 256;
    if (iters == 1) go(norm_fwd_reg_kernel<RMS, 1>);
    else if (iters == 2) go(norm_fwd_reg_kernel<RMS, 2>);
    else if (iters == 3) go(norm_fwd_reg_kernel<RMS, 3>);
    else go(norm_fwd_reg_kernel<RMS, 4>);
  } else {
    go(norm_fwd_kernel<RMS>);
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

// Stage 2: 32 columns x 32 chunk lanes per block.  Each thread adds every 32nd partial (independent, coalesced loads,
// four in flight), then the 32 lanes of a column are combined in a fixed order, so the result does not depend on
// scheduling.
constexpr int PF_LANES = 32;
__global__ void __launch_bounds__(32 * PF_LANES)
norm_bwd_param_final(const float* __restrict__ scratch, float* __restrict__ dgamma, float* __restrict__ dbeta, int C,
                     int chunks, int na, float* __restrict__ dxsum) {
  // scratch[chunk][na][C]: na = 2 partial sums per column (dgamma, dbeta), or 3 with the column sums of dx behind them
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sa[PF_LANES][33], sb[PF_LANES][33], sc[PF_LANES][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f, d = 0.f;
  if (c < C) {
    int k = ty;
    for (; k + 3 * PF_LANES < chunks; k += 4 * PF_LANES) {
      float va[4], vb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        va[u] = scratch[((long long)(k + u * PF_LANES) * na + 0) * C + c];
        vb[u] = scratch[((long long)(k + u * PF_LANES) * na + 1) * C + c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a += va[u];
        b += vb[u];
      }
      if (dxsum) {
#pragma unroll
        for (int u = 0; u < 4; ++u) d += scratch[((long long)(k + u * PF_LANES) * na + 2) * C + c];
      }
    }
    for (; k < chunks; k += PF_LANES) {
      a += scratch[((long long)k * na + 0) * C + c];
      b += scratch[((long long)k * na + 1) * C + c];
      if (dxsum) d += scratch[((long long)k * na + 2) * C + c];
    }
  }
  sa[ty][tx] = a;
  sb[ty][tx] = b;
  sc[ty][tx] = d;
  __syncthreads();
  if (ty == 0 && c < C) {
#pragma unroll
    for (int t = 1; t < PF_LANES; ++t) {
      a += sa[t][tx];
      b += sb[t][tx];
      d += sc[t][tx];
    }
    dgamma[c] += a;
    if (dbeta) dbeta[c] += b;
    if (dxsum) dxsum[c] += d;
  }
}

// ----------------------------------------------------------------------------- backward: dx and stage 1 in one pass
// For C <= 1024 (C % 8 == 0) a warp keeps its whole row of x and dy in registers, so dx and the per-column partial
// sums of dgamma / dbeta come out of ONE read of x and dy: block b owns rows [b * rows_per, ...), its 8 warps take every
// 8th row and add d * xhat and d into per-lane column accumulators, which are then combined in warp order (fixed, so
// the result does not depend on scheduling) and written to scratch[b][{g,b}][C] for norm_bwd_param_final.
// The row is held as the raw 16-byte loads (bf16) and unpacked where it is used; the per-column accumulators of each
// warp live in shared memory (element (it, i, lane) at it*256 + i*32 + lane: a warp touches 32 different banks), which
// keeps the kernel under 85 registers so that three blocks (24 warps) per SM have loads in flight.
template <bool RMS, int ITER>
__global__ void __launch_bounds__(NORM_WARPS * 32, 3)
norm_bwd_fused_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                      const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ scratch, long long rows, int C,
                      long long rows_per) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float acc_smem[];                     // [NORM_WARPS][2][ITER * 256]
  constexpr int W = ITER * 256;
  constexpr int NA = 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* gacc = acc_smem + (warp * NA + 0) * W;
  float* bacc = acc_smem + (warp * NA + 1) * W;
#pragma unroll
  for (int j = lane; j < W; j += 32) {
    gacc[j] = 0.f;
    bacc[j] = 0.f;
  }
  __syncwarp();
  const long long r0 = (long long)blockIdx.x * rows_per;
  const long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  const float inv_c = 1.f / C;
  for (long long r = r0 + warp; r < r1; r += NORM_WARPS) {
    const float mean = RMS ? 0.f : mean_in[r];
    const float rstd = rstd_in[r];
    uint4 xraw[ITER], draw[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = it * 256 + lane * 8;
      const bool in = c < C;
      xraw[it] = in ? *reinterpret_cast<const uint4*>(x + r * C + c) : make_uint4(0, 0, 0, 0);
      draw[it] = in ? *reinterpret_cast<const uint4*>(dy + r * C + c) : make_uint4(0, 0, 0, 0);   // d = 0 past C
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = it * 256 + lane * 8;
      float f[8], d[8], g[8];
      unpack8(xraw[it], f);
      unpack8(draw[it], d);
      if (c < C) {
        load8(gamma + c, g);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (f[i] - mean) * rstd;
        const float gd = g[i] * d[i];
        s1 += gd;
        s2 += gd * xh;
        gacc[it * 256 + i * 32 + lane] += d[i] * xh;
        bacc[it * 256 + i * 32 + lane] += d[i];
      }
    }
    s1 = RMS ? 0.f : warp_sum(s1) * inv_c;
    s2 = warp_sum(s2) * inv_c;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = it * 256 + lane * 8;
      if (c < C) {
        float f[8], d[8], g[8], o[8];
        unpack8(xraw[it], f);
        unpack8(draw[it], d);
        load8(gamma + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (g[i] * d[i] - s1 - (f[i] - mean) * rstd * s2);
        if (dx_add) {
          float a[8];
          load8(dx_add + r * C + c, a);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += a[i];
        }
        store8(dx + r * C + c, o);
      }
    }
  }
  __syncthreads();
  // the 8 warps' accumulators are added in warp order
  for (int j = threadIdx.x; j < W; j += NORM_WARPS * 32) {
    const int c = (j & ~255) + (j & 31) * 8 + ((j >> 5) & 7);
    if (c < C) {
      float a = 0.f, bsum = 0.f;
#pragma unroll
      for (int w = 0; w < NORM_WARPS; ++w) {
        a += acc_smem[(w * NA + 0) * W + j];
        bsum += acc_smem[(w * NA + 1) * W + j];
      }
      scratch[((long long)blockIdx.x * NA + 0) * C + c] = a;
      scratch[((long long)blockIdx.x * NA + 1) * C + c] = bsum;
    }
  }
}

// The one-pass backward that also produces the column sums of the dx it writes (the incoming residual gradient
// included): that is the bias gradient of the linear layer whose output entered the residual stream in front of this
// norm, which then needs no column-sum launch of its own.  Three partial sums per column, and a two-stage pipeline:
// a warp has only a few rows to work through, so in the kernel above the memory system idles while every warp computes
// and the warps idle while every load is in flight.  Here a warp requests its next row (x, dy and the incoming residual
// gradient, with that row's mean and rstd) before it starts on the current one.  The second set of row registers
// costs occupancy: two blocks of 7 warps per SM (128 registers), each warp with up to two rows in flight; 7 rather
// than 8 because 8192 rows over 148 SMs are then exactly four rows per warp.
__device__ __forceinline__ uint4 ld_issue_here(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <int ITER>
struct NormRow {
  uint4 x[ITER], d[ITER], a[ITER];
  float mean, rstd;
};

template <bool RMS, int ITER, int CW>
__global__ void __launch_bounds__(CW * 32, 2)
norm_bwd_colsum_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                       const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dx_add,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ scratch, long long rows, int C,
                       long long rows_per) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float acc_smem[];                     // [CW][3][ITER * 256]
  constexpr int W = ITER * 256;
  constexpr int NA = 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* gacc = acc_smem + (warp * NA + 0) * W;
  float* bacc = acc_smem + (warp * NA + 1) * W;
  float* cacc = acc_smem + (warp * NA + 2) * W;
#pragma unroll
  for (int j = lane; j < W; j += 32) {
    gacc[j] = 0.f;
    bacc[j] = 0.f;
    cacc[j] = 0.f;
  }
  __syncwarp();
  const long long r0 = (long long)blockIdx.x * rows_per;
  const long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  const float inv_c = 1.f / C;
  auto fetch = [&](NormRow<ITER>& R, long long r) {
    R.mean = RMS ? 0.f : mean_in[r];
    R.rstd = rstd_in[r];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = it * 256 + lane * 8;
      const bool in = c < C;
      const uint4 zero = make_uint4(0, 0, 0, 0);
      // volatile: the request must be issued here, ahead of the work on the current row, and not where the
      // compiler would otherwise sink it to (next to its first use, which would undo the pipeline)
      R.x[it] = in ? ld_issue_here(x + r * C + c) : zero;
      R.d[it] = in ? ld_issue_here(dy + r * C + c) : zero;   // d = 0 past C
      R.a[it] = (in && dx_add) ? ld_issue_here(dx_add + r * C + c) : zero;
    }
  };
  NormRow<ITER> cur, nxt;
  long long r = r0 + warp;
  if (r < r1) fetch(cur, r);
  for (; r < r1; r += CW) {
    if (r + CW < r1) fetch(nxt, r + CW);
    const float rstd = cur.rstd;
    const float nmr = -cur.mean * rstd;   // xhat = x * rstd + nmr
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      float f[8], d[8], g[8];
      unpack8(cur.x[it], f);
      unpack8(cur.d[it], d);
      if (it * 256 + lane * 8 < C) {
        load8(gamma + it * 256 + lane * 8, g);   // from L1: the two blocks of an SM leave it most of its capacity
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[i] = fmaf(f[i], rstd, nmr);   // xhat
        const float gd = g[i] * d[i];
        s1 += gd;
        s2 = fmaf(gd, f[i], s2);
      }
      // accumulators as float2 (columns 2p, 2p + 1 of this lane's eight): half the shared-memory instructions of a
      // scalar layout, and 32 lanes x 8 bytes are still conflict-free
#pragma unroll
      for (int p2 = 0; p2 < 4; ++p2) {
        float2* ga = reinterpret_cast<float2*>(gacc) + it * 128 + p2 * 32 + lane;
        float2* ba = reinterpret_cast<float2*>(bacc) + it * 128 + p2 * 32 + lane;
        float2 gv = *ga, bv = *ba;
        gv.x = fmaf(d[2 * p2], f[2 * p2], gv.x);
        gv.y = fmaf(d[2 * p2 + 1], f[2 * p2 + 1], gv.y);
        bv.x += d[2 * p2];
        bv.y += d[2 * p2 + 1];
        *ga = gv;
        *ba = bv;
      }
    }
    s1 = RMS ? 0.f : warp_sum(s1) * inv_c;
    s2 = warp_sum(s2) * inv_c;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int c = it * 256 + lane * 8;
      if (c < C) {
        float f[8], d[8], g[8], a[8], o[8];
        unpack8(cur.x[it], f);
        unpack8(cur.d[it], d);
        load8(gamma + c, g);
        unpack8(cur.a[it], a);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = fmaf(f[i], rstd, nmr);
          o[i] = fmaf(rstd, fmaf(-xh, s2, g[i] * d[i] - s1), a[i]);
        }
        store8(dx + r * C + c, o);
#pragma unroll
        for (int p2 = 0; p2 < 4; ++p2) {
          float2* ca = reinterpret_cast<float2*>(cacc) + it * 128 + p2 * 32 + lane;
          float2 cv = *ca;
          cv.x += o[2 * p2];
          cv.y += o[2 * p2 + 1];
          *ca = cv;
        }
      }
    }
    cur = nxt;
  }
  __syncthreads();
  // the 8 warps' accumulators are added in warp order
  for (int j = threadIdx.x; j < W; j += CW * 32) {
    const int c = (j & ~255) + ((j & 63) >> 1) * 8 + ((j >> 6) & 3) * 2 + (j & 1);   // float2 layout above
    if (c < C) {
      float a = 0.f, bsum = 0.f, csum = 0.f;
#pragma unroll
      for (int w = 0; w < CW; ++w) {
        a += acc_smem[(w * NA + 0) * W + j];
        bsum += acc_smem[(w * NA + 1) * W + j];
        csum += acc_smem[(w * NA + 2) * W + j];
      }
      scratch[((long long)blockIdx.x * NA + 0) * C + c] = a;
      scratch[((long long)blockIdx.x * NA + 1) * C + c] = bsum;
      scratch[((long long)blockIdx.x * NA + 2) * C + c] = csum;
    }
  }
}

static bool fused_bwd_ok(int C) { return (C % 8) == 0 && C <= 1024; }

// blocks of the fused kernel = partial sums per column: one wave of three blocks per SM, within the 4 MiB of partial
// sums the allocation-free entry point owns
static long long fused_rows_per(long long rows, int C) {
  long long blocks = (rows + NORM_WARPS - 1) / NORM_WARPS;
  long long cap = (1ll << 20) / (2ll * C);
  if (cap > 444) cap = 444;   // three blocks per SM: one wave
  if (blocks > cap) blocks = cap;
  return (rows + blocks - 1) / blocks;
}

// the pipelined kernel with column sums runs two blocks per SM: one wave of 296
constexpr int COLSUM_WARPS = 7;   // 2 x 7 warps per SM: 8192 rows over 148 SMs are four rows per warp, none idle
static long long colsum_rows_per(long long rows) {
  long long blocks = (rows + COLSUM_WARPS - 1) / COLSUM_WARPS;
  if (blocks > 296) blocks = 296;
  return (rows + blocks - 1) / blocks;
}
static int colsum_chunks(long long rows) {
  const long long rp = colsum_rows_per(rows);
  return (int)((rows + rp - 1) / rp);
}

static int param_chunks(long long rows, int C) {
  if (fused_bwd_ok(C)) {
    const long long rp = fused_rows_per(rows, C);
    return (int)((rows + rp - 1) / rp);
  }
  long long c = (rows + 127) / 128;
  if (c > 64) c = 64;
  if (c < 1) c = 1;
  return (int)c;
}

template <bool RMS>
static int norm_bwd_launch(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                           const void* dx_add, void* dx, float* dgamma, float* dbeta, float* scratch, long long rows,
                           int C, cudaStream_t s, float* dxsum = nullptr) {
  if (rows <= 0 || C <= 0) return INCIN_ERR_ARGUMENT;
  if (dxsum && !(dgamma && fused_bwd_ok(C))) return INCIN_ERR_ARGUMENT;   // column sums of dx: one-pass kernel only
  if (dgamma && fused_bwd_ok(C)) {
    if (!scratch) return INCIN_ERR_ARGUMENT;
    const long long rp = dxsum ? colsum_rows_per(rows) : fused_rows_per(rows, C);
    const int chunks = dxsum ? colsum_chunks(rows) : param_chunks(rows, C);
    const int iters = (C + 255) / 256;
    const int na = dxsum ? 3 : 2;
    const int warps = dxsum ? COLSUM_WARPS : NORM_WARPS;
    const size_t acc_bytes = (size_t)warps * na * iters * 256 * sizeof(float);   // 8 KB per 256 columns and sum
    static PerDeviceFlags attr_set[10];   // per kernel (RMS is a template argument here) and per device
    bool attr_ok = true;
    auto go = [&](auto kern) {
      if (!ensure_dynamic_smem(kern, (int)acc_bytes, attr_set[iters + (dxsum ? 5 : 0)])) {
        attr_ok = false;   // nothing was launched: the partial sums must not be reduced either
        return;
      }
      launch_pdl(kern, dim3((unsigned)chunks), dim3(warps * 32), acc_bytes, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                 (const __nv_bfloat16*)gamma, mean, rstd, (const __nv_bfloat16*)dx_add, (__nv_bfloat16*)dx, scratch, rows, C, rp);
    };
    if (dxsum) {
      if (iters == 1) go(norm_bwd_colsum_kernel<RMS, 1, COLSUM_WARPS>);
      else if (iters == 2) go(norm_bwd_colsum_kernel<RMS, 2, COLSUM_WARPS>);
      else if (iters == 3) go(norm_bwd_colsum_kernel<RMS, 3, COLSUM_WARPS>);
      else go(norm_bwd_colsum_kernel<RMS, 4, COLSUM_WARPS>);
    } else if (iters == 1) go(norm_bwd_fused_kernel<RMS, 1>);
    else if (iters == 2) go(norm_bwd_fused_kernel<RMS, 2>);
    else if (iters == 3) go(norm_bwd_fused_kernel<RMS, 3>);
    else go(norm_bwd_fused_kernel<RMS, 4>);
    if (!attr_ok) return INCIN_ERR_DRIVER;
    launch_pdl(norm_bwd_param_final, dim3((C + 31) / 32), dim3(32 * PF_LANES), 0, s, scratch, dgamma, dbeta, C, chunks, na, dxsum);
    return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
  }
  const unsigned blocks = (unsigned)((rows + NORM_WARPS - 1) / NORM_WARPS);
  launch_pdl(norm_bwd_dx_kernel<RMS>, dim3(blocks), dim3(NORM_WARPS * 32), 0, s, 
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd,
      (const __nv_bfloat16*)dx_add, (__nv_bfloat16*)dx, rows, C);
  if (dgamma) {
    if (!scratch) return INCIN_ERR_ARGUMENT;
    const int chunks = param_chunks(rows, C);
    if ((C % 8) == 0) {
      dim3 grid((C + 255) / 256, chunks);
      launch_pdl(norm_bwd_param_partial_vec<RMS>, dim3(grid), dim3(256), 0, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean,
                                                           rstd, scratch, rows, C, chunks);
    } else {
      dim3 grid((C + PG_COLS - 1) / PG_COLS, chunks);
      launch_pdl(norm_bwd_param_partial<RMS>, dim3(grid), dim3(32 * PG_TY), 0, s, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                               mean, rstd, scratch, rows, C, chunks);
    }
    launch_pdl(norm_bwd_param_final, dim3((C + 31) / 32), dim3(32 * PF_LANES), 0, s, scratch, dgamma, dbeta, C, chunks, 2, (float*)nullptr);
  }
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace incin

using namespace incin;

extern "C" int incin_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                                   float* rstd, long long rows, int C, float eps, void* stream) {
  if (rows <= 0 || C <= 0 || !x || !gamma || !y || !rstd) return INCIN_ERR_ARGUMENT;
  norm_fwd_launch<false>(x, gamma, beta, y, mean, rstd, rows, C, eps, (cudaStream_t)stream);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, long long rows, int C,
                                 float eps, void* stream) {
  if (rows <= 0 || C <= 0 || !x || !gamma || !y || !rstd) return INCIN_ERR_ARGUMENT;
  norm_fwd_launch<true>(x, gamma, nullptr, y, nullptr, rstd, rows, C, eps, (cudaStream_t)stream);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" long long incin_layernorm_bwd_scratch_floats(long long rows, int C) {
  return (long long)param_chunks(rows, C) * 2 * C;
}

extern "C" int incin_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                                   const float* rstd, const void* dx_add, void* dx, float* dgamma, float* dbeta,
                                   float* scratch, long long rows, int C, void* stream) {
  return norm_bwd_launch<false>(dy, x, gamma, mean, rstd, dx_add, dx, dgamma, dbeta, scratch, rows, C,
                                (cudaStream_t)stream);
}

// LayerNorm backward that also accumulates the column sums of the dx it writes into dxsum[C] (fp32, +=): the bias
// gradient of the linear layer in front of this norm on the residual stream.  C % 8 == 0 and C <= 1024 (the one-pass
// kernel); scratch holds incin_layernorm_bwd_colsum_scratch_floats(rows, C) floats.
extern "C" long long incin_layernorm_bwd_colsum_scratch_floats(long long rows, int C) {
  return (long long)colsum_chunks(rows) * 3 * C;
}

extern "C" int incin_layernorm_bwd_colsum(const void* dy, const void* x, const void* gamma, const float* mean,
                                          const float* rstd, const void* dx_add, void* dx, float* dgamma, float* dbeta,
                                          float* dxsum, float* scratch, long long rows, int C, void* stream) {
  if (!dxsum) return INCIN_ERR_ARGUMENT;
  return norm_bwd_launch<false>(dy, x, gamma, mean, rstd, dx_add, dx, dgamma, dbeta, scratch, rows, C,
                                (cudaStream_t)stream, dxsum);
}

extern "C" int incin_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd,
                                 const void* dx_add, void* dx, float* dgamma, float* scratch, long long rows, int C,
                                 void* stream) {
  return norm_bwd_launch<true>(dy, x, gamma, nullptr, rstd, dx_add, dx, dgamma, nullptr, scratch, rows, C,
                               (cudaStream_t)stream);
}
