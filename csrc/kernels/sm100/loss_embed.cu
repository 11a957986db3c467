// Embedding gather/scatter, fused softmax-cross-entropy (online log-sum-exp),
// causal softmax for the materialised-scores attention path, column sums.
//
// The reference computes cross entropy as softmax (8 launches) -> log -> nll
// -> mean (crates/incin-backends/src/cuda/backend.rs:1849-1867) and its
// nll_loss kernel reads int64 targets through an int* (loss.cu:6); here targets
// are int64 end to end and the whole loss is two passes over the logits.
#include "ptx.cuh"
#include "launch.cuh"
#include "../../include/incin_b200.h"
#include <math_constants.h>

namespace incin {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum_f(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) t = warp_sum_f(t);
  if (threadIdx.x == 0) sh[0] = t;
  __syncthreads();
  return sh[0];
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max_f(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? sh[threadIdx.x] : -CUDART_INF_F;
  if (w == 0) t = warp_max_f(t);
  if (threadIdx.x == 0) sh[0] = t;
  __syncthreads();
  return sh[0];
}

// ----------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ tok, const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out,
                                     long long BT, int T, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  if (row >= BT) return;
  const int t = (int)(row % T);
  const __nv_bfloat16* e = wte + tok[row] * (long long)C;
  const __nv_bfloat16* p = wpe ? wpe + (long long)t * C : nullptr;
  __nv_bfloat16* o = out + row * C;
  if ((C & 7) == 0) {
    for (int c = threadIdx.x * 8; c < C; c += blockDim.x * 8) {
      uint4 a = *reinterpret_cast<const uint4*>(e + c);
      if (p) {
        const uint4 b = *reinterpret_cast<const uint4*>(p + c);
        uint32_t* aw = reinterpret_cast<uint32_t*>(&a);
        const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 x = unpack_bf16x2(aw[i]), y = unpack_bf16x2(bw[i]);
          aw[i] = pack_bf16x2(x.x + y.x, x.y + y.y);
        }
      }
      *reinterpret_cast<uint4*>(o + c) = a;
    }
  } else {
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float v = __bfloat162float(e[c]);
      if (p) v += __bfloat162float(p[c]);
      o[c] = __float2bfloat16(v);
    }
  }
}

__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int64_t* __restrict__ tok,
                                     float* __restrict__ dwte, float* __restrict__ dwpe, long long BT, int T, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  if (row >= BT) return;
  const int t = (int)(row % T);
  float* ge = dwte + tok[row] * (long long)C;
  float* gp = dwpe ? dwpe + (long long)t * C : nullptr;
  const __nv_bfloat16* d = dout + row * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = __bfloat162float(d[c]);
    atomicAdd(ge + c, v);
    if (gp) atomicAdd(gp + c, v);
  }
}

// ----------------------------------------------------------------------------- cross entropy
constexpr int XENT_THREADS = 512;

// log-sum-exp of one row, computed by the whole block (online: running max m and sum s of exp(x - m)); every thread
// returns the same value
__device__ __forceinline__ float xent_row_lse(const __nv_bfloat16* __restrict__ lr, int V, long long ld, float* sh) {
  float m = -CUDART_INF_F, s = 0.f;
  const bool vec = (ld % 8 == 0);
  if (vec) {
    const int Vv = V & ~7;
    for (int c = threadIdx.x * 8; c < Vv; c += XENT_THREADS * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(lr + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      float f[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = unpack_bf16x2(w[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
      }
      float mx = f[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) mx = fmaxf(mx, f[i]);
      if (mx > m) {
        s *= __expf(m - mx);
        m = mx;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
    }
    for (int c = Vv + threadIdx.x; c < V; c += XENT_THREADS) {
      const float x = __bfloat162float(lr[c]);
      if (x > m) {
        s *= __expf(m - x);
        m = x;
      }
      s += __expf(x - m);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += XENT_THREADS) {
      const float x = __bfloat162float(lr[c]);
      if (x > m) {
        s *= __expf(m - x);
        m = x;
      }
      s += __expf(x - m);
    }
  }
  const float gm = block_max<XENT_THREADS>(m, sh);
  const float part = (m == -CUDART_INF_F) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<XENT_THREADS>(part, sh);
  return gm + logf(gs);
}

// the row becomes its own gradient: (softmax - onehot(t)) * g, zero in the padding columns [V, ld)
__device__ __forceinline__ void xent_row_grad(__nv_bfloat16* __restrict__ lr, long long t, float lse, float g, int V,
                                              long long ld) {
  const int LD = (int)ld;
  if (ld % 8 == 0) {
    for (int c = threadIdx.x * 8; c < LD; c += XENT_THREADS * 8) {
      uint4 u = *reinterpret_cast<const uint4*>(lr + c);
      uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack_bf16x2(w[i]);
        const int c0 = c + 2 * i, c1 = c0 + 1;
        const float p0 = c0 < V ? (__expf(x.x - lse) - (c0 == t ? 1.f : 0.f)) * g : 0.f;
        const float p1 = c1 < V ? (__expf(x.y - lse) - (c1 == t ? 1.f : 0.f)) * g : 0.f;
        w[i] = pack_bf16x2(p0, p1);
      }
      *reinterpret_cast<uint4*>(lr + c) = u;
    }
  } else {
    for (int c = threadIdx.x; c < LD; c += XENT_THREADS) {
      const float x = __bfloat162float(lr[c]);
      const float p = c < V ? (__expf(x - lse) - (c == t ? 1.f : 0.f)) * g : 0.f;
      lr[c] = __float2bfloat16(p);
    }
  }
}

__global__ void __launch_bounds__(XENT_THREADS)
xent_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                float* __restrict__ loss, float* __restrict__ lse_out, int V, long long ld) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  const float lse = xent_row_lse(lr, V, ld, sh);
  if (threadIdx.x == 0) {
    lse_out[row] = lse;
    const long long t = targets[row];
    loss[row] = (t >= 0 && t < V) ? lse - __bfloat162float(lr[t]) : 0.f;  // out-of-range = ignored row
  }
}

__global__ void __launch_bounds__(XENT_THREADS)
xent_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                const float* __restrict__ lse_in, const float* __restrict__ dloss, float scale, int V, long long ld) {
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  const long long t = targets[row];
  const bool live = (t >= 0 && t < V);
  const float g = live ? (dloss ? dloss[0] : 1.f) * scale : 0.f;
  xent_row_grad(logits + row * ld, t, lse_in[row], g, V, ld);
}

// Loss and gradient in one launch: the row is read for its log-sum-exp, read again (from L2: a row is at most a few
// hundred KB and was just touched by this block) and overwritten by (softmax - onehot) * scale.  The caller applies the
// upstream gradient of the loss as a device scalar in the GEMMs that consume the row gradients.
__global__ void __launch_bounds__(XENT_THREADS)
xent_fused_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets, float* __restrict__ loss,
                  float* __restrict__ lse_out, float scale, int V, long long ld) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long t = targets[row];
  const bool live = (t >= 0 && t < V);
  const float lse = xent_row_lse(lr, V, ld, sh);
  if (threadIdx.x == 0) {
    lse_out[row] = lse;
    loss[row] = live ? lse - __bfloat162float(lr[t]) : 0.f;
  }
  __syncthreads();   // the target logit has been read before any thread overwrites the row
  xent_row_grad(lr, t, lse, live ? scale : 0.f, V, ld);
}

__global__ void __launch_bounds__(1024) mean_kernel(const float* __restrict__ x, float* __restrict__ out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += 1024) s += x[i];
  const float t = block_sum<1024>(s, sh);
  if (threadIdx.x == 0) out[0] = t / (float)n;
}

// ----------------------------------------------------------------------------- causal softmax (composed attention)
// one warp per row; row r of a [T, T] score matrix keeps columns 0..r
__global__ void __launch_bounds__(256)
causal_softmax_fwd_kernel(__nv_bfloat16* __restrict__ s, long long total_rows, int T, float scale) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int r = (int)(row % T);
  __nv_bfloat16* p = s + row * T;
  const int n = r + 1;
  float m = -CUDART_INF_F;
  for (int c = lane; c < n; c += 32) m = fmaxf(m, __bfloat162float(p[c]) * scale);
  m = warp_max_f(m);
  float sum = 0.f;
  for (int c = lane; c < n; c += 32) sum += __expf(__bfloat162float(p[c]) * scale - m);
  sum = warp_sum_f(sum);
  const float inv = 1.f / sum;
  for (int c = lane; c < T; c += 32) {
    const float v = c < n ? __expf(__bfloat162float(p[c]) * scale - m) * inv : 0.f;
    p[c] = __float2bfloat16(v);
  }
}

__global__ void __launch_bounds__(256)
causal_softmax_bwd_kernel(__nv_bfloat16* __restrict__ dp, const __nv_bfloat16* __restrict__ pr, long long total_rows,
                          int T, float scale) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= total_rows) return;
  const int r = (int)(row % T);
  __nv_bfloat16* d = dp + row * T;
  const __nv_bfloat16* p = pr + row * T;
  const int n = r + 1;
  float dot = 0.f;
  for (int c = lane; c < n; c += 32) dot += __bfloat162float(d[c]) * __bfloat162float(p[c]);
  dot = warp_sum_f(dot);
  for (int c = lane; c < T; c += 32) {
    const float v = c < n ? __bfloat162float(p[c]) * (__bfloat162float(d[c]) - dot) * scale : 0.f;
    d[c] = __float2bfloat16(v);
  }
}

// ----------------------------------------------------------------------------- column sum (bias gradient)
// block = 32 x 8 threads covering 64 columns; grid.y row chunks; fp32 atomics into the gradient buffer
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ dbias, long long rows, int N, long long ld,
              int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 64 + tx * 2;
  const long long rows_per = (rows + chunks - 1) / chunks;
  const long long r0 = (long long)blockIdx.y * rows_per;
  const long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  float a0 = 0.f, a1 = 0.f;
  if (c0 < N) {
    const bool pair = (c0 + 1 < N) && ((ld & 1) == 0);
    for (long long r = r0 + ty; r < r1; r += 8) {
      if (pair) {
        const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + r * ld + c0));
        a0 += v.x;
        a1 += v.y;
      } else {
        a0 += __bfloat162float(dy[r * ld + c0]);
        if (c0 + 1 < N) a1 += __bfloat162float(dy[r * ld + c0 + 1]);
      }
    }
  }
  sh[ty][tx * 2] = a0;
  sh[ty][tx * 2 + 1] = a1;
  __syncthreads();
  if (ty == 0) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      if (c0 + e < N) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += sh[k][tx * 2 + e];
        atomicAdd(dbias + c0 + e, t);
      }
    }
  }
}

// 16-byte variant: 32 lanes x 8 columns = 256 columns per block, 8 row lanes, needs N % 8 == 0 and ld % 8 == 0
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ dbias, long long rows, int N,
                  long long ld, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + tx * 8;
  const long long rows_per = (rows + chunks - 1) / chunks;
  const long long r0 = (long long)blockIdx.y * rows_per;
  const long long r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
  float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < N) {
    for (long long r = r0 + ty; r < r1; r += 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(dy + r * ld + c0);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(w[i]);
        a[2 * i] += f.x;
        a[2 * i + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sh[ty][tx * 8 + i] = a[i];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sh[k][threadIdx.x];
    atomicAdd(dbias + c, t);
  }
}

}  // namespace incin

using namespace incin;
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH)

extern "C" int incin_embedding_fwd(const int64_t* tokens, const void* wte, const void* wpe, void* out, long long B,
                                   int T, int C, void* stream) {
  const long long BT = B * T;
  if (BT <= 0 || C <= 0 || BT > 0x7fffffffLL) return INCIN_ERR_ARGUMENT;
  int threads = C / 8 >= 128 ? 128 : 64;
  launch_pdl(embedding_fwd_kernel, dim3((unsigned)BT), dim3(threads), 0, (cudaStream_t)stream, 
      tokens, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, BT, T, C);
  return CHECK_LAUNCH();
}

extern "C" int incin_embedding_bwd(const void* dout, const int64_t* tokens, float* dwte, float* dwpe, long long B,
                                   int T, int C, void* stream) {
  const long long BT = B * T;
  if (BT <= 0 || C <= 0 || BT > 0x7fffffffLL) return INCIN_ERR_ARGUMENT;
  launch_pdl(embedding_bwd_kernel, dim3((unsigned)BT), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)dout, tokens, dwte, dwpe,
                                                                        BT, T, C);
  return CHECK_LAUNCH();
}

extern "C" int incin_xent_fwd(const void* logits, const int64_t* targets, float* loss, float* lse, long long rows,
                              int V, long long ld, void* stream) {
  if (rows <= 0 || V <= 0 || ld < V || rows > 0x7fffffffLL) return INCIN_ERR_ARGUMENT;
  launch_pdl(xent_fwd_kernel, dim3((unsigned)rows), dim3(XENT_THREADS), 0, (cudaStream_t)stream, (const __nv_bfloat16*)logits, targets,
                                                                              loss, lse, V, ld);
  return CHECK_LAUNCH();
}

extern "C" int incin_xent_fused(void* logits, const int64_t* targets, float* loss, float* lse, float scale,
                                long long rows, int V, long long ld, void* stream) {
  if (!logits || !targets || !loss || !lse || rows <= 0 || V <= 0 || ld < V) return INCIN_ERR_ARGUMENT;
  launch_pdl(xent_fused_kernel, dim3((unsigned)rows), dim3(XENT_THREADS), 0, (cudaStream_t)stream, (__nv_bfloat16*)logits,
             targets, loss, lse, scale, V, ld);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_xent_bwd(void* logits, const int64_t* targets, const float* lse, const float* dloss, float scale,
                              long long rows, int V, long long ld, void* stream) {
  if (rows <= 0 || V <= 0 || ld < V || rows > 0x7fffffffLL || ld > 0x7fffffffLL) return INCIN_ERR_ARGUMENT;
  launch_pdl(xent_bwd_kernel, dim3((unsigned)rows), dim3(XENT_THREADS), 0, (cudaStream_t)stream, (__nv_bfloat16*)logits, targets, lse,
                                                                              dloss, scale, V, ld);
  return CHECK_LAUNCH();
}

extern "C" int incin_mean_f32(const float* x, float* out, long long n, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  launch_pdl(mean_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, x, out, n);
  return CHECK_LAUNCH();
}

extern "C" int incin_causal_softmax_fwd(void* scores, long long batch, int T, float scale, void* stream) {
  const long long rows = batch * T;
  if (rows <= 0) return INCIN_ERR_ARGUMENT;
  causal_softmax_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)scores, rows,
                                                                                           T, scale);
  return CHECK_LAUNCH();
}

extern "C" int incin_causal_softmax_bwd(void* dp, const void* p, long long batch, int T, float scale, void* stream) {
  const long long rows = batch * T;
  if (rows <= 0) return INCIN_ERR_ARGUMENT;
  causal_softmax_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)dp, (const __nv_bfloat16*)p, rows, T, scale);
  return CHECK_LAUNCH();
}

extern "C" int incin_colsum_accum(const void* dy, float* dbias, long long rows, int N, long long ld, void* stream) {
  if (rows <= 0 || N <= 0) return INCIN_ERR_ARGUMENT;
  if ((N % 8) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0) {
    const int colblocks = (N + 255) / 256;
    long long chunks = (148 * 4 + colblocks - 1) / colblocks;
    if (chunks > (rows + 31) / 32) chunks = (rows + 31) / 32;
    if (chunks < 1) chunks = 1;
    dim3 grid(colblocks, (unsigned)chunks);
    launch_pdl(colsum_vec_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)dy, dbias, rows, N, ld, (int)chunks);
    return CHECK_LAUNCH();
  }
  long long chunks = (rows + 255) / 256;
  if (chunks > 128) chunks = 128;
  dim3 grid((N + 63) / 64, (unsigned)chunks);
  launch_pdl(colsum_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)dy, dbias, rows, N, ld, (int)chunks);
  return CHECK_LAUNCH();
}
