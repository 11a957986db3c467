// Convolution helpers, pooling and batch normalisation for sm_100a (NCHW, bf16 or fp32 io, fp32 arithmetic).
//
// Counterparts in the reference: im2col / col2im (crates/incin-backends/src/cuda/ops/kernels/conv.cu:5-181, fold
// with atomicAdd), pooling (pool.cu:7-248, backward with atomics) and the inference-only per-element batch norm
// (crates/incin-backends/src/kernel.rs:1345-1389).  Differences here:
//   * im2col writes the [N*OH*OW, C*KH*KW] matrix the tcgen05 GEMM consumes directly (K-major rows), and col2im
//     GATHERS the contributions of each input pixel, so the data gradient needs no atomics and is deterministic;
//   * max pooling keeps the argmax (int32 offset inside the plane) so its backward is a gather as well;
//   * batch norm has a training forward (per-channel mean / biased variance in one pass over the channel with a
//     block per channel, running statistics updated in the same kernel) and a full backward.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "incin_b200.h"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

struct ConvGeom {
  int N, C, H, W, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
};

// cols[(n*OH+oh)*OW+ow][(c*KH+kh)*KW+kw] = x[n][c][oh*sh-ph+kh*dh][ow*sw-pw+kw*dw] (0 outside)
template <typename T>
__global__ void im2col_kernel(const T* __restrict__ x, T* __restrict__ cols, ConvGeom g, long long total) {
  const int K = g.C * g.KH * g.KW;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(t % K);
    const long long row = t / K;
    const int ow = (int)(row % g.OW), oh = (int)((row / g.OW) % g.OH), n = (int)(row / ((long long)g.OW * g.OH));
    const int kw = k % g.KW, kh = (k / g.KW) % g.KH, c = k / (g.KW * g.KH);
    const int ih = oh * g.sh - g.ph + kh * g.dh, iw = ow * g.sw - g.pw + kw * g.dw;
    T v = T(0.0f);
    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) v = x[(((long long)n * g.C + c) * g.H + ih) * g.W + iw];
    cols[t] = v;
  }
}

// dx[n][c][ih][iw] = sum over the (kh, kw, oh, ow) that read this pixel: a gather, no atomics
template <typename T>
__global__ void col2im_kernel(const T* __restrict__ cols, T* __restrict__ dx, ConvGeom g, long long total) {
  const int K = g.C * g.KH * g.KW;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int iw = (int)(t % g.W), ih = (int)((t / g.W) % g.H);
    const int c = (int)((t / ((long long)g.W * g.H)) % g.C), n = (int)(t / ((long long)g.W * g.H * g.C));
    float acc = 0.0f;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int hh = ih + g.ph - kh * g.dh;
      if (hh < 0 || hh % g.sh) continue;
      const int oh = hh / g.sh;
      if (oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int ww = iw + g.pw - kw * g.dw;
        if (ww < 0 || ww % g.sw) continue;
        const int ow = ww / g.sw;
        if (ow >= g.OW) continue;
        acc += ldf(cols, (((long long)n * g.OH + oh) * g.OW + ow) * K + (c * g.KH + kh) * g.KW + kw);
      }
    }
    stf(dx, t, acc);
  }
}

// ---- pooling ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int* __restrict__ arg, ConvGeom g, long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(t % g.OW), oh = (int)((t / g.OW) % g.OH);
    const long long plane = t / ((long long)g.OW * g.OH);
    const T* p = x + plane * g.H * g.W;
    float best = -INFINITY;
    int best_i = -1;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int ih = oh * g.sh - g.ph + kh;
      if (ih < 0 || ih >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int iw = ow * g.sw - g.pw + kw;
        if (iw < 0 || iw >= g.W) continue;
        const float v = ldf(p, (long long)ih * g.W + iw);
        if (v > best || v != v || best_i < 0) {
          best = v;
          best_i = ih * g.W + iw;
        }
      }
    }
    stf(y, t, best);
    if (arg) arg[t] = best_i;
  }
}

// dx[plane][i] = sum of dy over the windows whose argmax is i: gather over the windows that cover pixel i
template <typename T>
__global__ void maxpool_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ arg, T* __restrict__ dx, ConvGeom g,
                                   long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int iw = (int)(t % g.W), ih = (int)((t / g.W) % g.H);
    const long long plane = t / ((long long)g.W * g.H);
    const int me = ih * g.W + iw;
    float acc = 0.0f;
    const int oh_lo = max(0, (ih + g.ph - g.KH + g.sh) / g.sh), oh_hi = min(g.OH - 1, (ih + g.ph) / g.sh);
    const int ow_lo = max(0, (iw + g.pw - g.KW + g.sw) / g.sw), ow_hi = min(g.OW - 1, (iw + g.pw) / g.sw);
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const long long o = (plane * g.OH + oh) * g.OW + ow;
        if (arg[o] == me) acc += ldf(dy, o);
      }
    stf(dx, t, acc);
  }
}

// average pooling (padding counted in the divisor, like the CPU oracle); backward when `bwd`
template <typename T>
__global__ void avgpool_kernel(const T* __restrict__ in, T* __restrict__ out, ConvGeom g, long long total, int bwd) {
  const float inv = 1.0f / (float)(g.KH * g.KW);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    float acc = 0.0f;
    if (!bwd) {
      const int ow = (int)(t % g.OW), oh = (int)((t / g.OW) % g.OH);
      const long long plane = t / ((long long)g.OW * g.OH);
      for (int kh = 0; kh < g.KH; ++kh) {
        const int ih = oh * g.sh - g.ph + kh;
        if (ih < 0 || ih >= g.H) continue;
        for (int kw = 0; kw < g.KW; ++kw) {
          const int iw = ow * g.sw - g.pw + kw;
          if (iw >= 0 && iw < g.W) acc += ldf(in, (plane * g.H + ih) * g.W + iw);
        }
      }
    } else {
      const int iw = (int)(t % g.W), ih = (int)((t / g.W) % g.H);
      const long long plane = t / ((long long)g.W * g.H);
      const int oh_lo = max(0, (ih + g.ph - g.KH + g.sh) / g.sh), oh_hi = min(g.OH - 1, (ih + g.ph) / g.sh);
      const int ow_lo = max(0, (iw + g.pw - g.KW + g.sw) / g.sw), ow_hi = min(g.OW - 1, (iw + g.pw) / g.sw);
      for (int oh = oh_lo; oh <= oh_hi; ++oh)
        for (int ow = ow_lo; ow <= ow_hi; ++ow) acc += ldf(in, (plane * g.OH + oh) * g.OW + ow);
    }
    stf(out, t, acc * inv);
  }
}

// ---- batch norm (one block per channel) -------------------------------------------------------------------------
__device__ __forceinline__ float2 block_sum2(float a, float b) {
  __shared__ float sa[32], sb[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    sa[threadIdx.x >> 5] = a;
    sb[threadIdx.x >> 5] = b;
  }
  __syncthreads();
  float ra = 0.0f, rb = 0.0f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    ra += sa[w];
    rb += sb[w];
  }
  return make_float2(ra, rb);
}

template <typename T>
__global__ void __launch_bounds__(512) batchnorm_train_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                                                  const float* __restrict__ beta, T* __restrict__ y,
                                                                  float* __restrict__ save_mean, float* __restrict__ save_rstd,
                                                                  float* __restrict__ run_mean, float* __restrict__ run_var, int N, int C,
                                                                  long long HW, float eps, float momentum) {
  const int c = blockIdx.x;
  const long long count = (long long)N * HW;
  // shifted sums (shift = first element of the channel) keep the one-pass variance accurate for large means
  const float shift = ldf(x, (long long)c * HW);
  float s = 0.0f, ss = 0.0f;
  for (long long i = threadIdx.x; i < count; i += blockDim.x) {
    const long long n = i / HW, j = i % HW;
    const float v = ldf(x, (n * C + c) * HW + j) - shift;
    s += v;
    ss += v * v;
  }
  const float2 r = block_sum2(s, ss);
  const float m_sh = r.x / (float)count;
  const float var = fmaxf(r.y / (float)count - m_sh * m_sh, 0.0f);
  const float mean = m_sh + shift, rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    save_mean[c] = mean;
    save_rstd[c] = rstd;
    if (run_mean) run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * mean;
    if (run_var) run_var[c] = (1.0f - momentum) * run_var[c] + momentum * var * ((float)count / (float)(count > 1 ? count - 1 : 1));
  }
  const float ga = gamma ? gamma[c] : 1.0f, be = beta ? beta[c] : 0.0f;
  for (long long i = threadIdx.x; i < count; i += blockDim.x) {
    const long long n = i / HW, j = i % HW, o = (n * C + c) * HW + j;
    stf(y, o, (ldf(x, o) - mean) * rstd * ga + be);
  }
}

template <typename T>
__global__ void batchnorm_eval_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                      const float* __restrict__ mean, const float* __restrict__ var, T* __restrict__ y, int C,
                                      long long HW, float eps, long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int c = (int)((t / HW) % C);
    const float ga = gamma ? gamma[c] : 1.0f, be = beta ? beta[c] : 0.0f;
    stf(y, t, (ldf(x, t) - mean[c]) * rsqrtf(var[c] + eps) * ga + be);
  }
}

// dx = gamma*rstd/M * (M*dy - sum(dy) - xhat*sum(dy*xhat)); dgamma += sum(dy*xhat); dbeta += sum(dy)
template <typename T>
__global__ void __launch_bounds__(512) batchnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                            const float* __restrict__ gamma, const float* __restrict__ save_mean,
                                                            const float* __restrict__ save_rstd, T* __restrict__ dx,
                                                            float* __restrict__ dgamma, float* __restrict__ dbeta, int N, int C,
                                                            long long HW) {
  const int c = blockIdx.x;
  const long long count = (long long)N * HW;
  const float mean = save_mean[c], rstd = save_rstd[c];
  float s1 = 0.0f, s2 = 0.0f;
  for (long long i = threadIdx.x; i < count; i += blockDim.x) {
    const long long o = ((i / HW) * C + c) * HW + i % HW;
    const float g = ldf(dy, o);
    s1 += g;
    s2 += g * (ldf(x, o) - mean) * rstd;
  }
  const float2 r = block_sum2(s1, s2);
  if (threadIdx.x == 0) {
    if (dgamma) dgamma[c] += r.y;
    if (dbeta) dbeta[c] += r.x;
  }
  const float ga = gamma ? gamma[c] : 1.0f;
  const float k = ga * rstd / (float)count;
  for (long long i = threadIdx.x; i < count; i += blockDim.x) {
    const long long o = ((i / HW) * C + c) * HW + i % HW;
    const float xh = (ldf(x, o) - mean) * rstd;
    stf(dx, o, k * ((float)count * ldf(dy, o) - r.x - xh * r.y));
  }
}

// ---- adaptive average pooling: output cell (oh, ow) averages rows [floor(oh*H/OH), ceil((oh+1)*H/OH)) x the same in w
// (crates/incin-backends/src/cuda/ops/kernels/pool.cu adaptive_avg_pool2d_{fwd,bwd}; the backward there scatters with
// atomics, here every input pixel gathers from the output cells whose window contains it)
__device__ __forceinline__ int ad_start(int o, int in, int out) { return (int)(((long long)o * in) / out); }
__device__ __forceinline__ int ad_end(int o, int in, int out) { return (int)((((long long)o + 1) * in + out - 1) / out); }

template <typename T>
__global__ void adaptive_avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W, int OH, int OW, long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(t % OW), oh = (int)((t / OW) % OH);
    const long long plane = t / ((long long)OW * OH);
    const int h0 = ad_start(oh, H, OH), h1 = ad_end(oh, H, OH), w0 = ad_start(ow, W, OW), w1 = ad_end(ow, W, OW);
    const T* p = x + plane * H * W;
    float acc = 0.0f;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) acc += ldf(p, (long long)h * W + w);
    stf(y, t, acc / (float)((h1 - h0) * (w1 - w0)));
  }
}

template <typename T>
__global__ void adaptive_avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int H, int W, int OH, int OW, long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(t % W), h = (int)((t / W) % H);
    const long long plane = t / ((long long)W * H);
    const T* p = dy + plane * OH * OW;
    // output rows whose window [start, end) contains h: start(oh) <= h  and  end(oh) > h
    int oh_lo = (int)(((long long)h * OH) / H), oh_hi = (int)((((long long)h + 1) * OH + H - 1) / H);
    while (oh_lo > 0 && ad_end(oh_lo - 1, H, OH) > h) --oh_lo;
    while (oh_hi < OH && ad_start(oh_hi, H, OH) <= h) ++oh_hi;
    int ow_lo = (int)(((long long)w * OW) / W), ow_hi = (int)((((long long)w + 1) * OW + W - 1) / W);
    while (ow_lo > 0 && ad_end(ow_lo - 1, W, OW) > w) --ow_lo;
    while (ow_hi < OW && ad_start(ow_hi, W, OW) <= w) ++ow_hi;
    float acc = 0.0f;
    for (int oh = oh_lo; oh < oh_hi; ++oh) {
      const int h0 = ad_start(oh, H, OH), h1 = ad_end(oh, H, OH);
      if (h < h0 || h >= h1) continue;
      for (int ow = ow_lo; ow < ow_hi; ++ow) {
        const int w0 = ad_start(ow, W, OW), w1 = ad_end(ow, W, OW);
        if (w < w0 || w >= w1) continue;
        acc += ldf(p, (long long)oh * OW + ow) / (float)((h1 - h0) * (w1 - w0));
      }
    }
    stf(dx, t, acc);
  }
}

inline unsigned grid_for(long long n) {
  long long g = (n + 255) / 256;
  return (unsigned)(g < 1 ? 1 : (g > 148LL * 16 ? 148LL * 16 : g));
}

ConvGeom geom(const incin_conv_geom* d) {
  ConvGeom g;
  g.N = d->N; g.C = d->C; g.H = d->H; g.W = d->W; g.KH = d->KH; g.KW = d->KW;
  g.sh = d->stride_h; g.sw = d->stride_w; g.ph = d->pad_h; g.pw = d->pad_w;
  g.dh = d->dil_h > 0 ? d->dil_h : 1; g.dw = d->dil_w > 0 ? d->dil_w : 1;
  g.OH = (g.H + 2 * g.ph - g.dh * (g.KH - 1) - 1) / g.sh + 1;
  g.OW = (g.W + 2 * g.pw - g.dw * (g.KW - 1) - 1) / g.sw + 1;
  return g;
}

bool valid(const incin_conv_geom* d) {
  return d && d->N > 0 && d->C > 0 && d->H > 0 && d->W > 0 && d->KH > 0 && d->KW > 0 && d->stride_h > 0 && d->stride_w > 0 &&
         d->pad_h >= 0 && d->pad_w >= 0 && (d->H + 2 * d->pad_h - (d->dil_h > 0 ? d->dil_h : 1) * (d->KH - 1) - 1) >= 0 &&
         (d->W + 2 * d->pad_w - (d->dil_w > 0 ? d->dil_w : 1) * (d->KW - 1) - 1) >= 0;
}

}  // namespace

#define DISPATCH(is_bf16, CALL_BF16, CALL_F32) \
  do {                                         \
    if (is_bf16) { CALL_BF16; } else { CALL_F32; } \
  } while (0)

extern "C" int incin_conv_out_hw(const incin_conv_geom* d, int* oh, int* ow) {
  if (!valid(d) || !oh || !ow) return INCIN_ERR_ARGUMENT;
  const ConvGeom g = geom(d);
  *oh = g.OH;
  *ow = g.OW;
  return INCIN_OK;
}

extern "C" int incin_im2col(const void* x, void* cols, const incin_conv_geom* d, int is_bf16, void* stream) {
  if (!x || !cols || !valid(d)) return INCIN_ERR_ARGUMENT;
  const ConvGeom g = geom(d);
  const long long total = (long long)g.N * g.OH * g.OW * g.C * g.KH * g.KW;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (im2col_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(cols), g, total)),
           (im2col_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(cols), g, total)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_col2im(const void* cols, void* dx, const incin_conv_geom* d, int is_bf16, void* stream) {
  if (!cols || !dx || !valid(d)) return INCIN_ERR_ARGUMENT;
  const ConvGeom g = geom(d);
  const long long total = (long long)g.N * g.C * g.H * g.W;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (col2im_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(cols), static_cast<__nv_bfloat16*>(dx), g, total)),
           (col2im_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(cols), static_cast<float*>(dx), g, total)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_maxpool2d_fwd(const void* x, void* y, int* argmax, const incin_conv_geom* d, int is_bf16, void* stream) {
  if (!x || !y || !valid(d)) return INCIN_ERR_ARGUMENT;
  const ConvGeom g = geom(d);
  const long long total = (long long)g.N * g.C * g.OH * g.OW;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (maxpool_fwd_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), argmax, g, total)),
           (maxpool_fwd_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(y), argmax, g, total)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_maxpool2d_bwd(const void* dy, const int* argmax, void* dx, const incin_conv_geom* d, int is_bf16,
                                   void* stream) {
  if (!dy || !argmax || !dx || !valid(d)) return INCIN_ERR_ARGUMENT;
  const ConvGeom g = geom(d);
  const long long total = (long long)g.N * g.C * g.H * g.W;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (maxpool_bwd_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), argmax, static_cast<__nv_bfloat16*>(dx), g, total)),
           (maxpool_bwd_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(dy), argmax, static_cast<float*>(dx), g, total)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_avgpool2d(const void* in, void* out, const incin_conv_geom* d, int backward, int is_bf16, void* stream) {
  if (!in || !out || !valid(d)) return INCIN_ERR_ARGUMENT;
  const ConvGeom g = geom(d);
  const long long total = backward ? (long long)g.N * g.C * g.H * g.W : (long long)g.N * g.C * g.OH * g.OW;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (avgpool_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), g, total, backward)),
           (avgpool_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(in), static_cast<float*>(out), g, total, backward)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_batchnorm_train_fwd(const void* x, const float* gamma, const float* beta, void* y, float* save_mean,
                                         float* save_rstd, float* running_mean, float* running_var, int N, int C, long long HW,
                                         float eps, float momentum, int is_bf16, void* stream) {
  if (!x || !y || !save_mean || !save_rstd || N <= 0 || C <= 0 || HW <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (batchnorm_train_fwd_kernel<__nv_bfloat16><<<C, 512, 0, s>>>(static_cast<const __nv_bfloat16*>(x), gamma, beta, static_cast<__nv_bfloat16*>(y), save_mean, save_rstd, running_mean, running_var, N, C, HW, eps, momentum)),
           (batchnorm_train_fwd_kernel<float><<<C, 512, 0, s>>>(static_cast<const float*>(x), gamma, beta, static_cast<float*>(y), save_mean, save_rstd, running_mean, running_var, N, C, HW, eps, momentum)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_batchnorm_eval(const void* x, const float* gamma, const float* beta, const float* mean, const float* var,
                                    void* y, int N, int C, long long HW, float eps, int is_bf16, void* stream) {
  if (!x || !y || !mean || !var || N <= 0 || C <= 0 || HW <= 0) return INCIN_ERR_ARGUMENT;
  const long long total = (long long)N * C * HW;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (batchnorm_eval_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), gamma, beta, mean, var, static_cast<__nv_bfloat16*>(y), C, HW, eps, total)),
           (batchnorm_eval_kernel<float><<<grid_for(total), 256, 0, s>>>(static_cast<const float*>(x), gamma, beta, mean, var, static_cast<float*>(y), C, HW, eps, total)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_batchnorm_bwd(const void* dy, const void* x, const float* gamma, const float* save_mean,
                                   const float* save_rstd, void* dx, float* dgamma, float* dbeta, int N, int C, long long HW,
                                   int is_bf16, void* stream) {
  if (!dy || !x || !dx || !save_mean || !save_rstd || N <= 0 || C <= 0 || HW <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH(is_bf16, (batchnorm_bwd_kernel<__nv_bfloat16><<<C, 512, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma, save_mean, save_rstd, static_cast<__nv_bfloat16*>(dx), dgamma, dbeta, N, C, HW)),
           (batchnorm_bwd_kernel<float><<<C, 512, 0, s>>>(static_cast<const float*>(dy), static_cast<const float*>(x), gamma, save_mean, save_rstd, static_cast<float*>(dx), dgamma, dbeta, N, C, HW)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_adaptive_avgpool2d(const void* in, void* out, long long planes, int H, int W, int OH, int OW, int backward,
                                        int is_bf16, void* stream) {
  if (!in || !out || planes <= 0 || H <= 0 || W <= 0 || OH <= 0 || OW <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = planes * (backward ? (long long)H * W : (long long)OH * OW);
  if (backward)
    DISPATCH(is_bf16,
             (adaptive_avgpool_bwd_kernel<<<grid_for(total), 256, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, H, W, OH, OW, total)),
             (adaptive_avgpool_bwd_kernel<<<grid_for(total), 256, 0, s>>>((const float*)in, (float*)out, H, W, OH, OW, total)));
  else
    DISPATCH(is_bf16,
             (adaptive_avgpool_fwd_kernel<<<grid_for(total), 256, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, H, W, OH, OW, total)),
             (adaptive_avgpool_fwd_kernel<<<grid_for(total), 256, 0, s>>>((const float*)in, (float*)out, H, W, OH, OW, total)));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}
