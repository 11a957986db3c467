// Flat-buffer optimisers (AdamW / SGD with fp32 master weights and a bf16
// shadow copy), device-side gradient health check, casts, activations, SwiGLU,
// rotary embedding, Philox RNG and dropout.  All of these are bandwidth bound:
// 16-byte accesses, grid sized to a few waves of the 148 SMs, one launch per
// flat buffer rather than one per parameter tensor.
//
// The reference composes AdamW from ~15 elementwise launches per parameter
// (crates/incin-core/src/tensor/backend.rs:841-884), its dead fused kernel
// skips bias correction (cuda/ops/kernels/fused_adamw.cu:1-67) and its RNG is
// host-side thread_rng + H2D (cuda/backend.rs:993-1007).  The arithmetic here
// follows the CPU contract: bias-corrected moments, decoupled weight decay
// (crates/incin-backends/src/cpu/ops/optimizer.rs:43-59).
#include "ptx.cuh"
#include "launch.cuh"
#include "../../include/incin_b200.h"

namespace incin {

static inline unsigned grid_for(long long n, int per_block, int max_blocks = 148 * 16) {
  long long b = (n + per_block - 1) / per_block;
  if (b > max_blocks) b = max_blocks;
  if (b < 1) b = 1;
  return (unsigned)b;
}

// ----------------------------------------------------------------------------- optimisers
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ w, float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g,
                  __nv_bfloat16* __restrict__ shadow, long long n, long long n_decay,
                  const float* __restrict__ hyper) {
  pdl_launch_dependents();
  pdl_wait();
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4], step = hyper[5];
  const float gs = hyper[6];
  const float bc1 = 1.f - powf(b1, step), bc2 = 1.f - powf(b2, step);
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 gw = reinterpret_cast<const float4*>(g)[i];
    float4 ww = reinterpret_cast<float4*>(w)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* gp = reinterpret_cast<float*>(&gw);
    float* wp = reinterpret_cast<float*>(&ww);
    float* mp = reinterpret_cast<float*>(&mm);
    float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gr = gp[k] * gs;
      mp[k] = b1 * mp[k] + (1.f - b1) * gr;
      vp[k] = b2 * vp[k] + (1.f - b2) * gr * gr;
      const float mh = mp[k] / bc1, vh = vp[k] / bc2;
      const float decay = (i * 4 + k) < n_decay ? wd : 0.f;
      wp[k] = wp[k] - lr * decay * wp[k] - lr * mh / (sqrtf(vh) + eps);
    }
    reinterpret_cast<float4*>(w)[i] = ww;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (shadow) {
      uint2 o;
      o.x = pack_bf16x2(wp[0], wp[1]);
      o.y = pack_bf16x2(wp[2], wp[3]);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gr = g[i] * gs;
    const float mn = b1 * m[i] + (1.f - b1) * gr;
    const float vn = b2 * v[i] + (1.f - b2) * gr * gr;
    m[i] = mn;
    v[i] = vn;
    const float decay = i < n_decay ? wd : 0.f;
    const float wn = w[i] - lr * decay * w[i] - lr * (mn / bc1) / (sqrtf(vn / bc2) + eps);
    w[i] = wn;
    if (shadow) shadow[i] = __float2bfloat16(wn);
  }
}

__global__ void __launch_bounds__(256)
sgd_flat_kernel(float* __restrict__ w, float* __restrict__ mom, const float* __restrict__ g,
                __nv_bfloat16* __restrict__ shadow, long long n, long long n_decay, const float* __restrict__ hyper) {
  const float lr = hyper[0], mu = hyper[1], wd = hyper[4], gs = hyper[6];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float gr = g[i] * gs + (i < n_decay ? wd : 0.f) * w[i];
    if (mom) {
      const float b = mu * mom[i] + gr;
      mom[i] = b;
      gr = b;
    }
    const float wn = w[i] - lr * gr;
    w[i] = wn;
    if (shadow) shadow[i] = __float2bfloat16(wn);
  }
}

// out[0] += sum(x^2), out[1] = 1 if any non-finite
__global__ void __launch_bounds__(256)
sumsq_nonfinite_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float sh[8];
  float s = 0.f;
  bool bad = false;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = x[i];
    s += v * v;
    bad |= !isfinite(v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const bool any_bad = __syncthreads_or(bad);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < 8; ++k) t += sh[k];
    atomicAdd(out, t);
    if (any_bad) out[1] = 1.f;
  }
}

// ----------------------------------------------------------------------------- fills / casts
__global__ void fill_f32_kernel(float* __restrict__ x, float value, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n4 = n >> 2;
  const float4 v4 = make_float4(value, value, value, value);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
    reinterpret_cast<float4*>(x)[i] = v4;
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = value;
}
__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(x[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __bfloat162float(x[i]);
}

// ----------------------------------------------------------------------------- activations
__device__ __forceinline__ float act_apply(float x, int act) {
  return act == INCIN_ACT_GELU ? gelu_erf(x) : (act == INCIN_ACT_SILU ? silu(x) : x);
}
__device__ __forceinline__ float act_grad(float x, int act) {
  return act == INCIN_ACT_GELU ? gelu_erf_grad(x) : (act == INCIN_ACT_SILU ? silu_grad(x) : 1.f);
}
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                               int act) {
  pdl_launch_dependents();
  pdl_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(act_apply(__bfloat162float(x[i]), act));
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ pre,
                               __nv_bfloat16* __restrict__ dx, long long n, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = __float2bfloat16(__bfloat162float(dy[i]) * act_grad(__bfloat162float(pre[i]), act));
}

// gate_up: [rows][2F] with gate = [:, :F], up = [:, F:]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, long long rows,
                                  int F) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = rows * F;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / F;
    const int c = (int)(i - r * F);
    const float g = __bfloat162float(gu[r * 2 * F + c]);
    const float u = __bfloat162float(gu[r * 2 * F + F + c]);
    y[i] = __float2bfloat16(silu(g) * u);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = rows * F;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / F;
    const int c = (int)(i - r * F);
    const float g = __bfloat162float(gu[r * 2 * F + c]);
    const float u = __bfloat162float(gu[r * 2 * F + F + c]);
    const float d = __bfloat162float(dy[i]);
    dgu[r * 2 * F + c] = __float2bfloat16(d * u * silu_grad(g));
    dgu[r * 2 * F + F + c] = __float2bfloat16(d * silu(g));
  }
}

// Rotary embedding, "rotate-half" convention: pairs (i, i + D/2), angle = t * theta^(-2i/D).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, long long B, int T, int H, int D, long long sb,
                            long long st, long long sh, float theta, int inverse) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = D / 2;
  const long long total = B * T * H * half;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int d = (int)(i % half);
    long long r = i / half;
    const int h = (int)(r % H);
    r /= H;
    const int t = (int)(r % T);
    const long long b = r / T;
    __nv_bfloat16* p = x + b * sb + (long long)t * st + (long long)h * sh;
    const float freq = powf(theta, -2.f * d / D);
    float sn, cs;
    sincosf(t * freq, &sn, &cs);
    if (inverse) sn = -sn;
    const float a = __bfloat162float(p[d]), c = __bfloat162float(p[d + half]);
    p[d] = __float2bfloat16(a * cs - c * sn);
    p[d + half] = __float2bfloat16(c * cs + a * sn);
  }
}

// ----------------------------------------------------------------------------- Philox4x32-10
struct Philox {
  uint32_t c[4], k[2];
};
__device__ __forceinline__ void philox_round(Philox& s) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, s.c[0]), lo0 = M0 * s.c[0];
  const uint32_t hi1 = __umulhi(M1, s.c[2]), lo1 = M1 * s.c[2];
  const uint32_t n0 = hi1 ^ s.c[1] ^ s.k[0], n1 = lo1, n2 = hi0 ^ s.c[3] ^ s.k[1], n3 = lo0;
  s.c[0] = n0;
  s.c[1] = n1;
  s.c[2] = n2;
  s.c[3] = n3;
  s.k[0] += 0x9E3779B9u;
  s.k[1] += 0xBB67AE85u;
}
// counter = (index, offset), key = seed: 4 random words per 128-bit counter
__device__ __forceinline__ uint4 philox4x32_10(uint64_t seed, uint64_t ctr_lo, uint64_t ctr_hi) {
  Philox s;
  s.c[0] = (uint32_t)ctr_lo;
  s.c[1] = (uint32_t)(ctr_lo >> 32);
  s.c[2] = (uint32_t)ctr_hi;
  s.c[3] = (uint32_t)(ctr_hi >> 32);
  s.k[0] = (uint32_t)seed;
  s.k[1] = (uint32_t)(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) philox_round(s);
  return make_uint4(s.c[0], s.c[1], s.c[2], s.c[3]);
}
__device__ __forceinline__ float u32_to_unit(uint32_t x) { return ((x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

template <typename OutT, bool NORMAL>
__global__ void philox_kernel(OutT* __restrict__ out, long long n, uint64_t seed, uint64_t offset, float a, float b) {
  const long long n4 = (n + 3) >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const uint4 r = philox4x32_10(seed, (uint64_t)i, offset);
    float f[4] = {u32_to_unit(r.x), u32_to_unit(r.y), u32_to_unit(r.z), u32_to_unit(r.w)};
    if (NORMAL) {  // Box-Muller on pairs
      const float r0 = sqrtf(-2.f * logf(f[0])), r1 = sqrtf(-2.f * logf(f[2]));
      float s0, c0, s1, c1;
      sincospif(2.f * f[1], &s0, &c0);
      sincospif(2.f * f[3], &s1, &c1);
      f[0] = a + b * r0 * c0;
      f[1] = a + b * r0 * s0;
      f[2] = a + b * r1 * c1;
      f[3] = a + b * r1 * s1;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long j = i * 4 + k;
      if (j < n) out[j] = static_cast<OutT>(f[k]);
    }
  }
}

__global__ void dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n,
                               float p, uint64_t seed, uint64_t offset) {
  const long long n4 = (n + 3) >> 2;
  const float inv = 1.f / (1.f - p);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const uint4 r = philox4x32_10(seed, (uint64_t)i, offset);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long j = i * 4 + k;
      if (j < n) y[j] = __float2bfloat16(u32_to_unit(w[k]) >= p ? __bfloat162float(x[j]) * inv : 0.f);
    }
  }
}

}  // namespace incin

using namespace incin;
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH)
#define ST(s) ((cudaStream_t)(s))

extern "C" int incin_adamw_flat(float* master, float* m, float* v, const float* grad, void* shadow, long long n,
                                long long n_decay, const float* hyper, void* stream) {
  if (n <= 0 || !master || !m || !v || !grad || !hyper) return INCIN_ERR_ARGUMENT;
  launch_pdl(adamw_flat_kernel, dim3(grid_for(n, 1024)), dim3(256), 0, ST(stream), master, m, v, grad, (__nv_bfloat16*)shadow, n, n_decay,
                                                               hyper);
  return CHECK_LAUNCH();
}
extern "C" int incin_sgd_flat(float* master, float* mom, const float* grad, void* shadow, long long n,
                              long long n_decay, const float* hyper, void* stream) {
  if (n <= 0 || !master || !grad || !hyper) return INCIN_ERR_ARGUMENT;
  sgd_flat_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(master, mom, grad, (__nv_bfloat16*)shadow, n, n_decay,
                                                            hyper);
  return CHECK_LAUNCH();
}
extern "C" int incin_sumsq_nonfinite_f32(const float* x, long long n, float* out, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  sumsq_nonfinite_kernel<<<grid_for(n, 2048, 148 * 4), 256, 0, ST(stream)>>>(x, n, out);
  return CHECK_LAUNCH();
}
extern "C" int incin_fill_f32(float* x, float value, long long n, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  launch_pdl(fill_f32_kernel, dim3(grid_for(n, 1024)), dim3(256), 0, ST(stream), x, value, n);
  return CHECK_LAUNCH();
}
extern "C" int incin_cast_f32_to_bf16(const float* x, void* y, long long n, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(x, (__nv_bfloat16*)y, n);
  return CHECK_LAUNCH();
}
extern "C" int incin_cast_bf16_to_f32(const void* x, float* y, long long n, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  cast_bf16_f32_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, y, n);
  return CHECK_LAUNCH();
}
extern "C" int incin_act_fwd(const void* x, void* y, long long n, int act, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  launch_pdl(act_fwd_kernel, dim3(grid_for(n, 256)), dim3(256), 0, ST(stream), (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, act);
  return CHECK_LAUNCH();
}
extern "C" int incin_act_bwd(const void* dy, const void* pre, void* dx, long long n, int act, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  launch_pdl(act_bwd_kernel, dim3(grid_for(n, 256)), dim3(256), 0, ST(stream), (const __nv_bfloat16*)dy, (const __nv_bfloat16*)pre,
                                                           (__nv_bfloat16*)dx, n, act);
  return CHECK_LAUNCH();
}
extern "C" int incin_swiglu_fwd(const void* gate_up, void* y, long long rows, int F, void* stream) {
  if (rows <= 0 || F <= 0) return INCIN_ERR_ARGUMENT;
  launch_pdl(swiglu_fwd_kernel, dim3(grid_for(rows * F, 256)), dim3(256), 0, ST(stream), (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)y,
                                                                     rows, F);
  return CHECK_LAUNCH();
}
extern "C" int incin_swiglu_bwd(const void* dy, const void* gate_up, void* dgate_up, long long rows, int F,
                                void* stream) {
  if (rows <= 0 || F <= 0) return INCIN_ERR_ARGUMENT;
  launch_pdl(swiglu_bwd_kernel, dim3(grid_for(rows * F, 256)), dim3(256), 0, ST(stream), 
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)dgate_up, rows, F);
  return CHECK_LAUNCH();
}
extern "C" int incin_rope(void* x, long long B, int T, int H, int D, long long stride_b, long long stride_t,
                          long long stride_h, float theta, int inverse, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0 || (D & 1)) return INCIN_ERR_ARGUMENT;
  launch_pdl(rope_kernel, dim3(grid_for(B * T * H * (D / 2), 256)), dim3(256), 0, ST(stream), (__nv_bfloat16*)x, B, T, H, D, stride_b,
                                                                          stride_t, stride_h, theta, inverse);
  return CHECK_LAUNCH();
}
extern "C" int incin_philox_uniform_f32(float* out, long long n, uint64_t seed, uint64_t offset, void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  philox_kernel<float, false><<<grid_for((n + 3) / 4, 256), 256, 0, ST(stream)>>>(out, n, seed, offset, 0.f, 1.f);
  return CHECK_LAUNCH();
}
extern "C" int incin_philox_normal_f32(float* out, long long n, uint64_t seed, uint64_t offset, float mean, float std,
                                       void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  philox_kernel<float, true><<<grid_for((n + 3) / 4, 256), 256, 0, ST(stream)>>>(out, n, seed, offset, mean, std);
  return CHECK_LAUNCH();
}
extern "C" int incin_philox_normal_bf16(void* out, long long n, uint64_t seed, uint64_t offset, float mean, float std,
                                        void* stream) {
  if (n <= 0) return INCIN_ERR_ARGUMENT;
  philox_kernel<__nv_bfloat16, true>
      <<<grid_for((n + 3) / 4, 256), 256, 0, ST(stream)>>>((__nv_bfloat16*)out, n, seed, offset, mean, std);
  return CHECK_LAUNCH();
}
extern "C" int incin_dropout_bf16(const void* x, void* y, long long n, float p, uint64_t seed, uint64_t offset,
                                  void* stream) {
  if (n <= 0 || p < 0.f || p >= 1.f) return INCIN_ERR_ARGUMENT;
  dropout_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, ST(stream)>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, p,
                                                                     seed, offset);
  return CHECK_LAUNCH();
}
extern "C" const char* incin_sm100_version(void) { return "incin_b200 sm_100a kernels 0.1"; }
namespace incin { int device_sm_count(); }
extern "C" int incin_sm100_num_sms(void) { return incin::device_sm_count(); }
