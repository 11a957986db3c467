// CPU oracle: plain, readable fp32 implementations of every op the sm_100a
// kernels provide, behind a C ABI.  It is the correctness reference for the
// CUDA tests and the compute engine of the CPU backend for small models.
//
// Semantics follow the reference's CPU backend, which is its contract:
//   matmul            crates/incin-backends/src/cpu/ops/matmul.rs:316-493
//   softmax/CE        crates/incin-backends/src/cpu/ops/loss.rs:35-92 (log_softmax * one_hot)
//   AdamW             crates/incin-backends/src/cpu/ops/optimizer.rs:43-59 (bias corrected, decoupled decay)
//   SDPA              crates/incin-backends/src/cpu/ops/shape_ops.rs:1245-1269 (softmax(QK^T s + mask) V)
//   Q8_0              crates/incin-core/src/tensor/dtype.rs:131-194 (34 bytes per 32 elements)
// plus CPU restatements of arithmetic that only exists in the reference's
// WGSL/MSL shaders (tanh-approximate GELU: wgpu/shaders/unary.wgsl:14-19).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {
inline float gelu_erf(float x) { return 0.5f * x * (1.0f + std::erf(x * 0.70710678118654752f)); }
inline float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.0f + std::tanh(k * (x + 0.044715f * x * x * x)));
}
inline float silu(float x) { return x / (1.0f + std::exp(-x)); }

// IEEE half <-> float (round to nearest even), used by Q8_0 scales
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return (uint16_t)(sign | h);
}
inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, x;
  if (exp == 0) {
    if (man == 0) {
      x = sign;
    } else {
      exp = 127 - 15 + 1;
      while (!(man & 0x400u)) {
        man <<= 1;
        --exp;
      }
      x = sign | (exp << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7f800000u | (man << 13);
  } else {
    x = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}
}  // namespace

// C[b] (M x N) = alpha * op(A[b]) * op(B[b]) + beta * C[b]; generic strides in elements.
API void incin_cpu_gemm_f32(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N, int64_t K,
                            int64_t a_bs, int64_t a_rs, int64_t a_cs, int64_t b_bs, int64_t b_rs, int64_t b_cs,
                            int64_t c_bs, int64_t c_rs, float alpha, float beta) {
  for (int64_t b = 0; b < batch; ++b) {
    const float* a = A + b * a_bs;
    const float* bb = B + b * b_bs;
    float* c = C + b * c_bs;
    for (int64_t i = 0; i < M; ++i) {
      std::vector<double> acc((size_t)N, 0.0);
      for (int64_t k = 0; k < K; ++k) {
        const double av = a[i * a_rs + k * a_cs];
        const float* brow = bb + k * b_rs;
        for (int64_t j = 0; j < N; ++j) acc[(size_t)j] += av * brow[j * b_cs];
      }
      for (int64_t j = 0; j < N; ++j)
        c[i * c_rs + j] = alpha * (float)acc[(size_t)j] + (beta != 0.f ? beta * c[i * c_rs + j] : 0.f);
    }
  }
}

API void incin_cpu_unary_f32(const float* x, float* y, int64_t n, int op) {
  for (int64_t i = 0; i < n; ++i) {
    const float v = x[i];
    float r;
    switch (op) {
      case 0: r = v > 0 ? v : 0; break;                       // relu
      case 1: r = gelu_erf(v); break;                          // gelu (exact, CPU/CUDA contract)
      case 2: r = gelu_tanh(v); break;                         // gelu (tanh approximation, WGSL restatement)
      case 3: r = silu(v); break;                              // swish
      case 4: r = 1.0f / (1.0f + std::exp(-v)); break;         // sigmoid
      case 5: r = std::tanh(v); break;
      case 6: r = std::exp(v); break;
      case 7: r = std::log(v); break;
      case 8: r = std::sqrt(v); break;
      case 9: r = -v; break;
      case 10: r = std::fabs(v); break;
      case 11: r = v * std::tanh(std::log1p(std::exp(v))); break;  // mish
      case 12: r = v > 0 ? v : std::expm1(v); break;               // elu(alpha=1)
      case 13: r = std::log1p(std::exp(v)); break;                 // softplus
      case 14: r = (v > 0) - (v < 0); break;                       // sign
      default: r = v;
    }
    y[i] = r;
  }
}

API void incin_cpu_softmax_f32(const float* x, float* y, int64_t rows, int64_t C, int log_softmax) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * C;
    float* yr = y + r * C;
    float m = -std::numeric_limits<float>::infinity();
    for (int64_t c = 0; c < C; ++c) m = std::max(m, xr[c]);
    double s = 0;
    for (int64_t c = 0; c < C; ++c) s += std::exp((double)xr[c] - m);
    const double ls = std::log(s);
    for (int64_t c = 0; c < C; ++c)
      yr[c] = log_softmax ? (float)((double)xr[c] - m - ls) : (float)(std::exp((double)xr[c] - m) / s);
  }
}

API void incin_cpu_layernorm_f32(const float* x, const float* g, const float* b, float* y, int64_t rows, int64_t C,
                                 float eps, int rms) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * C;
    double mean = 0;
    if (!rms) {
      for (int64_t c = 0; c < C; ++c) mean += xr[c];
      mean /= C;
    }
    double var = 0;
    for (int64_t c = 0; c < C; ++c) var += (xr[c] - mean) * (xr[c] - mean);
    const double rstd = 1.0 / std::sqrt(var / C + eps);
    for (int64_t c = 0; c < C; ++c)
      y[r * C + c] = (float)((xr[c] - mean) * rstd) * (g ? g[c] : 1.f) + (b ? b[c] : 0.f);
  }
}

// mean softmax cross-entropy; dlogits (optional) = (softmax - onehot) / rows
API float incin_cpu_cross_entropy_f32(const float* logits, const int64_t* targets, float* dlogits, int64_t rows,
                                      int64_t V) {
  double total = 0;
  for (int64_t r = 0; r < rows; ++r) {
    const float* lr = logits + r * V;
    float m = -std::numeric_limits<float>::infinity();
    for (int64_t c = 0; c < V; ++c) m = std::max(m, lr[c]);
    double s = 0;
    for (int64_t c = 0; c < V; ++c) s += std::exp((double)lr[c] - m);
    const double lse = m + std::log(s);
    total += lse - lr[targets[r]];
    if (dlogits)
      for (int64_t c = 0; c < V; ++c)
        dlogits[r * V + c] = (float)((std::exp((double)lr[c] - lse) - (c == targets[r] ? 1.0 : 0.0)) / rows);
  }
  return (float)(total / rows);
}

API void incin_cpu_sgd_f32(float* w, const float* g, int64_t n, float lr) {
  for (int64_t i = 0; i < n; ++i) w[i] -= lr * g[i];
}

API void incin_cpu_adamw_f32(float* w, float* m, float* v, const float* g, int64_t n, float lr, float b1, float b2,
                             float eps, float wd, int step) {
  const float bc1 = 1.f - std::pow(b1, (float)step), bc2 = 1.f - std::pow(b2, (float)step);
  for (int64_t i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + (1.f - b1) * g[i];
    v[i] = b2 * v[i] + (1.f - b2) * g[i] * g[i];
    const float mh = m[i] / bc1, vh = v[i] / bc2;
    w[i] = w[i] - lr * wd * w[i] - lr * mh / (std::sqrt(vh) + eps);
  }
}

// Causal (or full) attention for one [T, D] head: o = softmax(q k^T * scale + mask) v, fp64 accumulation.
API void incin_cpu_attention_f32(const float* q, const float* k, const float* v, float* o, int64_t heads, int64_t T,
                                 int64_t D, float scale, int causal) {
  std::vector<double> p((size_t)T);
  for (int64_t h = 0; h < heads; ++h) {
    const float *qh = q + h * T * D, *kh = k + h * T * D, *vh = v + h * T * D;
    float* oh = o + h * T * D;
    for (int64_t i = 0; i < T; ++i) {
      const int64_t n = causal ? i + 1 : T;
      double m = -1e300;
      for (int64_t j = 0; j < n; ++j) {
        double s = 0;
        for (int64_t d = 0; d < D; ++d) s += (double)qh[i * D + d] * kh[j * D + d];
        p[(size_t)j] = s * scale;
        m = std::max(m, p[(size_t)j]);
      }
      double sum = 0;
      for (int64_t j = 0; j < n; ++j) {
        p[(size_t)j] = std::exp(p[(size_t)j] - m);
        sum += p[(size_t)j];
      }
      for (int64_t d = 0; d < D; ++d) {
        double acc = 0;
        for (int64_t j = 0; j < n; ++j) acc += p[(size_t)j] * vh[j * D + d];
        oh[i * D + d] = (float)(acc / sum);
      }
    }
  }
}

// ---- Q8_0: blocks of 32 values = f16 scale + 32 int8 (34 bytes) ---------------------------------
API int64_t incin_cpu_q8_0_bytes(int64_t n) { return (n + 31) / 32 * 34; }
API void incin_cpu_quantize_q8_0(const float* x, uint8_t* out, int64_t n) {
  const int64_t blocks = (n + 31) / 32;
  for (int64_t b = 0; b < blocks; ++b) {
    float amax = 0;
    for (int64_t i = 0; i < 32 && b * 32 + i < n; ++i) amax = std::max(amax, std::fabs(x[b * 32 + i]));
    const float d = amax / 127.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    const uint16_t dh = f32_to_f16(d);
    std::memcpy(out + b * 34, &dh, 2);
    for (int64_t i = 0; i < 32; ++i) {
      const float v = (b * 32 + i < n) ? x[b * 32 + i] * id : 0.f;
      out[b * 34 + 2 + i] = (uint8_t)(int8_t)std::lround(v);
    }
  }
}
API void incin_cpu_dequantize_q8_0(const uint8_t* in, float* y, int64_t n) {
  const int64_t blocks = (n + 31) / 32;
  for (int64_t b = 0; b < blocks; ++b) {
    uint16_t dh;
    std::memcpy(&dh, in + b * 34, 2);
    const float d = f16_to_f32(dh);
    for (int64_t i = 0; i < 32 && b * 32 + i < n; ++i) y[b * 32 + i] = d * (float)(int8_t)in[b * 34 + 2 + i];
  }
}

// ---- Philox4x32-10: bit-identical to the device generator -----------------------------------------
namespace {
inline void philox(uint64_t seed, uint64_t lo, uint64_t hi, uint32_t out[4]) {
  uint32_t c[4] = {(uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32)};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1,
                   n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  std::memcpy(out, c, 16);
}
inline float unit(uint32_t x) { return ((x >> 8) + 0.5f) * (1.0f / 16777216.0f); }
}  // namespace

API void incin_cpu_philox_uniform_f32(float* out, int64_t n, uint64_t seed, uint64_t offset) {
  for (int64_t i = 0; i < (n + 3) / 4; ++i) {
    uint32_t r[4];
    philox(seed, (uint64_t)i, offset, r);
    for (int k = 0; k < 4 && i * 4 + k < n; ++k) out[i * 4 + k] = unit(r[k]);
  }
}
API void incin_cpu_philox_normal_f32(float* out, int64_t n, uint64_t seed, uint64_t offset, float mean, float std_) {
  const double two_pi = 6.283185307179586;
  for (int64_t i = 0; i < (n + 3) / 4; ++i) {
    uint32_t r[4];
    philox(seed, (uint64_t)i, offset, r);
    const float f[4] = {unit(r[0]), unit(r[1]), unit(r[2]), unit(r[3])};
    const float r0 = std::sqrt(-2.f * std::log(f[0])), r1 = std::sqrt(-2.f * std::log(f[2]));
    const float v[4] = {mean + std_ * r0 * (float)std::cos(two_pi * f[1]), mean + std_ * r0 * (float)std::sin(two_pi * f[1]),
                        mean + std_ * r1 * (float)std::cos(two_pi * f[3]), mean + std_ * r1 * (float)std::sin(two_pi * f[3])};
    for (int k = 0; k < 4 && i * 4 + k < n; ++k) out[i * 4 + k] = v[k];
  }
}
