// Deterministic in-process reference transport: every collective takes ALL ranks' buffers in one call
// and produces all ranks' outputs with plain host arithmetic.  It is the oracle the fused peer-memory
// kernels and the NCCL path are checked against, and what the CPU-only tests of the DP/TP/PP logic run on.
//
// Same contract as the reference's ReferenceTransport (crates/incin-backends/src/dist/reference.rs:164-681):
// f16/bf16 reduce through f32, integer reductions are overflow-checked, reduce order is rank 0..n-1.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {
enum DType : int { F32 = 0, F64 = 1, F16 = 2, BF16 = 3, I64 = 4, U32 = 5, U8 = 6 };
enum Op : int { SUM = 0, MEAN = 1, MAX = 2, MIN = 3, PROD = 4 };
enum Err : int { OK = 0, E_ARG = 1, E_OVERFLOW = 2, E_DTYPE = 3 };

int elem_size(int dt) {
  switch (dt) {
    case F32: case U32: return 4;
    case F64: case I64: return 8;
    case F16: case BF16: return 2;
    case U8: return 1;
  }
  return 0;
}
float bf16_to_f32(uint16_t h) {
  uint32_t x = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}
uint16_t f32_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);  // quiet NaN
  x += 0x7fffu + ((x >> 16) & 1);
  return (uint16_t)(x >> 16);
}
float f16_to_f32(uint16_t h) {
  const uint32_t s = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ffu, x;
  if (e == 0) {
    if (!m) x = s;
    else {
      e = 113;
      while (!(m & 0x400u)) { m <<= 1; --e; }
      x = s | (e << 23) | ((m & 0x3ffu) << 13);
    }
  } else if (e == 31) x = s | 0x7f800000u | (m << 13);
  else x = s | ((e + 112) << 23) | (m << 13);
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}
uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t s = (x >> 16) & 0x8000u;
  const int32_t e = (int32_t)((x >> 23) & 0xff) - 112;
  uint32_t m = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0));
  if (e >= 31) return (uint16_t)(s | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)s;
    m |= 0x800000u;
    const int sh = 14 - e;
    uint32_t h = m >> sh;
    const uint32_t rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return (uint16_t)(s | h);
  }
  uint32_t h = ((uint32_t)e << 10) | (m >> 13);
  const uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return (uint16_t)(s | h);
}

template <typename T>
double combine_f(double a, T b, int op) {
  switch (op) {
    case SUM: case MEAN: return a + (double)b;
    case MAX: return a > (double)b ? a : (double)b;
    case MIN: return a < (double)b ? a : (double)b;
    default: return a * (double)b;
  }
}

// reduce element i over ranks for floating types held as float/double/half formats
int reduce_float(const void* const* in, int world, int64_t i, int dt, int op, void* out_elem) {
  double acc = 0;
  for (int r = 0; r < world; ++r) {
    double v;
    switch (dt) {
      case F32: v = ((const float*)in[r])[i]; break;
      case F64: v = ((const double*)in[r])[i]; break;
      case F16: v = f16_to_f32(((const uint16_t*)in[r])[i]); break;
      default: v = bf16_to_f32(((const uint16_t*)in[r])[i]); break;
    }
    acc = r == 0 ? v : combine_f<double>(acc, v, op);
  }
  if (op == MEAN) acc /= world;
  switch (dt) {
    case F32: *(float*)out_elem = (float)acc; break;
    case F64: *(double*)out_elem = acc; break;
    case F16: *(uint16_t*)out_elem = f32_to_f16((float)acc); break;
    default: *(uint16_t*)out_elem = f32_to_bf16((float)acc); break;
  }
  return OK;
}

int reduce_int(const void* const* in, int world, int64_t i, int dt, int op, void* out_elem) {
  if (op == MEAN) return E_DTYPE;  // a mean of integers is not an integer
  __int128 acc = 0;
  __int128 lo, hi;
  if (dt == I64) { lo = std::numeric_limits<int64_t>::min(); hi = std::numeric_limits<int64_t>::max(); }
  else if (dt == U32) { lo = 0; hi = std::numeric_limits<uint32_t>::max(); }
  else { lo = 0; hi = 255; }
  for (int r = 0; r < world; ++r) {
    __int128 v = dt == I64 ? (__int128)((const int64_t*)in[r])[i]
                           : dt == U32 ? (__int128)((const uint32_t*)in[r])[i] : (__int128)((const uint8_t*)in[r])[i];
    if (r == 0) acc = v;
    else if (op == SUM) acc += v;
    else if (op == PROD) acc *= v;
    else if (op == MAX) acc = acc > v ? acc : v;
    else acc = acc < v ? acc : v;
    if (acc < lo || acc > hi) return E_OVERFLOW;  // checked, never wraps silently
  }
  if (dt == I64) *(int64_t*)out_elem = (int64_t)acc;
  else if (dt == U32) *(uint32_t*)out_elem = (uint32_t)acc;
  else *(uint8_t*)out_elem = (uint8_t)acc;
  return OK;
}

int reduce_elem(const void* const* in, int world, int64_t i, int dt, int op, void* out_elem) {
  return (dt == I64 || dt == U32 || dt == U8) ? reduce_int(in, world, i, dt, op, out_elem)
                                              : reduce_float(in, world, i, dt, op, out_elem);
}
}  // namespace

// out[r][i] = reduce over ranks of in[*][i], for every rank r
API int incin_ref_all_reduce(const void* const* in, void* const* out, int world, int64_t n, int dtype, int op) {
  const int es = elem_size(dtype);
  if (!es || world < 1 || n < 0) return E_ARG;
  std::vector<uint8_t> tmp((size_t)(n * es));
  for (int64_t i = 0; i < n; ++i) {
    const int rc = reduce_elem(in, world, i, dtype, op, tmp.data() + i * es);
    if (rc) return rc;
  }
  for (int r = 0; r < world; ++r) std::memcpy(out[r], tmp.data(), tmp.size());
  return OK;
}

// out[r] = concat over ranks of in[rank] (rank-major), n elements per rank
API int incin_ref_all_gather(const void* const* in, void* const* out, int world, int64_t n, int dtype) {
  const int es = elem_size(dtype);
  if (!es || world < 1 || n < 0) return E_ARG;
  for (int r = 0; r < world; ++r)
    for (int s = 0; s < world; ++s) std::memcpy((uint8_t*)out[r] + (size_t)s * n * es, in[s], (size_t)(n * es));
  return OK;
}

// out[r] = reduce over ranks of chunk r; n elements per rank in, n / world out
API int incin_ref_reduce_scatter(const void* const* in, void* const* out, int world, int64_t n, int dtype, int op) {
  const int es = elem_size(dtype);
  if (!es || world < 1 || n < 0 || n % world) return E_ARG;
  const int64_t c = n / world;
  for (int r = 0; r < world; ++r)
    for (int64_t i = 0; i < c; ++i) {
      const int rc = reduce_elem(in, world, r * c + i, dtype, op, (uint8_t*)out[r] + i * es);
      if (rc) return rc;
    }
  return OK;
}

// out[r] chunk s = in[s] chunk r
API int incin_ref_all_to_all(const void* const* in, void* const* out, int world, int64_t n, int dtype) {
  const int es = elem_size(dtype);
  if (!es || world < 1 || n < 0 || n % world) return E_ARG;
  const size_t cb = (size_t)(n / world) * es;
  for (int r = 0; r < world; ++r)
    for (int s = 0; s < world; ++s) std::memcpy((uint8_t*)out[r] + s * cb, (const uint8_t*)in[s] + r * cb, cb);
  return OK;
}

// out[dst] = in[src]; every other rank's output is left untouched
API int incin_ref_send_recv(const void* const* in, void* const* out, int world, int64_t n, int dtype, int src,
                            int dst) {
  const int es = elem_size(dtype);
  if (!es || src < 0 || dst < 0 || src >= world || dst >= world || src == dst) return E_ARG;
  std::memcpy(out[dst], in[src], (size_t)(n * es));
  return OK;
}
