// Reductions for sm_100a: sum / mean / max / min / prod / argmax / argmin over one axis of a dense tensor viewed
// as [outer, reduce, inner], a deterministic single-launch reduction of a whole tensor, and cumulative sums.
//
// Counterpart of the reference's `incin_reduce_*` row kernels (crates/incin-backends/src/kernel.rs:1054-1184: one
// block per row, or one THREAD per output with a serial loop for strided axes) and of its whole-tensor reductions,
// which the reference composes from repeated row reductions.  Here:
//   * inner == 1   one warp (short rows) or one block (long rows) per row, 128-bit loads, shuffle tree;
//   * inner  > 1   threads run along `inner` (coalesced), a block's y dimension splits `reduce`, shared-memory
//                  combine - no serial one-thread loop;
//   * whole tensor one launch: every block reduces a grid-stride slice, the last block to finish (ticket counter)
//                  combines the partials in a fixed order, so the result is bitwise reproducible.
// bf16 and fp32 inputs; accumulation is always fp32; outputs keep the input dtype (indices are int64).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cfloat>

#include "incin_b200.h"

namespace {

enum { OP_SUM = 0, OP_MEAN = 1, OP_MAX = 2, OP_MIN = 3, OP_PROD = 4, OP_ARGMAX = 5, OP_ARGMIN = 6 };

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

struct Acc {
  float v;
  long long i;
};

__device__ __forceinline__ Acc identity(int op) {
  Acc a;
  a.i = 0x7fffffffffffffffLL;
  a.v = (op == OP_MAX || op == OP_ARGMAX) ? -INFINITY : (op == OP_MIN || op == OP_ARGMIN) ? INFINITY : (op == OP_PROD ? 1.0f : 0.0f);
  return a;
}

// NaN propagates through max/min like the CPU oracle (a NaN wins); ties in arg* keep the lowest index.
__device__ __forceinline__ Acc combine(Acc a, Acc b, int op) {
  switch (op) {
    case OP_SUM:
    case OP_MEAN: a.v += b.v; return a;
    case OP_PROD: a.v *= b.v; return a;
    case OP_MAX: a.v = (b.v > a.v || b.v != b.v) ? b.v : a.v; return a;
    case OP_MIN: a.v = (b.v < a.v || b.v != b.v) ? b.v : a.v; return a;
    case OP_ARGMAX: {
      const bool a_nan = a.v != a.v, b_nan = b.v != b.v;
      const bool take = (b_nan && (!a_nan || b.i < a.i)) || (!a_nan && !b_nan && (b.v > a.v || (b.v == a.v && b.i < a.i)));
      return take ? b : a;
    }
    default: {
      const bool a_nan = a.v != a.v, b_nan = b.v != b.v;
      const bool take = (b_nan && (!a_nan || b.i < a.i)) || (!a_nan && !b_nan && (b.v < a.v || (b.v == a.v && b.i < a.i)));
      return take ? b : a;
    }
  }
}

__device__ __forceinline__ Acc warp_reduce(Acc a, int op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Acc b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = combine(a, b, op);
  }
  return a;
}

template <typename T>
__device__ __forceinline__ void finish(Acc a, int op, long long reduce, T* out, long long* idx, long long o) {
  if (op == OP_ARGMAX || op == OP_ARGMIN) {
    idx[o] = a.i;
  } else {
    stf(out, o, op == OP_MEAN ? a.v / (float)reduce : a.v);
  }
}

// ---- inner == 1, one warp per row ------------------------------------------------------------------------------
template <typename T>
__global__ void reduce_rows_warp(const T* __restrict__ x, T* __restrict__ out, long long* __restrict__ idx, long long rows,
                                 long long n, int op) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* p = x + row * n;
  Acc a = identity(op);
  for (long long i = lane; i < n; i += 32) {
    Acc b;
    b.v = ldf(p, i);
    b.i = i;
    a = combine(a, b, op);
  }
  a = warp_reduce(a, op);
  if (lane == 0) finish(a, op, n, out, idx, row);
}

// ---- inner == 1, one block per row (long rows): 128-bit loads --------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) reduce_rows_block(const T* __restrict__ x, T* __restrict__ out, long long* __restrict__ idx,
                                                         long long n, int op) {
  constexpr int VEC = 16 / sizeof(T);
  const long long row = blockIdx.x;
  const T* p = x + row * n;
  Acc a = identity(op);
  const bool aligned = (reinterpret_cast<uintptr_t>(p) & 15) == 0;
  long long done = 0;
  if (aligned) {
    const long long nv = n / VEC;
    for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 raw = reinterpret_cast<const uint4*>(p)[i];
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        Acc b;
        b.v = ldf(e, k);
        b.i = i * VEC + k;
        a = combine(a, b, op);
      }
    }
    done = nv * VEC;
  }
  for (long long i = done + threadIdx.x; i < n; i += blockDim.x) {
    Acc b;
    b.v = ldf(p, i);
    b.i = i;
    a = combine(a, b, op);
  }
  __shared__ float sv[8];
  __shared__ long long si[8];
  a = warp_reduce(a, op);
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = a.v;
    si[threadIdx.x >> 5] = a.i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    Acc r;
    r.v = sv[0];
    r.i = si[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
      Acc b;
      b.v = sv[w];
      b.i = si[w];
      r = combine(r, b, op);
    }
    finish(r, op, n, out, idx, row);
  }
}

// ---- inner > 1: threads along inner, blockDim.y splits the reduced axis ---------------------------------------
template <typename T>
__global__ void reduce_mid(const T* __restrict__ x, T* __restrict__ out, long long* __restrict__ idx, long long outer,
                           long long reduce, long long inner, int op) {
  const long long in = (long long)blockIdx.x * 32 + threadIdx.x;
  __shared__ float sv[8][33];
  __shared__ long long si[8][33];
  for (long long o = blockIdx.y; o < outer; o += gridDim.y) {
    Acc a = identity(op);
    if (in < inner) {
      const T* p = x + o * reduce * inner + in;
      for (long long r = threadIdx.y; r < reduce; r += blockDim.y) {
        Acc b;
        b.v = ldf(p, r * inner);
        b.i = r;
        a = combine(a, b, op);
      }
    }
    sv[threadIdx.y][threadIdx.x] = a.v;
    si[threadIdx.y][threadIdx.x] = a.i;
    __syncthreads();
    if (threadIdx.y == 0 && in < inner) {
      for (int y = 1; y < (int)blockDim.y; ++y) {
        Acc b;
        b.v = sv[y][threadIdx.x];
        b.i = si[y][threadIdx.x];
        a = combine(a, b, op);
      }
      finish(a, op, reduce, out, idx, o * inner + in);
    }
    __syncthreads();
  }
}

// ---- whole tensor, one launch, deterministic ------------------------------------------------------------------
constexpr int ALL_BLOCKS = 592;   // 4 per SM on 148 SMs
__device__ float g_partial_v[ALL_BLOCKS];
__device__ long long g_partial_i[ALL_BLOCKS];
__device__ unsigned int g_ticket;

template <typename T>
__global__ void __launch_bounds__(256) reduce_all_kernel(const T* __restrict__ x, float* __restrict__ out, long long* __restrict__ idx,
                                                         long long n, int op) {
  constexpr int VEC = 16 / sizeof(T);
  Acc a = identity(op);
  const long long nv = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? n / VEC : 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      Acc b;
      b.v = ldf(e, k);
      b.i = i * VEC + k;
      a = combine(a, b, op);
    }
  }
  for (long long i = nv * VEC + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    Acc b;
    b.v = ldf(x, i);
    b.i = i;
    a = combine(a, b, op);
  }
  __shared__ float sv[8];
  __shared__ long long si[8];
  __shared__ bool last;
  a = warp_reduce(a, op);
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = a.v;
    si[threadIdx.x >> 5] = a.i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    Acc r;
    r.v = sv[0];
    r.i = si[0];
    for (int w = 1; w < 8; ++w) {
      Acc b;
      b.v = sv[w];
      b.i = si[w];
      r = combine(r, b, op);
    }
    g_partial_v[blockIdx.x] = r.v;
    g_partial_i[blockIdx.x] = r.i;
    __threadfence();
    last = atomicAdd(&g_ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    Acc r = identity(op);
    for (int b = 0; b < (int)gridDim.x; ++b) {   // fixed order: the result does not depend on block scheduling
      Acc q;
      q.v = g_partial_v[b];
      q.i = g_partial_i[b];
      r = combine(r, q, op);
    }
    if (op == OP_ARGMAX || op == OP_ARGMIN) idx[0] = r.i;
    else out[0] = op == OP_MEAN ? r.v / (float)n : r.v;
    g_ticket = 0;   // ready for the next launch on this stream
  }
}

// ---- cumulative sum ---------------------------------------------------------------------------------------------
// inner == 1: one block per row walks the row in tiles of 1024 with a running carry (warp scan + block scan).
template <typename T>
__global__ void __launch_bounds__(1024) cumsum_rows(const T* __restrict__ x, T* __restrict__ out, long long n) {
  const T* p = x + (long long)blockIdx.x * n;
  T* q = out + (long long)blockIdx.x * n;
  __shared__ float warp_tot[32];
  __shared__ float carry_s;
  if (threadIdx.x == 0) carry_s = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long base = 0; base < n; base += 1024) {
    const long long i = base + threadIdx.x;
    float v = i < n ? ldf(p, i) : 0.0f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += t;
    }
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
      float t = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, t, o);
        if (lane >= o) t += u;
      }
      warp_tot[lane] = t;   // inclusive totals
    }
    __syncthreads();
    const float carry = carry_s;
    const float prefix = warp > 0 ? warp_tot[warp - 1] : 0.0f;
    if (i < n) stf(q, i, v + prefix + carry);
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + warp_tot[31];
    __syncthreads();
  }
}

// inner > 1: one thread per (outer, inner) column, coalesced across inner.
template <typename T>
__global__ void cumsum_mid(const T* __restrict__ x, T* __restrict__ out, long long outer, long long n, long long inner) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= outer * inner) return;
  const long long o = t / inner, in = t % inner;
  const T* p = x + o * n * inner + in;
  T* q = out + o * n * inner + in;
  float acc = 0.0f;
  for (long long r = 0; r < n; ++r) {
    acc += ldf(p, r * inner);
    stf(q, r * inner, acc);
  }
}

template <typename T>
int launch_reduce(const void* x_, void* out_, long long* idx, long long outer, long long reduce, long long inner, int op,
                  cudaStream_t s) {
  const T* x = static_cast<const T*>(x_);
  T* out = static_cast<T*>(out_);
  if (inner == 1) {
    if (reduce <= 2048) {
      const int warps = 8;
      reduce_rows_warp<T><<<(unsigned)((outer + warps - 1) / warps), warps * 32, 0, s>>>(x, out, idx, outer, reduce, op);
    } else {
      reduce_rows_block<T><<<(unsigned)outer, 256, 0, s>>>(x, out, idx, reduce, op);
    }
  } else {
    dim3 grid((unsigned)((inner + 31) / 32), (unsigned)(outer > 65535 ? 65535 : outer)), block(32, 8);
    reduce_mid<T><<<grid, block, 0, s>>>(x, out, idx, outer, reduce, inner, op);
  }
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace

extern "C" int incin_reduce_axis(const void* x, void* out, long long* idx_out, long long outer, long long reduce,
                                 long long inner, int op, int is_bf16, void* stream) {
  if (!x || outer <= 0 || reduce <= 0 || inner <= 0 || op < 0 || op > OP_ARGMIN) return INCIN_ERR_ARGUMENT;
  const bool arg = op == OP_ARGMAX || op == OP_ARGMIN;
  if ((arg && !idx_out) || (!arg && !out)) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return is_bf16 ? launch_reduce<__nv_bfloat16>(x, out, idx_out, outer, reduce, inner, op, s)
                 : launch_reduce<float>(x, out, idx_out, outer, reduce, inner, op, s);
}

extern "C" int incin_reduce_all(const void* x, float* out, long long* idx_out, long long n, int op, int is_bf16,
                                void* stream) {
  if (!x || n <= 0 || op < 0 || op > OP_ARGMIN) return INCIN_ERR_ARGUMENT;
  const bool arg = op == OP_ARGMAX || op == OP_ARGMIN;
  if ((arg && !idx_out) || (!arg && !out)) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  long long want = (n + 256 * 8 - 1) / (256 * 8);
  const int blocks = (int)(want < 1 ? 1 : (want > ALL_BLOCKS ? ALL_BLOCKS : want));
  if (is_bf16) reduce_all_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), out, idx_out, n, op);
  else reduce_all_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), out, idx_out, n, op);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_cumsum(const void* x, void* out, long long outer, long long n, long long inner, int is_bf16,
                            void* stream) {
  if (!x || !out || outer <= 0 || n <= 0 || inner <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (inner == 1) {
    if (is_bf16) cumsum_rows<__nv_bfloat16><<<(unsigned)outer, 1024, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n);
    else cumsum_rows<float><<<(unsigned)outer, 1024, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(out), n);
  } else {
    const long long t = outer * inner;
    if (is_bf16) cumsum_mid<__nv_bfloat16><<<(unsigned)((t + 127) / 128), 128, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), outer, n, inner);
    else cumsum_mid<float><<<(unsigned)((t + 127) / 128), 128, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(out), outer, n, inner);
  }
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}
