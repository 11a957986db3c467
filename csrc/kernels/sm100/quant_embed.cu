// Q8_0 block quantisation on the device, and the deterministic embedding backward.
//
// Q8_0 (GGUF layout): 32 values share one fp16 scale d = max|x| / 127, stored as {fp16 d; int8 q[32]} = 34 bytes.
// Counterpart of crates/incin-backends/src/cuda/ops/kernels/quant.cu:13-58 (one thread per block, serial loops).
// Here a warp handles one block per step (lane = element): the max is a shuffle tree and the 34-byte record is
// written by the lanes that own its bytes.  `incin_dequantize_q8_0` with bf16 output produces the bf16 operand of the tcgen05
// GEMM, which is how a quantised matmul runs: dequantise the weight once into bf16, then the tensor-core GEMM.
//
// Embedding backward, deterministic mode: the reference scatters with float atomicAdd
// (crates/incin-backends/src/cuda/ops/kernels/embedding.cu:5-81), whose sum order changes from run to run.  Given
// the token positions sorted by token id, one block per distinct token adds its rows in position order, so the
// gradient is bitwise reproducible and needs no atomics.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "incin_b200.h"

namespace {

constexpr int QK = 32, QBYTES = 34;

template <typename T>
__global__ void quantize_q8_0_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, long long n, long long n_blocks) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long b = warp; b < n_blocks; b += n_warps) {
    const long long i = b * QK + lane;
    float v = 0.0f;
    if (i < n) {
      if constexpr (sizeof(T) == 2) v = __bfloat162float(x[i]);
      else v = x[i];
    }
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);   // exact division: the record must match the CPU oracle bit for bit
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    const int q = (int)roundf(__fmul_rn(v, id));
    uint8_t* rec = out + b * QBYTES;
    rec[2 + lane] = (uint8_t)(int8_t)q;
    const unsigned bits = __half_as_ushort(__float2half_rn(d));   // every lane holds the same scale
    if (lane < 2) rec[lane] = (uint8_t)((bits >> (8 * lane)) & 0xffu);
  }
}

template <typename T>
__global__ void dequantize_q8_0_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const uint8_t* rec = in + (i / QK) * QBYTES;
    const unsigned short bits = (unsigned short)((unsigned)rec[0] | ((unsigned)rec[1] << 8));
    const float d = __half2float(__ushort_as_half(bits));
    const float v = d * (float)(int8_t)rec[2 + (i % QK)];
    if constexpr (sizeof(T) == 2) out[i] = __float2bfloat16(v);
    else out[i] = v;
  }
}

// segment s covers sorted positions [seg_start[s], seg_start[s+1]) which all hold token seg_token[s]
__global__ void embedding_bwd_sorted_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ order,
                                            const long long* __restrict__ seg_start, const long long* __restrict__ seg_token,
                                            float* __restrict__ dwte, int C, long long vocab) {
  const long long s = blockIdx.x;
  const long long tok = seg_token[s];
  if (tok < 0 || tok >= vocab) return;
  const long long lo = seg_start[s], hi = seg_start[s + 1];
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.0f;
    for (long long j = lo; j < hi; ++j) acc += __bfloat162float(dout[order[j] * C + c]);
    dwte[tok * C + c] += acc;
  }
}

// positional rows: position t receives the rows t, T+t, 2T+t, ... in batch order
__global__ void posemb_bwd_kernel(const __nv_bfloat16* __restrict__ dout, float* __restrict__ dwpe, long long B, int T, int C) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.0f;
    for (long long b = 0; b < B; ++b) acc += __bfloat162float(dout[(b * T + t) * C + c]);
    dwpe[(long long)t * C + c] += acc;
  }
}

inline unsigned grid_for(long long n) {
  long long g = (n + 255) / 256;
  return (unsigned)(g < 1 ? 1 : (g > 148LL * 16 ? 148LL * 16 : g));
}

}  // namespace

extern "C" int incin_quantize_q8_0(const void* x, void* packed, long long n, int is_bf16, void* stream) {
  if (!x || !packed || n <= 0) return INCIN_ERR_ARGUMENT;
  const long long nb = (n + QK - 1) / QK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(nb * 32);
  if (is_bf16) quantize_q8_0_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(packed), n, nb);
  else quantize_q8_0_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<uint8_t*>(packed), n, nb);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_dequantize_q8_0(const void* packed, void* out, long long n, int out_bf16, void* stream) {
  if (!packed || !out || n <= 0) return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (out_bf16) dequantize_q8_0_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, s>>>(static_cast<const uint8_t*>(packed), static_cast<__nv_bfloat16*>(out), n);
  else dequantize_q8_0_kernel<float><<<grid_for(n), 256, 0, s>>>(static_cast<const uint8_t*>(packed), static_cast<float*>(out), n);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_embedding_bwd_sorted(const void* dout, const long long* order, const long long* seg_start,
                                          const long long* seg_token, long long n_segments, float* dwte, float* dwpe, long long B,
                                          int T, int C, long long vocab, void* stream) {
  if (!dout || !order || !seg_start || !seg_token || !dwte || n_segments <= 0 || C <= 0 || n_segments > 0x7fffffffLL)
    return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  embedding_bwd_sorted_kernel<<<(unsigned)n_segments, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dout), order, seg_start, seg_token, dwte, C, vocab);
  if (dwpe) posemb_bwd_kernel<<<T, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dout), dwpe, B, T, C);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}
