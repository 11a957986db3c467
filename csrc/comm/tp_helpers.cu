// Small kernels around the fused tensor-parallel GEMMs: a cross-GPU barrier, the owner-side slot reduction of the
// GEMM -> reduce-scatter path, and an in-place sum of fp32 ranges over a peer sub-group.  All peer traffic is
// plain loads/stores on IPC-mapped pointers; every wait is bounded and reports through the status word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/incin_b200.h"
#include "../include/incin_comm.h"

namespace incin {

#ifndef INCIN_PEER_WAIT_CLOCKS
#define INCIN_PEER_WAIT_CLOCKS (6000000000ll)
#endif

constexpr int BAR_SLOTS = 64;
constexpr int BAR_WORDS = 16;  // per slot: arrive[8], epoch, pad

// pad layout: [slot][BAR_WORDS] uint32
__global__ void peer_barrier_kernel(uint32_t* const* pads_in, int world, int rank, int slot, int* status) {
  __shared__ uint32_t* pads[INCIN_MAX_PEERS];
  if (threadIdx.x < world) pads[threadIdx.x] = pads_in[threadIdx.x];
  __syncthreads();
  uint32_t* mine = pads[rank] + slot * BAR_WORDS;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine + INCIN_MAX_PEERS) + 1;
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    uint32_t* dst = pads[threadIdx.x] + slot * BAR_WORDS + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
    const long long t0 = clock64();
    uint32_t v;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + threadIdx.x) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (clock64() - t0 > INCIN_PEER_WAIT_CLOCKS) {
        if (status) atomicCAS(status, 0, 5 /* kStatusTimeoutPeer */);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(mine + INCIN_MAX_PEERS) = epoch;
}

__global__ void __launch_bounds__(256)
slot_reduce_kernel(const __nv_bfloat16* __restrict__ slots, long long slot_stride, int world,
                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, long long rows, int N,
                   long long ld) {
  const long long vec_per_row = N / 8;
  const long long total = rows * vec_per_row;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / vec_per_row;
    const long long off = r * ld + (i - r * vec_per_row) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s) {
      const uint4 u = *reinterpret_cast<const uint4*>(slots + s * slot_stride + off);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    if (residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(residual + off);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) oh[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + off) = o;
  }
}

__global__ void __launch_bounds__(256)
peer_sum_ranges_kernel(float* const* bases_in, int world, const long long* __restrict__ ranges, int n_ranges,
                       float* __restrict__ scratch, int stage) {
  __shared__ float* bases[INCIN_MAX_PEERS];
  if (threadIdx.x < world) bases[threadIdx.x] = bases_in[threadIdx.x];
  __syncthreads();
  long long soff = 0;
  for (int k = 0; k < n_ranges; ++k) {
    const long long off = ranges[2 * k], len = ranges[2 * k + 1];
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
      if (stage == 0) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += bases[r][off + i];   // rank order: identical result on every peer
        scratch[soff + i] = a;
      } else {
        bases[0][off + i] = scratch[soff + i];                    // bases[0] is this rank's own buffer in stage 1
      }
    }
    soff += len;
  }
}

}  // namespace incin

using namespace incin;

extern "C" int incin_barrier_pad_bytes(void) { return BAR_SLOTS * BAR_WORDS * 4; }

extern "C" int incin_peer_barrier(void* const* pads, int world, int rank, int slot, void* status, void* stream) {
  if (!pads || world < 1 || world > INCIN_MAX_PEERS || rank < 0 || rank >= world || slot < 0 || slot >= BAR_SLOTS)
    return INCIN_ERR_ARGUMENT;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t* const*)pads, world, rank, slot, (int*)status);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_slot_reduce(const void* slots, long long slot_stride, int world, const void* residual, void* out,
                                 long long rows, int N, long long ld, void* stream) {
  if (!slots || !out || world < 1 || rows <= 0 || N <= 0 || (N % 8) || (ld % 8) || (slot_stride % 8))
    return INCIN_ERR_ARGUMENT;
  long long blocks = (rows * (N / 8) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  slot_reduce_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)slots, slot_stride, world, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, rows, N, ld);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_peer_sum_ranges(void* const* bases, int world, const void* ranges, int n_ranges, void* scratch,
                                     int stage, void* stream) {
  if (!bases || world < 1 || world > INCIN_MAX_PEERS || !ranges || n_ranges < 1 || !scratch) return INCIN_ERR_ARGUMENT;
  peer_sum_ranges_kernel<<<148, 256, 0, (cudaStream_t)stream>>>((float* const*)bases, world, (const long long*)ranges,
                                                               n_ranges, (float*)scratch, stage);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}
