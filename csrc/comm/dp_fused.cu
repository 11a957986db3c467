// Data-parallel gradient reduction fused with the optimiser, over NVLink peer memory.
//
// One kernel per gradient bucket does, on every rank at once:
//   1. handshake   : tell every peer "my gradients of this bucket are final", wait for theirs
//                    (flag words in peer-mapped memory, release/acquire at system scope,
//                    every spin bounded by a clock budget -> status word, never a hang);
//   2. reduce      : each rank owns 1/world of the bucket and sums that slice straight out of
//                    every peer's fp32 gradient buffer with 16-byte P2P loads (reduce-scatter
//                    without a staging buffer), scales by 1/world;
//   3. update      : bias-corrected AdamW on the owned slice of the fp32 master weights and
//                    moments (optimizer work and state traffic drop to 1/world per rank);
//   4. broadcast   : writes the new bf16 weights into every peer's parameter buffer with P2P
//                    stores (all-gather without a staging buffer);
//   5. handshake   : signals "done" to every peer and holds the stream until all peers are done,
//                    so the next forward pass never reads a half-written parameter buffer and
//                    the next zero-grad never clears a buffer a peer is still reading.
//
// The reference performs one ncclAllReduce(Avg) per parameter tensor after backward, waits on the
// host between them, and runs the optimiser as ~15 separate elementwise launches per tensor
// (crates/incin-backends/src/dist/nccl.rs:606-632,896-975,1842).
//
// Two variants of steps 2 and 4.  The default uses plain peer loads / stores only, so a rank that dies between steps
// cannot fault its peers' GPUs.  The multicast variant (incin_dp_reduce_adamw_mc) sums the owned slice inside
// NVSwitch (multimem.ld_reduce) and broadcasts the new weights with one multimem.st: per GPU and step 1/world of the
// gradient bytes come in instead of (world-1)/world of them, and 1/world of the weights go out instead of
// (world-1)/world.  It needs every rank alive while the buffers are bound to the multicast object.  Neither variant
// issues a TMA load from peer memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/incin_b200.h"
#include "../include/incin_comm.h"

namespace incin {

#ifndef INCIN_PEER_WAIT_CLOCKS
#define INCIN_PEER_WAIT_CLOCKS (6000000000ll)  // ~3 s: peers may be a whole backward pass behind
#endif

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// wait until flags[0..world) (local memory, written by peers) all reach `target`; false on timeout
__device__ bool wait_flags(const uint32_t* flags, int world, uint32_t target, int* status) {
  const long long t0 = clock64();
  for (int r = 0; r < world; ++r) {
    while ((int32_t)(ld_acquire_sys(flags + r) - target) < 0) {
      if (clock64() - t0 > INCIN_PEER_WAIT_CLOCKS) {
        if (status) atomicCAS(status, 0, 5 /* kStatusTimeoutPeer */);
        return false;
      }
      __nanosleep(200);
    }
  }
  return true;
}

// NVSwitch multicast ("multimem") accesses: a load that returns the sum over every GPU bound to the address, and a
// store that lands in every bound GPU's memory.  16-byte aligned multicast addresses.
__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_b128(void* mc, uint4 o) {   // 16 bytes, bit pattern unchanged
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(o.x)),
               "f"(__uint_as_float(o.y)), "f"(__uint_as_float(o.z)), "f"(__uint_as_float(o.w))
               : "memory");
}

struct DpParams {
  float* grads[INCIN_MAX_PEERS];           // every rank's flat fp32 gradient buffer (index = rank)
  __nv_bfloat16* shadows[INCIN_MAX_PEERS];  // every rank's flat bf16 parameter buffer
  uint32_t* pads[INCIN_MAX_PEERS];          // every rank's signal pad
  float *master, *m, *v;                    // local optimiser state (full length, owned slice is used)
  const float* hyper;
  long long lo, hi, n_decay;  // bucket range in elements (multiples of 8)
  int world, rank, slot;
  int* status;
  const float* mc_grads;        // multicast view of the gradient buffers (MC kernels only)
  __nv_bfloat16* mc_shadows;    // multicast view of the parameter buffers
};

// pad layout per slot: [ready: MAX_PEERS][done: MAX_PEERS][epoch][arrived][pad..] = 32 words
constexpr int PAD_WORDS_PER_SLOT = 32;

template <bool MC_G, bool MC_S>
__global__ void __launch_bounds__(512)
dp_reduce_adamw_kernel(const DpParams p) {
  uint32_t* mypad = p.pads[p.rank] + (size_t)p.slot * PAD_WORDS_PER_SLOT;
  uint32_t* ready = mypad;
  uint32_t* done = mypad + INCIN_MAX_PEERS;
  uint32_t* epoch_w = mypad + 2 * INCIN_MAX_PEERS;
  uint32_t* arrived = epoch_w + 1;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(epoch_w) + 1;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;

  // 1. handshake in
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.pads[threadIdx.x] + (size_t)p.slot * PAD_WORDS_PER_SLOT + p.rank, epoch);
  }
  if (threadIdx.x == 0) s_ok = wait_flags(ready, p.world, epoch, p.status) ? 1 : 0;
  __syncthreads();

  if (s_ok) {
    // 2-4. owned slice of this bucket, 8 elements per thread per iteration
    const long long len = p.hi - p.lo;
    long long per = ((len + p.world - 1) / p.world + 7) & ~7LL;
    const long long s0 = p.lo + per * p.rank;
    const long long s1 = (s0 + per < p.hi) ? s0 + per : p.hi;
    const float lr = p.hyper[0], b1 = p.hyper[1], b2 = p.hyper[2], eps = p.hyper[3], wd = p.hyper[4];
    const float step = p.hyper[5], gs = p.hyper[6] / (float)p.world;
    const float bc1 = 1.f - powf(b1, step), bc2 = 1.f - powf(b2, step);
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = s0 + ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < s1; i += stride) {
      float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if constexpr (MC_G) {   // the switch adds the world's gradients: one 16-byte response per 16 bytes of the slice
        const float4 a = mc_ld_reduce_f32x4(p.mc_grads + i);
        const float4 b = mc_ld_reduce_f32x4(p.mc_grads + i + 4);
        g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
        g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
      } else {
        for (int r = 0; r < p.world; ++r) {
          const int src = (p.rank + r) % p.world;  // stagger so peers are not all hit in the same order
          const float4 a = *reinterpret_cast<const float4*>(p.grads[src] + i);
          const float4 b = *reinterpret_cast<const float4*>(p.grads[src] + i + 4);
          g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
          g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
        }
      }
      float w[8], mm[8], vv[8];
      *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(p.master + i);
      *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(p.master + i + 4);
      *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(p.m + i);
      *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(p.m + i + 4);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(p.v + i);
      *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(p.v + i + 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float gr = g[k] * gs;
        mm[k] = b1 * mm[k] + (1.f - b1) * gr;
        vv[k] = b2 * vv[k] + (1.f - b2) * gr * gr;
        const float decay = (i + k) < p.n_decay ? wd : 0.f;
        w[k] = w[k] - lr * decay * w[k] - lr * (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps);
      }
      *reinterpret_cast<float4*>(p.master + i) = *reinterpret_cast<float4*>(w);
      *reinterpret_cast<float4*>(p.master + i + 4) = *reinterpret_cast<float4*>(w + 4);
      *reinterpret_cast<float4*>(p.m + i) = *reinterpret_cast<float4*>(mm);
      *reinterpret_cast<float4*>(p.m + i + 4) = *reinterpret_cast<float4*>(mm + 4);
      *reinterpret_cast<float4*>(p.v + i) = *reinterpret_cast<float4*>(vv);
      *reinterpret_cast<float4*>(p.v + i + 4) = *reinterpret_cast<float4*>(vv + 4);
      uint4 o;
      __nv_bfloat162 t;
      t = __floats2bfloat162_rn(w[0], w[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
      t = __floats2bfloat162_rn(w[2], w[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
      t = __floats2bfloat162_rn(w[4], w[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
      t = __floats2bfloat162_rn(w[6], w[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
      if constexpr (MC_S) {
        mc_st_b128(p.mc_shadows + i, o);   // one store, replicated by the switch into every rank's buffer
      } else {
        for (int r = 0; r < p.world; ++r) {
          const int dst = (p.rank + r) % p.world;
          *reinterpret_cast<uint4*>(p.shadows[dst] + i) = o;
        }
      }
    }
  }

  // 5. handshake out: the last block of this rank signals and waits
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(arrived, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(p.pads[threadIdx.x] + (size_t)p.slot * PAD_WORDS_PER_SLOT + INCIN_MAX_PEERS + p.rank, epoch);
    }
    if (threadIdx.x == 0) {
      wait_flags(done, p.world, epoch, p.status);
      *arrived = 0;
      *reinterpret_cast<volatile uint32_t*>(epoch_w) = epoch;
      __threadfence();
    }
  }
}

}  // namespace incin

using namespace incin;

static int dp_launch(const incin_dp_desc* d, void* mc_grads, void* mc_shadows, void* stream);

extern "C" int incin_dp_reduce_adamw(const incin_dp_desc* d, void* stream) { return dp_launch(d, nullptr, nullptr, stream); }

extern "C" int incin_dp_reduce_adamw_mc(const incin_dp_desc* d, void* mc_grads, void* mc_shadows, void* stream) {
  if ((!mc_grads && !mc_shadows) || (reinterpret_cast<uintptr_t>(mc_grads) & 15) || (reinterpret_cast<uintptr_t>(mc_shadows) & 15))
    return INCIN_ERR_ARGUMENT;   // either may be null: that side then uses the plain peer pointers
  return dp_launch(d, mc_grads, mc_shadows, stream);
}

static int dp_launch(const incin_dp_desc* d, void* mc_grads, void* mc_shadows, void* stream) {
  if (!d || d->world < 1 || d->world > INCIN_MAX_PEERS || d->rank < 0 || d->rank >= d->world) return INCIN_ERR_ARGUMENT;
  if ((d->lo & 7) || (d->hi & 7) || d->hi <= d->lo || d->slot < 0 || d->slot >= INCIN_DP_MAX_SLOTS)
    return INCIN_ERR_ARGUMENT;
  DpParams p;
  for (int r = 0; r < d->world; ++r) {
    p.grads[r] = (float*)d->grads[r];
    p.shadows[r] = (__nv_bfloat16*)d->shadows[r];
    p.pads[r] = (uint32_t*)d->pads[r];
    if (!p.grads[r] || !p.shadows[r] || !p.pads[r]) return INCIN_ERR_ARGUMENT;
  }
  p.master = (float*)d->master;
  p.m = (float*)d->m;
  p.v = (float*)d->v;
  p.hyper = (const float*)d->hyper;
  p.lo = d->lo;
  p.hi = d->hi;
  p.n_decay = d->n_decay;
  p.world = d->world;
  p.rank = d->rank;
  p.slot = d->slot;
  p.status = (int*)d->status;
  p.mc_grads = (const float*)mc_grads;
  p.mc_shadows = (__nv_bfloat16*)mc_shadows;
  int ctas = d->ctas > 0 ? d->ctas : 32;
  const long long per = (d->hi - d->lo + d->world - 1) / d->world;
  const long long need = (per + 512 * 8 - 1) / (512 * 8);
  if (need < ctas) ctas = (int)(need > 0 ? need : 1);
  if (mc_grads && mc_shadows) dp_reduce_adamw_kernel<true, true><<<ctas, 512, 0, (cudaStream_t)stream>>>(p);
  else if (mc_grads) dp_reduce_adamw_kernel<true, false><<<ctas, 512, 0, (cudaStream_t)stream>>>(p);
  else if (mc_shadows) dp_reduce_adamw_kernel<false, true><<<ctas, 512, 0, (cudaStream_t)stream>>>(p);
  else dp_reduce_adamw_kernel<false, false><<<ctas, 512, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_dp_pad_bytes(void) { return INCIN_DP_MAX_SLOTS * PAD_WORDS_PER_SLOT * 4; }
