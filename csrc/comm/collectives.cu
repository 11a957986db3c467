// Stand-alone collectives over peer-mapped (symmetric) buffers: all-gather, reduce-scatter, all-reduce, all-to-all
// and point-to-point send / wait for pipeline stages.  One process per GPU; `bufs[r]` is rank r's buffer as mapped
// into this process (CUDA IPC), so a peer's data is read with plain 128-bit loads over NVLink.
//
// Counterparts: the reference's NCCL launches (crates/incin-backends/src/transport/nccl.rs:1842-1935: ncclAllReduce,
// ncclAllGather, ncclReduceScatter, grouped ncclSend/ncclRecv for all-to-all and pipeline transfers) and the
// semantics of its in-process ReferenceTransport (transport/reference.rs:170-260).  These kernels are the utility
// layer; the hot tensor-parallel and data-parallel paths use the fused kernels instead.
//
// Synchronisation contract: the caller brackets a collective with the cross-GPU barrier kernel (every rank's input
// is written before anyone reads it; every rank has finished reading before an input buffer is reused).  Send /
// wait carry their own signal: the sender copies into the receiver's buffer and then releases a sequence number
// into the receiver's flag word at system scope; the receiver's wait kernel spins on its LOCAL flag with a bound
// and writes a status word if the bound is hit, so a missing sender never hangs the GPU.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "incin_b200.h"
#include "incin_comm.h"

namespace {

enum { RED_SUM = 0, RED_MEAN = 1, RED_MAX = 2, RED_MIN = 3 };
constexpr int MAX_WORLD = 8;

struct Peers {
  const char* p[MAX_WORLD];
};

inline unsigned grid_for(long long n, int per_thread = 1) {
  long long g = (n + 256LL * per_thread - 1) / (256LL * per_thread);
  return (unsigned)(g < 1 ? 1 : (g > 148LL * 8 ? 148LL * 8 : g));
}

// out[r * bytes + i] = bufs[r][off + i]     (all-gather: chunk = bytes, src_rank_stride = 0)
// out[r * bytes + i] = bufs[r][off + rank * bytes + i]   (all-to-all: src_rank_stride = bytes)
__global__ void gather_chunks_kernel(Peers peers, int world, int rank, long long off, long long bytes, long long src_rank_stride,
                                     char* __restrict__ out) {
  const long long vec_per = bytes / 16;
  const long long total = vec_per * world;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    // start with the own chunk's neighbour so the ranks do not all read the same peer at the same time
    const int r = (int)((t / vec_per + rank) % world);
    const long long i = t % vec_per;
    const uint4 v = reinterpret_cast<const uint4*>(peers.p[r] + off + rank * src_rank_stride)[i];
    reinterpret_cast<uint4*>(out + (long long)r * bytes)[i] = v;
  }
}

__device__ __forceinline__ float red(float a, float b, int op) {
  return op == RED_MAX ? fmaxf(a, b) : (op == RED_MIN ? fminf(a, b) : a + b);
}

// out[i] = reduce over r of bufs[r][off + i]  for i in [0, n) (16-byte vectors; fp32 or bf16 elements, fp32 math).
// Ranks are combined in rank order on every GPU, so all ranks compute bitwise identical results.
template <bool BF16>
__global__ void reduce_peers_kernel(Peers peers, int world, long long off_bytes, long long n_vec, int op, void* __restrict__ out) {
  const float scale = op == RED_MEAN ? 1.0f / (float)world : 1.0f;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n_vec; t += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    uint4 v = reinterpret_cast<const uint4*>(peers.p[0] + off_bytes)[t];
    constexpr int E = BF16 ? 8 : 4;
    if (BF16) {
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = __bfloat162float(e[k]);
    } else {
      const float* e = reinterpret_cast<const float*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] = e[k];
    }
    for (int r = 1; r < world; ++r) {
      v = reinterpret_cast<const uint4*>(peers.p[r] + off_bytes)[t];
      if (BF16) {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = red(acc[k], __bfloat162float(e[k]), op);
      } else {
        const float* e = reinterpret_cast<const float*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[k] = red(acc[k], e[k], op);
      }
    }
    uint4 o;
    if (BF16) {
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int k = 0; k < E; ++k) e[k] = __float2bfloat16(acc[k] * scale);
    } else {
      float* e = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int k = 0; k < E; ++k) e[k] = acc[k] * scale;
    }
    reinterpret_cast<uint4*>(out)[t] = o;
  }
}

__global__ void copy_vec_kernel(const char* __restrict__ src, char* __restrict__ dst, long long n_vec) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n_vec; t += (long long)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(dst)[t] = reinterpret_cast<const uint4*>(src)[t];
}

__global__ void signal_kernel(uint32_t* peer_flag, uint32_t seq) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(seq) : "memory");
}

__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t seq, int* status, long long max_clocks) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t f;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(f) : "l"(flag) : "memory");
    if ((int32_t)(f - seq) >= 0) return;   // sequence numbers wrap
    if (clock64() - t0 > max_clocks) {
      if (status) atomicCAS(status, 0, 5 /* waited for a flag another GPU never set */);
      return;
    }
    __nanosleep(200);
  }
}

bool fill(Peers& P, void* const* bufs, int world) {
  if (!bufs || world < 1 || world > MAX_WORLD) return false;
  for (int r = 0; r < world; ++r) {
    if (!bufs[r]) return false;
    P.p[r] = static_cast<const char*>(bufs[r]);
  }
  return true;
}

}  // namespace

extern "C" int incin_coll_all_gather(void* const* bufs, int world, int rank, long long offset_bytes, long long bytes, void* out,
                                     void* stream) {
  Peers P;
  if (!fill(P, bufs, world) || !out || bytes <= 0 || (bytes % 16) || (offset_bytes % 16) || rank < 0 || rank >= world)
    return INCIN_ERR_ARGUMENT;
  gather_chunks_kernel<<<grid_for(bytes / 16 * world, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      P, world, rank, offset_bytes, bytes, 0, static_cast<char*>(out));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_coll_all_to_all(void* const* bufs, int world, int rank, long long offset_bytes, long long chunk_bytes,
                                     void* out, void* stream) {
  Peers P;
  if (!fill(P, bufs, world) || !out || chunk_bytes <= 0 || (chunk_bytes % 16) || (offset_bytes % 16) || rank < 0 || rank >= world)
    return INCIN_ERR_ARGUMENT;
  gather_chunks_kernel<<<grid_for(chunk_bytes / 16 * world, 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      P, world, rank, offset_bytes, chunk_bytes, chunk_bytes, static_cast<char*>(out));
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

// out[0..n) = reduce_r bufs[r][offset + first_elem + i]; reduce-scatter passes first_elem = rank * n, all-reduce 0.
extern "C" int incin_coll_reduce(void* const* bufs, int world, long long offset_bytes, long long first_elem, long long n, int op,
                                 int is_bf16, void* out, void* stream) {
  Peers P;
  const int esz = is_bf16 ? 2 : 4;
  if (!fill(P, bufs, world) || !out || n <= 0 || op < 0 || op > RED_MIN || (offset_bytes % 16) || (n * esz) % 16 ||
      (first_elem * esz) % 16)
    return INCIN_ERR_ARGUMENT;
  const long long n_vec = n * esz / 16, off = offset_bytes + first_elem * esz;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16) reduce_peers_kernel<true><<<grid_for(n_vec, 2), 256, 0, s>>>(P, world, off, n_vec, op, out);
  else reduce_peers_kernel<false><<<grid_for(n_vec, 2), 256, 0, s>>>(P, world, off, n_vec, op, out);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_p2p_send(void* peer_dst, const void* src, long long bytes, void* peer_flag, unsigned seq, void* stream) {
  if (!peer_dst || !src || !peer_flag || bytes <= 0 || (bytes % 16) || ((uintptr_t)peer_dst % 16) || ((uintptr_t)src % 16))
    return INCIN_ERR_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  copy_vec_kernel<<<grid_for(bytes / 16, 4), 256, 0, s>>>(static_cast<const char*>(src), static_cast<char*>(peer_dst), bytes / 16);
  signal_kernel<<<1, 1, 0, s>>>(static_cast<uint32_t*>(peer_flag), seq);   // after the copy in stream order
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

extern "C" int incin_p2p_wait(const void* local_flag, unsigned seq, void* status, long long timeout_ms, void* stream) {
  if (!local_flag) return INCIN_ERR_ARGUMENT;
  if (timeout_ms <= 0) timeout_ms = 1000;
  if (timeout_ms > 10000) timeout_ms = 10000;
  wait_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(local_flag), seq,
                                                                      static_cast<int*>(status), timeout_ms * 2000000LL);
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}
