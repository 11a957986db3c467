// Kernel launch with programmatic dependent launch: the next kernel of the stream may be scheduled while this one is
// still draining, runs its prologue (barrier set-up, tensor-memory allocation, descriptor prefetch) and then waits at
// pdl_wait() until every kernel before it has completed and its writes are visible.  That hides the launch gap and
// the prologue behind the tail of the previous kernel; inside a captured CUDA graph the edge is kept as a
// programmatic dependency.
//
// Contract for a kernel launched through launch_pdl():
//   * it touches no global memory before pdl_wait();
//   * it calls pdl_launch_dependents() only after it holds every per-SM resource a successor could take away from
//     one of its own CTAs (tensor memory: a successor CTA that allocated first would wait for this grid to finish
//     while this grid waits for the allocation).  Plain kernels call it first thing.
// Both instructions are no-ops in a kernel that was launched the ordinary way, and a successor launched the ordinary
// way simply waits for full completion, so instrumented and plain kernels mix freely.
// INCIN_PDL selects who gets the attribute: 2 (default) = only the tensor-core kernels (GEMM, attention), 1 = every
// instrumented kernel, 0 = nobody.  Measured on one B200 inside the captured graph of a GPT-2-small training step
// (20 steps, two runs each): off 12.70 / 12.73 ms, tensor-core kernels only 12.61 / 12.62 ms, everything 12.94 ms -
// early-scheduled grids of the small bandwidth kernels cost more than their hidden launch gaps give back.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace incin {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 0: off.  1: every instrumented kernel.  2 (default): only the tensor-core kernels (GEMM, attention).
inline int pdl_mode() {
  static const int mode = [] {
    const char* e = std::getenv("INCIN_PDL");
    return (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;
  }();
  return mode;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-DEVICE property of a kernel, so "already set" is remembered per
// device: a process that launches on a second GPU sets it there too instead of launching with the 48 KB default.
// A static instance is zero-initialised; flags are read and written with atomics because any host thread may launch.
constexpr int kMaxDevicesPerProcess = 64;
struct PerDeviceFlags {
  unsigned char set[kMaxDevicesPerProcess];
};

template <typename Kern>
inline bool ensure_dynamic_smem(Kern kern, int bytes, PerDeviceFlags& flags) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  const bool tracked = dev >= 0 && dev < kMaxDevicesPerProcess;
  if (tracked && __atomic_load_n(&flags.set[dev], __ATOMIC_ACQUIRE)) return true;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (tracked) __atomic_store_n(&flags.set[dev], (unsigned char)1, __ATOMIC_RELEASE);
  return true;
}

template <bool HEAVY = false, typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mode() == 1 || (HEAVY && pdl_mode() == 2)) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace incin
