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
// The attribute is OFF by default and switched on with INCIN_PDL=1: measured on one B200 inside the captured graph
// of a GPT-2-small training step it made the step 1.8 % SLOWER (12.99 ms against 12.76 ms, two runs each; the
// early-scheduled successors raise the power draw until the power cap engages), so ordinary launches stay the default.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace incin {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("INCIN_PDL");
    return e && e[0] == '1';
  }();
  return on;
}

template <typename... KArgs, typename... Args>
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
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace incin
