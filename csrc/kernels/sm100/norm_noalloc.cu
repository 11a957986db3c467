// LayerNorm backward for callers that cannot allocate: same kernels as incin_layernorm_bwd(), with the
// dgamma/dbeta partial-sum scratch taken from a fixed device array instead of a caller-provided buffer.
// See incin_b200_noalloc.h for who needs this and for the rules of use.
#include <cuda_runtime.h>
#include <mutex>

#include "../../include/incin_b200.h"
#include "../../include/incin_b200_noalloc.h"

// Lives in this library's device data segment on every GPU that loads it (4 MiB), until process exit.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_ln_bwd_scratch[INCIN_LN_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device; looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return INCIN_ERR_DRIVER;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_ln_bwd_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // leave no sticky error behind for the caller
      return INCIN_ERR_DRIVER;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return INCIN_OK;
}
}  // namespace

extern "C" int incin_layernorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean,
                                           const float* rstd, const void* dx_add, void* dx, float* dgamma,
                                           float* dbeta, long long rows, int C, void* stream) {
  if (rows <= 0 || C <= 0 || !dy || !x || !gamma || !mean || !rstd || !dx) return INCIN_ERR_ARGUMENT;
  if (incin_layernorm_bwd_scratch_floats(rows, C) > INCIN_LN_NOALLOC_MAX_FLOATS) return INCIN_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != INCIN_OK) return rc;
  // The partial-sum kernel writes every scratch element the final kernel reads, so stale contents from
  // an earlier call are never observed and nothing has to be zeroed here.
  return incin_layernorm_bwd(dy, x, gamma, mean, rstd, dx_add, dx, dgamma, dbeta, scratch, rows, C, stream);
}
