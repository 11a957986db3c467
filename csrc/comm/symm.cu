// Peer-mapped buffers: plain cudaMalloc memory shared between the per-GPU processes through CUDA IPC
// handles.  A mapping obtained here is an ordinary device pointer into the peer's HBM, reached over
// NVLink/NVSwitch by plain loads and stores from inside kernels.  (The reference has no peer-memory
// path: its transport is NCCL calls only, crates/incin-backends/src/dist/nccl.rs:1842-1935.)
#include <cuda_runtime.h>
#include <cstring>

#include "../include/incin_b200.h"
#include "../include/incin_comm.h"

static_assert(sizeof(cudaIpcMemHandle_t) == INCIN_IPC_HANDLE_BYTES, "IPC handle size");

extern "C" int incin_symm_alloc(long long bytes, void** ptr_out, uint8_t* handle_out) {
  if (bytes <= 0 || !ptr_out || !handle_out) return INCIN_ERR_ARGUMENT;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return INCIN_ERR_DRIVER;
  if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess) return INCIN_ERR_DRIVER;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return INCIN_ERR_PEER;
  }
  std::memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return INCIN_OK;
}

extern "C" int incin_symm_open(const uint8_t* handle, void** ptr_out) {
  if (!handle || !ptr_out) return INCIN_ERR_ARGUMENT;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return INCIN_ERR_PEER;
  }
  *ptr_out = p;
  return INCIN_OK;
}

extern "C" int incin_symm_close(void* peer_ptr) {
  return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? INCIN_OK : INCIN_ERR_PEER;
}
extern "C" int incin_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? INCIN_OK : INCIN_ERR_DRIVER; }

extern "C" int incin_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return ok;
}
