// Cycles per tcgen05.mma (M 128, K 16, bf16) by N, operand layout and operand source: the figures behind the tile and
// pipeline choices of the attention and GEMM kernels.  Every wait is bounded.  Built and run by
// `python -m incin_b200.benchmarks.mma_rate`.
#include "../kernels/sm100/ptx.cuh"
#include <cstdio>
#include <vector>
using namespace incin;

struct Res { long long issue, done; int status; };

template <int N, bool A_MN, bool B_MN, bool TS, int NACC>
__global__ void __launch_bounds__(128, 1) rate_kernel(Res* out, int n_mma, int* status) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 128 * 1024);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
  for (int i = threadIdx.x; i < 128 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(bar, 1); *abort_flag = 0; mbar_init_fence(); }
  if (threadIdx.x < 32) { tmem_alloc(slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, N, A_MN, B_MN);
    const uint32_t aA = smem_u32(smem), aB = smem_u32(smem + 32 * 1024);
    long long t0 = clock64();
    for (int i = 0; i < n_mma; i += 8) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int k4 = kk & 3;
        const uint64_t ad = A_MN ? make_smem_desc(aA + kk * 2048, 16384, 1024) : make_smem_desc(aA + k4 * 32 + (kk >> 2) * 16384, 16, 1024);
        const uint64_t bd = B_MN ? make_smem_desc(aB + kk * 2048, 16384, 1024) : make_smem_desc(aB + k4 * 32 + (kk >> 2) * 32768, 16, 1024);
        const uint32_t d = tm + (((i >> 3) % NACC) * N) % 256;
        if (TS) umma_f16_ts(d, tm + 256 + kk * 8, bd, idesc, 1u);
        else umma_f16_ss(d, ad, bd, idesc, 1u);
      }
    }
    long long t1 = clock64();
    umma_commit(bar);
    bool ok = mbar_wait(bar, 0, abort_flag, status, kStatusTimeoutTmemFull);
    long long t2 = clock64();
    out[blockIdx.x].issue = t1 - t0;
    out[blockIdx.x].done = t2 - t0;
    out[blockIdx.x].status = ok ? 0 : 1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tm, 512);
}

template <int N, bool A_MN, bool B_MN, bool TS, int NACC>
void run(const char* name, int grid) {
  auto k = rate_kernel<N, A_MN, B_MN, TS, NACC>;
  const int smem = 128 * 1024 + 1024 + 256;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  Res* d; int* st;
  cudaMalloc(&d, sizeof(Res) * grid); cudaMalloc(&st, 4); cudaMemset(st, 0, 4);
  const int n = 512;
  for (int rep = 0; rep < 3; ++rep) k<<<grid, 128, smem>>>(d, n, st);
  cudaError_t e = cudaDeviceSynchronize();
  std::vector<Res> h(grid);
  cudaMemcpy(h.data(), d, sizeof(Res) * grid, cudaMemcpyDeviceToHost);
  double is = 0, dn = 0; int bad = 0;
  for (auto& r : h) { is += r.issue; dn += r.done; bad += r.status; }
  const double flop_per_clk = 2.0 * 128 * N * 16 / (dn / grid / n);
  printf("%-44s grid %3d  issue %.1f  done %.1f cycles/MMA  -> %.0f FLOP/clk/SM (peak 8192) err=%s bad=%d\n", name, grid,
         is / grid / n, dn / grid / n, flop_per_clk, cudaGetErrorString(e), bad);
  cudaFree(d); cudaFree(st);
}

int main() {
  for (int grid : {1, 148}) {
    run<64, false, false, false, 1>("N64  A K-major  B K-major", grid);
    run<128, false, false, false, 1>("N128 A K-major  B K-major", grid);
    run<256, false, false, false, 1>("N256 A K-major  B K-major", grid);
    run<64, false, true, false, 1>("N64  A K-major  B MN-major (dV,dK)", grid);
    run<64, true, true, false, 1>("N64  A MN-major B MN-major (dQ)", grid);
    run<128, false, true, false, 1>("N128 A K-major  B MN-major", grid);
    run<128, true, true, false, 1>("N128 A MN-major B MN-major", grid);
    run<64, false, false, false, 4>("N64  K/K, 4 accumulators in turn", grid);
    run<64, false, true, true, 1>("N64  A in TMEM, B MN-major", grid);
    run<128, false, true, true, 1>("N128 A in TMEM, B MN-major", grid);
    run<64, false, false, true, 1>("N64  A in TMEM, B K-major", grid);
    run<128, false, false, true, 1>("N128 A in TMEM, B K-major", grid);
  }
  return 0;
}
