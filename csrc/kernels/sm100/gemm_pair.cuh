// CTA-pair variant of the tcgen05 GEMM (cta_group::2): two CTAs of a 2-CTA cluster, on neighbouring SMs, compute
// one 256 x 256 output tile.  Each CTA loads 128 rows of A and 128 of the tile's 256 B rows per k-block (32 KB per
// stage, seven stages, or six plus the output staging area), the leader CTA issues M=256, N=256 MMAs for the pair, and each CTA's tensor memory receives
// the accumulator of its own 128 rows.  Per FLOP a CTA reads one third less shared memory than the single-CTA
// 128 x 256 tile, which is the bound of that kernel; the operand traffic from L2 halves for B.
//
// Synchronisation (all waits bounded, same status codes as the single-CTA kernel):
//   full[s]    leader's barrier: one arrive.expect_tx by the leader's producer for the bytes of BOTH CTAs; the TMA
//              loads of both CTAs signal it (the peer's loads name the leader's barrier through its cluster address)
//   empty[s]   one per CTA: the leader's MMA thread commits to its own and to the peer's after consuming stage s
//   tfull[a]   one per CTA: committed by the leader when accumulator a is complete
//   tempty[a]  leader's: 16 arrivals = 8 epilogue warps of each CTA (the peer's arrive remotely)
// Included by gemm_tcgen05.cu (shares its tensor-map helper and launch plumbing).
#pragma once
#include "gemm_common.cuh"

namespace incin {

template <bool STG = true>
struct PairCfg {
  static constexpr int BN = 256;                 // tile N (pair)
  static constexpr int BN_CTA = 128;             // B rows each CTA loads
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN_CTA * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = STG ? 6 : 7;     // 192 KB of operands + 32 KB of output staging, or 224 KB of operands
  static constexpr int ACC_STRIDE = 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int STG_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = STG_OFF + (STG ? STG_BYTES : 0);
  static constexpr int SMEM_BYTES = BAR_OFF + 1024 /*align*/ + 256 /*barriers*/;
};

// tile order of the pair kernel: 256-row blocks, m fastest (neighbouring pairs share a B tile in L2)
__device__ __forceinline__ Unit decode_pair_unit(const GemmKernelParams& p, int tiles_m2, int u) {
  Unit w;
  const int split = u % p.splits;
  int t = u / p.splits;
  w.m_blk = t % tiles_m2;
  t /= tiles_m2;
  w.n_blk = t % p.tiles_n;
  const int b = t / p.tiles_n;
  w.b_lo = b % p.batch_lo;
  w.b_hi = b / p.batch_lo;
  const int kb_total = (p.K + BK - 1) / BK;
  w.kb0 = static_cast<int>((static_cast<long long>(split) * kb_total) / p.splits);
  w.kb1 = static_cast<int>((static_cast<long long>(split + 1) * kb_total) / p.splits);
  return w;
}

// p.tiles_n counts 256-wide tiles here; p.total_units = tiles_m2 * tiles_n * batch * splits
template <bool A_MN, bool B_MN, bool STG>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
                         const GemmKernelParams p, const int tiles_m2) {
  using Cfg = PairCfg<STG>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* full_bar = bars;                      // [STAGES]  (the leader's are the ones in use)
  uint64_t* empty_bar = bars + Cfg::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]       (the leader's are the ones in use)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = (int)blockIdx.x >> 1;
  const int n_pairs = (int)gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 16);
    }
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tma_out && p.out_fp32) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // both CTAs' barriers are initialised and both allocations are done before anyone signals
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();   // both CTAs hold their tensor memory
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (one per CTA)
    // the whole warp walks the loop (warp-uniform waits and coordinate arithmetic); one elected lane issues the copies
    const bool lead_lane = elect_one() != 0;
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair; u < p.total_units && ok; u += n_pairs) {
        const Unit w = decode_pair_unit(p, tiles_m2, u);
        const int m0 = w.m_blk * 256 + (int)rank * BM;
        const int n0 = w.n_blk * Cfg::BN + (int)rank * Cfg::BN_CTA;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BK;
          if (lead_lane) {
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_4d_pair(sa, &tmA, bar, k0, m0, w.b_lo, w.b_hi);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_4d_pair(sa + c * 8192, &tmA, bar, m0 + c * 64, k0, w.b_lo, w.b_hi);
          }
          if (!B_MN) {
            tma_load_4d_pair(sb, &tmB, bar, k0, n0, w.b_lo, w.b_hi);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::BN_CTA / 64; ++c)
              tma_load_4d_pair(sb + c * 8192, &tmB, bar, n0 + c * 64, k0, w.b_lo, w.b_hi);
          }
          }
          __syncwarp();
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader CTA only)
    // the whole warp of the leader CTA walks the loop; one elected lane issues
    const bool lead_lane = elect_one() != 0;
    if (leader) {
      constexpr uint32_t idesc = make_idesc_bf16(256, Cfg::BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int u = pair; u < p.total_units && ok; u += n_pairs, ++iter) {
        const Unit w = decode_pair_unit(p, tiles_m2, u);
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, kStatusTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kStatusTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
          const uint64_t adesc = A_MN ? make_smem_desc(sa, 8192, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc(sb, 8192, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_adv = A_MN ? (uint64_t)(k * 2048 >> 4) : (uint64_t)(k * 32 >> 4);
            const uint64_t b_adv = B_MN ? (uint64_t)(k * 2048 >> 4) : (uint64_t)(k * 32 >> 4);
            if (lead_lane) umma_f16_ss_pair(d_tmem, adesc + a_adv, bdesc + b_adv, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          if (lead_lane) {
            umma_commit_pair(map_to_cta(eb, 0));
            umma_commit_pair(map_to_cta(eb, 1));
          }
          __syncwarp();
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && lead_lane) {   // accumulator complete: tell the epilogue warps of both CTAs
          const uint32_t tb = smem_u32(&tfull_bar[acc]);
          umma_commit_pair(map_to_cta(tb, 0));
          umma_commit_pair(map_to_cta(tb, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (8 warps per CTA: 4 lane quarters x 2 halves)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
    constexpr int CHUNKS_PER_HALF = Cfg::BN / 64;
    const int row_in_tile = quarter * 32 + lane;
    int iter = 0;
    for (int u = pair; u < p.total_units; u += n_pairs, ++iter) {
      const Unit w = decode_pair_unit(p, tiles_m2, u);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusTimeoutTmemFull)) break;
      tc_fence_after();
      const int m = w.m_blk * 256 + (int)rank * BM + row_in_tile;
      const int n0 = w.n_blk * Cfg::BN;
      const bool row_ok = m < p.M;
      const long long cbase = (long long)w.b_lo * p.c_stride_lo + (long long)w.b_hi * p.c_stride_hi + (long long)m * p.ldc;
      const bool vec_ok = (p.ldc % 8 == 0) && (p.c_stride_lo % 8 == 0) && (p.c_stride_hi % 8 == 0);
      if (STG && p.tma_out) {
        const int col_first = half * (Cfg::BN / 2);
        epilogue_staged(p, &tmC, &tmAux, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * Cfg::ACC_STRIDE + col_first,
                        smem + Cfg::STG_OFF + (warp - 2) * STG_WARP_BYTES, w.m_blk * 256 + (int)rank * BM + quarter * 32,
                        n0 + col_first, Cfg::BN / 2, w.b_lo, w.b_hi, cbase, row_ok, alpha, lane);
      } else {
#pragma unroll 1
      for (int c = half * CHUNKS_PER_HALF; c < (half + 1) * CHUNKS_PER_HALF; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * Cfg::ACC_STRIDE + c * 32, r);
        tmem_ld_wait();
        const int nc = n0 + c * 32;
        if (row_ok && nc < p.N) epilogue_chunk(p, r, p.C, cbase, nc, vec_ok, alpha);
        __syncwarp();
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
    }
    if (STG && p.tma_out && p.out_fp32 && lane == 0) bulk_wait_all();   // this warp's staged boxes have been written before the CTA retires
  }

  // common exit: every thread of both CTAs arrives here, also after a timed-out wait
  tc_fence_before();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);   // let copies that are still in flight land
  }
  cluster_sync_all();   // the peer may still read this CTA's shared memory / signal its barriers until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace incin
