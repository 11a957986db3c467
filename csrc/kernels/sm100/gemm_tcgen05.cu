// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[b][m][n] = epilogue( alpha * sum_k A[b][m][k] * B[b][n][k] )
//
// Data path: TMA (cp.async.bulk.tensor, this GPU's memory only, no cluster
// multicast) -> 128B-swizzled shared memory ring -> tcgen05.mma issued by one
// thread -> fp32 accumulators in tensor memory (double buffered, so the
// epilogue of tile i overlaps the main loop of tile i+1) -> tcgen05.ld ->
// fused epilogue (bias, GELU / SiLU, GELU-gradient mask, residual, bf16 or fp32
// store, fp32 atomic accumulate for split-K and gradient accumulation).
//
// Both operands may be K-major ("row = m, contiguous along k") or MN-major
// ("row = k, contiguous along m"), which covers the forward Linear
// (x @ W^T), the data gradient (dY @ W) and the weight gradient (dY^T @ X)
// without any transpose kernel.  Operands are addressed through 4-D tensor
// maps {inner, rows, batch_lo, batch_hi} so strided batches (attention heads
// inside a fused QKV buffer) need no copies either.
//
// Replaces the reference's f32 SIMT 128x128x8 SGEMM
// (crates/incin-backends/src/cuda/ops/kernels/matmul.cu:1-94), which is 2-D
// only and has no fused epilogue.
#include <type_traits>
#include "gemm_common.cuh"
#include "gemm_pair.cuh"

#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>
#include <cstdio>
#include <cstdlib>

#ifndef INCIN_GEMM_TMA_OUT_DEFAULT
#define INCIN_GEMM_TMA_OUT_DEFAULT 4
#endif

namespace incin {

template <int BN, bool A_MN, bool B_MN, bool STG>
__global__ void __launch_bounds__(GEMM_THREADS_COPY, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
                    const GemmKernelParams p) {
  using Cfg = GemmCfg<BN, STG>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BAR_OFF);
  uint64_t* full_bar = bars;                      // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* cw_bar = tempty_bar + 3;   // [2] barriers of the copy warp's two half rings (after tmem_slot and abort_flag)
  // Copy-warp mode: the last p.copy_warps operand stages are the copy warp's ring; the operand ring is that much shorter.
  constexpr int CW_CHUNK = 8 * 1024;
  const int n_stages = Cfg::STAGES - p.copy_warps;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // all-gather mode: the first CTAs of the grid (dispatched first) copy, the remaining gemm_ctas compute
  const int n_compute = ((p.ag_world > 1 || p.rs_push) && !p.copy_warps) ? p.gemm_ctas : (int)gridDim.x;
  const int n_copy = (int)gridDim.x - n_compute;
  const bool is_copier = (int)blockIdx.x < n_copy;
  const int cta = (int)blockIdx.x - n_copy;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
    }
    for (int b = 0; b < 2; ++b) mbar_init(&cw_bar[b], 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tma_out && p.out_fp32) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();   // tensor memory is held: a successor may be scheduled as SMs drain
  pdl_wait();                // nothing above touched global memory; everything below may depend on earlier kernels

  if (is_copier) {
    // ------------------------------------------------------------- copy CTA (one thread drives the bulk copies)
    // all-gather:     pulls 128-row tiles of the peers' shards (and the own shard) into the local gathered buffer
    //                 and publishes one flag per tile;
    // reduce-scatter: waits until a 128-row block of the partial product is complete in the local staging buffer
    //                 and pushes it into this rank's slot of the owner's buffer.
    // Either way the data moves global -> shared -> global in 32 KB bulk copies, so every byte crosses NVLink
    // exactly once and in large transfers.
    if (threadIdx.x == 0) {
      // 32 KB chunks through a ring that takes the whole operand memory.  What a copy CTA sustains is set by the bytes
      // it has in flight (measured between two B200s, 16 CTAs, loads from the peer: 64 KB ring 14 GB/s per CTA,
      // 192 KB ring 31-37 GB/s), so a buffer is recycled as soon as the store that drains it has read it; and by what
      // the one issuing thread spends per chunk (with 8 KB chunks the loop itself capped a CTA at 10 GB/s), hence the
      // large chunks.  The ring's barriers are the operand ring's (otherwise idle here), 2 * STAGES >= NBUF of them.
      constexpr int CHUNK = 32 * 1024;
      constexpr int NBUF = Cfg::STAGES * Cfg::STAGE_BYTES / CHUNK;
      constexpr int PENDING = NBUF / 2;   // bulk stores whose shared-memory reads may still be outstanding
      constexpr int LAG = 2;              // stores after which an earlier store is checked for completion
      static_assert(NBUF >= 4 && NBUF <= 2 * Cfg::STAGES, "staging ring");
      uint64_t* cbar = bars;
      const bool pull = p.ag_world > 1;
      const int copier = (int)blockIdx.x, n_copiers = n_copy;
      const long long row_bytes = pull ? (long long)p.K * 2 : (long long)p.N * 2;
      const long long tile_bytes = (long long)BM * row_bytes;
      const int chunks_per_tile = (int)((tile_bytes + CHUNK - 1) / CHUNK);
      const int tiles_per_rank = (pull ? p.ag_rows_per_rank : p.rs_rows_per_rank) / BM;
      // the list of 128-row tiles to move, in consumption order: every rank's rows but (push, or pull with the own
      // shard already in place) this rank's own, starting behind them
      const bool skip_own = !pull || p.ag_own_in_place;
      const int list_len = skip_own ? p.tiles_m - tiles_per_rank : p.tiles_m;
      const int first = (pull ? p.ag_rank + (skip_own ? 1 : 0) : p.rs_rank + 1) * tiles_per_rank;
      const int my_tiles = copier < list_len ? (list_len - copier + n_copiers - 1) / n_copiers : 0;
      const long long my_chunks = (long long)my_tiles * chunks_per_tile;
      const uint32_t ready_target = (uint32_t)p.tiles_n * 8u;   // 8 epilogue warps per output tile
      // chunk g of this CTA: tile g / chunks_per_tile of its list (consumption order), piece g % chunks_per_tile
      // (32-bit arithmetic: this thread is one serial instruction stream and 64-bit divisions cost it hundreds of cycles)
      auto locate = [&](long long g, int& m_blk, long long& off, uint32_t& bytes) {
        const uint32_t q = (uint32_t)g / (uint32_t)chunks_per_tile, r = (uint32_t)g - q * (uint32_t)chunks_per_tile;
        const int mi = copier + (int)q * n_copiers;
        m_blk = (mi + first) % p.tiles_m;
        off = (long long)r * CHUNK;
        bytes = (uint32_t)((tile_bytes - off) < CHUNK ? (tile_bytes - off) : CHUNK);
      };
      auto block_ready = [&](int m_blk) {
        uint32_t f;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(p.rs_ready + m_blk) : "memory");
        return f >= ready_target;
      };
      // pull: tile t of this CTA's list is complete in the gathered buffer -> its flag
      auto publish_tile = [&](long long t) {
        const int m_blk = (copier + (int)t * n_copiers + first) % p.tiles_m;
        fence_proxy_async_global();
        __threadfence();
        asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.ag_flags + m_blk), "r"(1u) : "memory");
      };
      // Loads run ahead of the stores, across tile boundaries.  A staging buffer is free for the next load once
      // the bulk store that drained it has READ it (wait_group.read), not once its writes have landed; whether a
      // tile's stores have landed is looked at LAG stores later, so nothing is waited for right after it was issued.
      long long loaded = 0, stored = 0, published = 0;
      long long ready_upto = pull ? my_chunks : 0;   // chunks below this index belong to blocks known to be complete
      bool ok = true;
      while (stored < my_chunks && ok) {
        const long long reusable = stored > PENDING ? stored - PENDING : 0;
        while (loaded < my_chunks && loaded < reusable + NBUF) {
          int m_blk; long long off; uint32_t bytes;
          locate(loaded, m_blk, off, bytes);
          if (loaded >= ready_upto) {
            // push mode, first chunk of a new block: go on only if the block is complete; if stores are still
            // owed, do those first and look again, else wait here (bounded)
            bool rdy = block_ready(m_blk);
            if (!rdy && stored == loaded) {
              const long long t0 = clock64();
              while (!(rdy = block_ready(m_blk))) {
                if (*abort_flag || clock64() - t0 > INCIN_WAIT_CLOCKS) {
                  *abort_flag = 1;
                  if (p.status) atomicCAS(p.status, 0, kStatusTimeoutPeer);
                  ok = false;
                  break;
                }
                __nanosleep(200);
              }
            }
            if (!rdy) break;
            fence_proxy_async_global();   // the block was written with ordinary stores; the bulk loads come after
            ready_upto = loaded + chunks_per_tile;
          }
          const int buf = (int)(loaded % NBUF);
          const char* src =
              pull ? reinterpret_cast<const char*>(p.ag_src[m_blk / tiles_per_rank]) + (long long)(m_blk % tiles_per_rank) * tile_bytes + off
                   : reinterpret_cast<const char*>(p.C) + (long long)m_blk * tile_bytes + off;
          mbar_expect_tx(&cbar[buf], bytes);
          bulk_load_1d(smem + buf * CHUNK, src, bytes, &cbar[buf]);
          ++loaded;
        }
        if (!ok || stored == loaded) continue;
        int m_blk; long long off; uint32_t bytes;
        locate(stored, m_blk, off, bytes);
        const int buf = (int)(stored % NBUF);
        if (!mbar_wait(&cbar[buf], (uint32_t)((stored / NBUF) & 1), abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
        char* dst = pull ? reinterpret_cast<char*>(p.ag_gathered) + (long long)m_blk * tile_bytes + off
                         : reinterpret_cast<char*>(p.rs_dst[m_blk / tiles_per_rank]) + p.rs_rank * p.rs_slot_stride * 2 +
                               (long long)(m_blk % tiles_per_rank) * tile_bytes + off;
        bulk_store_1d(dst, smem + buf * CHUNK, bytes);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        ++stored;
        asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
        if (pull) {
          // tiles whose last store is at least LAG stores old: those stores have landed after this wait
          while ((published + 1) * chunks_per_tile + LAG <= stored) {
            asm volatile("cp.async.bulk.wait_group %0;" ::"n"(LAG) : "memory");
            publish_tile(published++);
          }
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (pull) {
        while (ok && (published + 1) * chunks_per_tile <= stored) publish_tile(published++);
      } else {
        fence_proxy_async_global();
        __threadfence_system();   // pushed blocks are visible to their owners before the cross-GPU barrier that follows
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    // The whole warp walks the loop so that waits, loop control and coordinate arithmetic stay warp-uniform; one
    // elected lane issues the copies.
    const bool leader = elect_one() != 0;
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = cta; u < p.total_units && ok; u += n_compute) {
        const Unit w = decode_unit(p, u);
        const int m0 = w.m_blk * BM, n0 = w.n_blk * BN;
        if (p.ag_world > 1 && !(p.ag_own_in_place && w.m_blk / (p.ag_rows_per_rank / BM) == p.ag_rank)) {
          // the row block must have been gathered: bounded spin on its flag, then order the async proxy after it
          const long long t0 = clock64();
          uint32_t f = 0;
          for (;;) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(p.ag_flags + w.m_blk) : "memory");
            if (f >= p.ag_flag_target) break;
            if (*abort_flag || clock64() - t0 > INCIN_WAIT_CLOCKS) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0, kStatusTimeoutPeer);
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_global();
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const int k0 = kb * BK;
          if (leader) {
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_4d(sa, &tmA, &full_bar[stage], k0, m0, w.b_lo, w.b_hi);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_4d(sa + c * 8192, &tmA, &full_bar[stage], m0 + c * 64, k0, w.b_lo, w.b_hi);
          }
          if (!B_MN) {
            tma_load_4d(sb, &tmB, &full_bar[stage], k0, n0, w.b_lo, w.b_hi);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_4d(sb + c * 8192, &tmB, &full_bar[stage], n0 + c * 64, k0, w.b_lo, w.b_hi);
          }
          }
          __syncwarp();
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop (warp-uniform waits and descriptor arithmetic); one elected lane issues.
    const bool leader = elect_one() != 0;
    {
      // The issuing thread is latency critical (one dependent instruction stream feeding the tensor pipe), so the
      // operand kind is a compile-time constant of the loop: one copy of the loop per kind, chosen once.
      auto issue_all = [&](auto kind_tag) {
        constexpr int KIND = decltype(kind_tag)::value;
        constexpr uint32_t idesc_bf16 = make_idesc_bf16(BM, BN, A_MN, B_MN);
        constexpr uint32_t idesc = KIND == 0 ? idesc_bf16 : idesc_with_format(idesc_bf16, KIND == 2 ? 2u : 0u);
        // low / high halves of the shared-memory descriptors of stage 0 (LBO 16 for K-major, 8 KB for MN-major operands)
        const uint64_t a_desc0 = A_MN ? make_smem_desc(smem_u32(smem), 8192, 1024) : make_smem_desc(smem_u32(smem), 16, 1024);
        const uint32_t a_lo0 = static_cast<uint32_t>(a_desc0), desc_hi = static_cast<uint32_t>(a_desc0 >> 32);
        constexpr uint32_t lbo_k = (16u >> 4) << 16, lbo_mn = (8192u >> 4) << 16;
        const uint32_t b_lo_off = (Cfg::A_BYTES >> 4) + (B_MN ? lbo_mn : lbo_k) - (A_MN ? lbo_mn : lbo_k);
        int stage = 0;
        uint32_t phase = 0;
        int iter = 0;
        bool ok = true;
        for (int u = cta; u < p.total_units && ok; u += n_compute, ++iter) {
          const Unit w = decode_unit(p, u);
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
            if constexpr (KIND == 2) {
              const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
              const uint32_t sb = sa + Cfg::A_BYTES;
              const uint64_t adesc = make_smem_desc(sa, 16, 1024), bdesc = make_smem_desc(sb, 16, 1024);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                if (leader) umma_tf32_ss(d_tmem, adesc + (uint64_t)(k * 32 >> 4), bdesc + (uint64_t)(k * 32 >> 4), idesc,
                             (kb > w.kb0 || k > 0) ? 1u : 0u);
            } else {
              // descriptors: high halves are constants of the kernel, the low half is the stage's address field plus
              // the step inside the k-block (K-major: 16 elements = 32 B along the swizzle row; MN-major: 16 rows of
              // 128 B)
              const uint32_t a_lo = a_lo0 + stage * (Cfg::STAGE_BYTES >> 4), b_lo = a_lo + b_lo_off;
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                if (leader) umma_f16_ss_lohi(d_tmem, a_lo + (A_MN ? (k * 2048 >> 4) : (k * 32 >> 4)), desc_hi,
                                 b_lo + (B_MN ? (k * 2048 >> 4) : (k * 32 >> 4)), desc_hi, idesc,
                                 (kb > w.kb0 || k > 0) ? 1u : 0u);
            }
            if (leader) umma_commit(&empty_bar[stage]);  // slot is free once these MMAs have read it
            __syncwarp();
            if (++stage == n_stages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok && leader) umma_commit(&tfull_bar[acc]);  // accumulator complete
        }
      };
      if (p.in_kind == 0) issue_all(std::integral_constant<int, 0>{});
      else if (p.in_kind == 1) issue_all(std::integral_constant<int, 1>{});
      else issue_all(std::integral_constant<int, 2>{});
    }
  } else if (warp == GEMM_COPY_WARP) {
    // ------------------------------------------------------------- copy warp (fused collectives, copy-warp mode)
    // One lane of one extra warp in EVERY compute CTA moves a share of the collective's data in 8 KB bulk copies
    // global -> shared -> global.  What one SM can have in flight towards a peer is small (a dedicated copy CTA with
    // a 200 KB ring moves about 26 GB/s); spread over all SMs the same transfers need only a few operand stages of
    // shared memory per SM and take no SM away from the tensor-core work, and each byte still crosses NVLink once.
    //   all-gather:     chunk g of the tile list (consumption order) is pulled by CTA g % grid; a tile's flag counts
    //                   its completed chunks and the producer warps wait for ag_flag_target of them;
    //   reduce-scatter: chunk g of the list of remote row blocks is pushed by CTA g % grid once the block is complete
    //                   in the local staging buffer (rs_ready).
    // The ring is two halves: while the stores of one batch drain one half, the loads of the next batch fill the
    // other; completion (and the flags of a batch) is checked one batch late, so no copy is waited for right after it
    // was issued.  The warp waits only for its own copies and for epilogue counters, never for another copy warp, and
    // nothing but the producers' flag wait depends on it.
    if (p.copy_warps && lane == 0) {
      uint8_t* ring = smem + n_stages * Cfg::STAGE_BYTES;
      const int half_chunks = (Cfg::STAGES - n_stages) * Cfg::STAGE_BYTES / (2 * CW_CHUNK);
      const bool pull = p.ag_world > 1;
      const long long row_bytes = pull ? (long long)p.K * 2 : (long long)p.N * 2;
      const long long tile_bytes = (long long)BM * row_bytes;
      const int chunks_per_tile = (int)((tile_bytes + CW_CHUNK - 1) / CW_CHUNK);
      const int tiles_per_rank = (pull ? p.ag_rows_per_rank : p.rs_rows_per_rank) / BM;
      const bool skip_own = !pull || p.ag_own_in_place;     // push, or pull with the own shard already in place
      const int list_len = skip_own ? p.tiles_m - tiles_per_rank : p.tiles_m;
      const int first = (pull ? p.ag_rank + (skip_own ? 1 : 0) : p.rs_rank + 1) * tiles_per_rank;
      const long long total = (long long)list_len * chunks_per_tile;
      const long long n_mine = cta < total ? (total - cta + n_compute - 1) / n_compute : 0;
      const long long n_batches = (n_mine + half_chunks - 1) / half_chunks;
      const uint32_t ready_target = (uint32_t)p.tiles_n * 8u;   // 8 epilogue warps per output tile
      // 32-bit arithmetic on purpose: this lane is one serial instruction stream and a 64-bit division costs it
      // hundreds of cycles (total < 2^31 is checked on the host)
      auto locate = [&](long long i, int& m_blk, long long& off, uint32_t& bytes) {
        const uint32_t g = (uint32_t)cta + (uint32_t)i * (uint32_t)n_compute;
        const uint32_t q = g / (uint32_t)chunks_per_tile, r = g - q * (uint32_t)chunks_per_tile;
        uint32_t m = q + (uint32_t)first;
        if (m >= (uint32_t)p.tiles_m) m -= (uint32_t)p.tiles_m;
        m_blk = (int)m;
        off = (long long)r * CW_CHUNK;
        bytes = (uint32_t)((tile_bytes - off) < CW_CHUNK ? (tile_bytes - off) : CW_CHUNK);
      };
      int ready_blk = -1;       // push: the last block seen complete
      // loads of batch k into half k & 1 (push: once every block the batch touches is complete in the staging buffer)
      auto issue_loads = [&](long long k) -> bool {
        const long long i0 = k * half_chunks, i1 = (i0 + half_chunks < n_mine) ? i0 + half_chunks : n_mine;
        uint32_t sum = 0;
        for (long long i = i0; i < i1; ++i) {
          int m_blk; long long off; uint32_t bytes;
          locate(i, m_blk, off, bytes);
          sum += bytes;
          if (!pull && m_blk != ready_blk) {
            const long long t0 = clock64();
            for (;;) {
              uint32_t f;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(p.rs_ready + m_blk) : "memory");
              if (f >= ready_target) break;
              if (*abort_flag || clock64() - t0 > INCIN_WAIT_CLOCKS) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, kStatusTimeoutPeer);
                return false;
              }
              __nanosleep(200);
            }
            ready_blk = m_blk;
          }
        }
        if (!pull) fence_proxy_async_global();   // the blocks were written with ordinary stores; the bulk loads come after
        uint64_t* bar = &cw_bar[k & 1];
        uint8_t* half = ring + (k & 1) * half_chunks * CW_CHUNK;
        mbar_expect_tx(bar, sum);
        for (long long i = i0; i < i1; ++i) {
          int m_blk; long long off; uint32_t bytes;
          locate(i, m_blk, off, bytes);
          const char* src =
              pull ? reinterpret_cast<const char*>(p.ag_src[m_blk / tiles_per_rank]) + (long long)(m_blk % tiles_per_rank) * tile_bytes + off
                   : reinterpret_cast<const char*>(p.C) + (long long)m_blk * tile_bytes + off;
          bulk_load_1d(half + (i - i0) * CW_CHUNK, src, bytes, bar);
        }
        return true;
      };
      // all-gather: the chunks of batch k have landed in the gathered buffer.  One fence orders all of them before
      // the counts (a fence costs this thread more than a microsecond while the epilogue warps of its SM are storing,
      // so there is exactly one per batch and the counts themselves are relaxed).
      auto publish = [&](long long k) {
        const long long i0 = k * half_chunks, i1 = (i0 + half_chunks < n_mine) ? i0 + half_chunks : n_mine;
        fence_proxy_async_global();
        __threadfence();
        for (long long i = i0; i < i1; ++i) {
          int m_blk; long long off; uint32_t bytes;
          locate(i, m_blk, off, bytes);
          asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p.ag_flags + m_blk), "r"(1u) : "memory");
        }
      };
      bool ok = n_batches > 0 ? issue_loads(0) : true;
      long long done = 0;       // batches whose stores have been issued
      for (long long k = 0; k < n_batches && ok; ++k) {
        if (!mbar_wait(&cw_bar[k & 1], (uint32_t)((k >> 1) & 1), abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
        const long long i0 = k * half_chunks, i1 = (i0 + half_chunks < n_mine) ? i0 + half_chunks : n_mine;
        uint8_t* half = ring + (k & 1) * half_chunks * CW_CHUNK;
        for (long long i = i0; i < i1; ++i) {
          int m_blk; long long off; uint32_t bytes;
          locate(i, m_blk, off, bytes);
          char* dst = pull ? reinterpret_cast<char*>(p.ag_gathered) + (long long)m_blk * tile_bytes + off
                           : reinterpret_cast<char*>(p.rs_dst[m_blk / tiles_per_rank]) + p.rs_rank * p.rs_slot_stride * 2 +
                                 (long long)(m_blk % tiles_per_rank) * tile_bytes + off;
          bulk_store_1d(dst, half + (i - i0) * CW_CHUNK, bytes);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        done = k + 1;
        if (k + 1 < n_batches) {
          // the other half is free once the stores of batch k - 1 have read it
          if (k >= 1) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          ok = issue_loads(k + 1);
        }
        if (pull && k >= 1) {
          asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");   // batch k - 1 has landed (batch k stays in flight)
          publish(k - 1);
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (pull) {
        if (done >= 1) publish(done - 1);
      } else {
        fence_proxy_async_global();
        __threadfence_system();   // pushed blocks are visible to their owners before the cross-GPU barrier that follows
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (8 warps: 4 lane quarters x 2 column halves)
    const int quarter = warp & 3;  // TMEM lanes a warp may touch: 32 * (warp % 4)
    const int half = (warp - 2) >> 2;
    const float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
    constexpr int CHUNKS_PER_HALF = BN / 64;
    const int row_in_tile = quarter * 32 + lane;
    int iter = 0;
    for (int u = cta; u < p.total_units; u += n_compute, ++iter) {
      const Unit w = decode_unit(p, u);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, kStatusTimeoutTmemFull)) break;
      tc_fence_after();
      const int m = w.m_blk * BM + row_in_tile;
      const int n0 = w.n_blk * BN;
      const bool row_ok = m < p.M;
      long long cbase = (long long)w.b_lo * p.c_stride_lo + (long long)w.b_hi * p.c_stride_hi +
                        (long long)m * p.ldc;
      void* c_ptr = p.C;
      if (p.rs_world > 1) {
        // reduce-scatter: this tile belongs to `owner`; write it into this rank's slot of the owner's buffer
        // (push mode: only when this rank owns it; other tiles stay in the local staging buffer C for the copy CTAs)
        const int owner = (w.m_blk * BM) / p.rs_rows_per_rank;
        if (!p.rs_push || owner == p.rs_rank) {
          c_ptr = p.rs_dst[owner];
          cbase = (long long)p.rs_rank * p.rs_slot_stride + (long long)(m - owner * p.rs_rows_per_rank) * p.ldc;
        }
      }
      const bool vec_ok = (p.ldc % 8 == 0) && (p.c_stride_lo % 8 == 0) && (p.c_stride_hi % 8 == 0);
      if (STG && p.tma_out) {
        // the two warps of a lane quarter split the tile's columns in multiples of 64: 128 + 128, 128 + 64, 64 + 64, 64 + 0
        constexpr int COLS0 = (BN / 64 + 1) / 2 * 64;
        const int col_first = half ? COLS0 : 0, ncols = half ? BN - COLS0 : COLS0;
        epilogue_staged(p, &tmC, &tmAux, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * Cfg::ACC_STRIDE + col_first,
                        smem + Cfg::STG_OFF + (warp - 2) * STG_WARP_BYTES, w.m_blk * BM + quarter * 32, n0 + col_first, ncols,
                        w.b_lo, w.b_hi, cbase, row_ok, alpha, lane);
      } else {
#pragma unroll 1
      for (int c = half * CHUNKS_PER_HALF; c < (half + 1) * CHUNKS_PER_HALF; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * Cfg::ACC_STRIDE + c * 32, r);
        tmem_ld_wait();
        const int nc = n0 + c * 32;
        if (row_ok && nc < p.N) epilogue_chunk(p, r, c_ptr, cbase, nc, vec_ok, alpha);
        __syncwarp();  // tcgen05.ld is warp-collective: reconverge before the next chunk
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[acc]);
        if (p.rs_push) {
          // this warp's part of the tile is in the staging buffer: count it for the copiers.  The release of the
          // count orders the warp's stores (made visible to this lane by the __syncwarp above) before it; a separate
          // fence in front of it showed up as a fifth of all warp stalls of this launch.
          asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.rs_ready + w.m_blk), "r"(1u) : "memory");
        }
      }
    }
    if (STG && p.tma_out && p.out_fp32 && lane == 0) bulk_wait_all();   // this warp's staged boxes have been written before the CTA retires
  }

  // common exit: every thread arrives here, also after a timed-out wait
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the CTA retires
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// Tensor map over a bf16 operand: dims {inner, rows, batch_lo, batch_hi}, strides in elements.
int make_operand_map(CUtensorMap* out, const void* ptr, long long inner, long long rows, long long ld,
                     long long batch_lo, long long stride_lo, long long batch_hi, long long stride_hi, int box_inner,
                     int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return INCIN_ERR_DRIVER;
  // cuTensorMapEncodeTiled is a driver call and needs a current context on the calling thread.  Autograd
  // worker threads can reach this point before any runtime call has bound the primary context.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld % 8) || (batch_lo > 1 && stride_lo % 8) ||
      (batch_hi > 1 && stride_hi % 8))
    return INCIN_ERR_ALIGNMENT;
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch_lo, (cuuint64_t)batch_hi};
  // strides of dims 1..3 in bytes; a unit batch dimension still needs a legal (multiple of 16) stride
  cuuint64_t strides[3] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch_lo > 1 ? stride_lo : ld * rows) * 2,
                           (cuuint64_t)(batch_hi > 1 ? stride_hi : ld * rows) * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? INCIN_OK : INCIN_ERR_TENSOR_MAP;
}

// Tensor map over an fp32 tensor for tiled reduce-adds from 128-byte swizzled shared memory: dims {inner, rows,
// batch_lo, batch_hi}, strides in elements; box = {32 columns (128 bytes), box_rows, 1, 1}.
int make_f32_reduce_map(CUtensorMap* out, void* ptr, long long inner, long long rows, long long ld, long long batch_lo,
                        long long stride_lo, long long batch_hi, long long stride_hi, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return INCIN_ERR_DRIVER;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld % 4) || (batch_lo > 1 && stride_lo % 4) || (batch_hi > 1 && stride_hi % 4))
    return INCIN_ERR_ALIGNMENT;   // (a box that reaches past `inner` or `rows` is clipped, so neither needs to be a multiple of the box)
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch_lo, (cuuint64_t)batch_hi};
  cuuint64_t strides[3] = {(cuuint64_t)ld * 4, (cuuint64_t)(batch_lo > 1 ? stride_lo : ld * rows) * 4,
                           (cuuint64_t)(batch_hi > 1 ? stride_hi : ld * rows) * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? INCIN_OK : INCIN_ERR_TENSOR_MAP;
}

static int g_num_sms = 0;
int device_sm_count() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, bool A_MN, bool B_MN, bool STG>
static int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
                      const GemmKernelParams& p, int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, STG>;
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, STG>;
  static PerDeviceFlags attr_set;
  if (!ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, attr_set)) return INCIN_ERR_LAUNCH;
  int grid = p.total_units < max_ctas ? p.total_units : max_ctas;
  GemmKernelParams q = p;
  if ((p.ag_world > 1 || p.rs_push) && !p.copy_warps) {
    int copy = p.gemm_ctas;   // the caller's request for copy CTAs travels in gemm_ctas until here
    if (copy < 1) copy = 8;
    if (copy > max_ctas / 2) copy = max_ctas / 2;
    int compute = max_ctas - copy;
    if (compute > p.total_units) compute = p.total_units;
    q.gemm_ctas = compute;
    grid = compute + copy;
  }
  // fused-collective launches wait on other GPUs: those stay ordinary launches
  if (q.ag_world > 1 || q.rs_world > 1) {
    kern<<<grid, q.copy_warps ? GEMM_THREADS_COPY : GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, tc, tx, q);
    return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
  }
  return launch_pdl<true>(kern, dim3(grid), dim3(GEMM_THREADS), Cfg::SMEM_BYTES, stream, ta, tb, tc, tx, q) == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

template <int BN>
static int launch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                        const CUtensorMap& tx, const GemmKernelParams& p, int max_ctas, cudaStream_t s) {
  // 128 x 256 tiles always carry the staging area (it costs them no operand stage); the others only when asked to
  if (p.tma_out || BN == 256) {
    if (!a_mn && !b_mn) return launch_cfg<BN, false, false, true>(ta, tb, tc, tx, p, max_ctas, s);
    if (!a_mn && b_mn) return launch_cfg<BN, false, true, true>(ta, tb, tc, tx, p, max_ctas, s);
    if (a_mn && !b_mn) return launch_cfg<BN, true, false, true>(ta, tb, tc, tx, p, max_ctas, s);
    return launch_cfg<BN, true, true, true>(ta, tb, tc, tx, p, max_ctas, s);
  }
  if (!a_mn && !b_mn) return launch_cfg<BN, false, false, false>(ta, tb, tc, tx, p, max_ctas, s);
  if (!a_mn && b_mn) return launch_cfg<BN, false, true, false>(ta, tb, tc, tx, p, max_ctas, s);
  if (a_mn && !b_mn) return launch_cfg<BN, true, false, false>(ta, tb, tc, tx, p, max_ctas, s);
  return launch_cfg<BN, true, true, false>(ta, tb, tc, tx, p, max_ctas, s);
}

// CTA-pair kernel launch: as many clusters as the device can hold at once (at most one CTA per SM).
template <bool A_MN, bool B_MN, bool STG>
static int launch_pair_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
                           const GemmKernelParams& p, int tiles_m2, int max_ctas, cudaStream_t stream) {
  using PCfg = PairCfg<STG>;
  auto kern = gemm_tcgen05_pair_kernel<A_MN, B_MN, STG>;
  static PerDeviceFlags attr_set;
  if (!ensure_dynamic_smem(kern, PCfg::SMEM_BYTES, attr_set)) return INCIN_ERR_LAUNCH;
  static int max_clusters = 0;   // the same for every B200 of a node
  if (max_clusters == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = PCfg::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      return INCIN_ERR_LAUNCH;
    }
    max_clusters = n;
  }
  int pairs = max_clusters < max_ctas / 2 ? max_clusters : max_ctas / 2;
  if (pairs > p.total_units) pairs = p.total_units;
  if (pairs < 1) return INCIN_ERR_ARGUMENT;
  return launch_pdl<true>(kern, dim3(2 * pairs), dim3(GEMM_THREADS), PCfg::SMEM_BYTES, stream, ta, tb, tc, tx, p, tiles_m2) == cudaSuccess
             ? INCIN_OK
             : INCIN_ERR_LAUNCH;
}

static int launch_pair(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                       const CUtensorMap& tx, const GemmKernelParams& p, int tiles_m2, int max_ctas, cudaStream_t s) {
  if (p.tma_out) {
    if (!a_mn && !b_mn) return launch_pair_cfg<false, false, true>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
    if (!a_mn && b_mn) return launch_pair_cfg<false, true, true>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
    if (a_mn && !b_mn) return launch_pair_cfg<true, false, true>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
    return launch_pair_cfg<true, true, true>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
  }
  if (!a_mn && !b_mn) return launch_pair_cfg<false, false, false>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
  if (!a_mn && b_mn) return launch_pair_cfg<false, true, false>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
  if (a_mn && !b_mn) return launch_pair_cfg<true, false, false>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
  return launch_pair_cfg<true, true, false>(ta, tb, tc, tx, p, tiles_m2, max_ctas, s);
}

// Pick the tile and the split-K factor that minimise a cost model fitted to per-launch CUDA-event timings on a B200
// (L2 flushed before every launch; 18 shapes x 5 tiles x up to 4 split factors, candidates interleaved):
//     time = fixed(tile) + waves x k_blocks_per_split x step(tile) + split penalty
// step(tile) is the microseconds one 64-deep k-block costs a CTA when every SM is busy.  It is set by the operand
// traffic from L2 (all tiles sustain about 14 TB/s in aggregate, the CTA pair about 10.5 TB/s), so it grows more
// slowly than the tile: wider tiles do more work per byte.  fixed(tile) is prologue plus the tail epilogue, which
// grows with the tile; the pair pays for its cluster launch and two cluster-wide syncs.  A last wave that fills only
// part of the machine is cheaper than a full one because its CTAs contend less for L2.
struct TileChoice {
  int bn;       // 64 / 128 / 192 / 256, or 512 for the 256 x 256 tile of a CTA pair
  int splits;
};

static double waves_cost(long long units, int slots) {
  const long long full = units / slots;
  const double part = static_cast<double>(units % slots) / slots;
  return static_cast<double>(full) + (part > 0.0 ? 0.55 + 0.45 * part : 0.0);
}

static TileChoice choose_tile(long long M, long long N, long long K, long long batch, int fixed_bn, int fixed_splits,
                              bool may_split, bool may_pair, int sms) {
  static const int kBn[5] = {64, 128, 192, 256, 512};
  static const double kStep[5] = {0.370, 0.395, 0.420, 0.498, 0.452};
  static const double kFixed[5] = {10.0, 11.4, 13.6, 16.0, 21.0};
  static const int kSplits[7] = {1, 2, 3, 4, 5, 6, 8};
  const long long kb = (K + BK - 1) / BK;
  TileChoice best = {128, 1};
  double best_cost = 1e30;
  for (int t = 0; t < 5; ++t) {
    const int bn = kBn[t];
    if (fixed_bn > 0 && bn != fixed_bn) continue;
    const bool pair = bn == 512;
    if (pair && (!may_pair || sms < 148 || (fixed_bn != 512 && (M < 512 || N < 512)))) continue;
    const long long tiles = pair ? ((M + 255) / 256) * ((N + 255) / 256) * batch
                                 : ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * batch;
    const int slots = pair ? sms / 2 : sms;
    for (int si = 0; si < 7; ++si) {
      const int sp = kSplits[si];
      if (fixed_splits > 0 ? sp != fixed_splits : (sp > 1 && (!may_split || kb / sp < 4))) continue;
      const long long kbs = (kb + sp - 1) / sp;
      const double cost = kFixed[t] + waves_cost(tiles * sp, slots) * static_cast<double>(kbs) * kStep[t] + 1.5 * (sp - 1);
      if (cost < best_cost) {
        best_cost = cost;
        best.bn = bn;
        best.splits = sp;
      }
    }
  }
  if (fixed_splits > 0) best.splits = fixed_splits;
  return best;
}

}  // namespace incin

using namespace incin;

extern "C" int incin_gemm_bf16(const incin_gemm_desc* d, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!d || !d->A || !d->B || (!d->C && d->rs_world <= 1) || d->M <= 0 || d->N <= 0 || d->K <= 0) return INCIN_ERR_ARGUMENT;
  // Other operand types.  fp16 changes only the format field of the instruction.  fp32 operands are multiplied as
  // tf32: a row of fp32 is moved by the same tensor maps as a row of twice as many 2-byte units (the 128-byte swizzle
  // works on 16-byte chunks), so from here on K and the operand strides count 2-byte units; only the instruction kind
  // differs (8 fp32 = the same 32 bytes per product).  Both write fp32 and take no fused epilogue or collective.
  incin_gemm_desc widened;
  const int in_kind = d->in_dtype;
  if (in_kind != INCIN_GEMM_IN_BF16) {
    if ((in_kind != INCIN_GEMM_IN_FP16 && in_kind != INCIN_GEMM_IN_TF32) || !d->out_fp32 || d->bias || d->residual ||
        d->aux || d->act != INCIN_ACT_NONE || d->ag_world > 1 || d->rs_world > 1 || d->tile_n == 512)
      return INCIN_ERR_ARGUMENT;
    if (in_kind == INCIN_GEMM_IN_TF32) {
      if (d->a_mn_major || d->b_mn_major) return INCIN_ERR_ARGUMENT;   // K-contiguous operands only
      widened = *d;
      widened.K *= 2;
      widened.lda *= 2;
      widened.ldb *= 2;
      widened.a_stride_lo *= 2;
      widened.a_stride_hi *= 2;
      widened.b_stride_lo *= 2;
      widened.b_stride_hi *= 2;
      d = &widened;
    }
  }
  const int blo = d->batch_lo > 0 ? d->batch_lo : 1;
  const int bhi = d->batch_hi > 0 ? d->batch_hi : 1;
  const int sms = d->max_ctas > 0 ? d->max_ctas : device_sm_count();
  // splits == 0 asks for the split-K factor to be chosen together with the tile (fp32 accumulating outputs only)
  const bool can_split = d->out_fp32 && d->accumulate && !d->bias && !d->residual && d->act == INCIN_ACT_NONE &&
                         d->ag_world <= 1 && d->rs_world <= 1;
  const int kb_total = (d->K + BK - 1) / BK;
  int splits = d->splits > 0 ? d->splits : (can_split ? 0 : 1);
  if (splits > kb_total) splits = kb_total;
  if (splits > 1 && !(d->out_fp32 && d->accumulate)) return INCIN_ERR_ARGUMENT;
  if (splits > 1 && (d->bias || d->residual || d->act != INCIN_ACT_NONE)) return INCIN_ERR_ARGUMENT;
  if ((d->act == INCIN_ACT_DGELU || d->act == INCIN_ACT_DSILU) && !d->aux) return INCIN_ERR_ARGUMENT;
  const bool fused_collective = d->ag_world > 1 || d->rs_world > 1;
  int bn = d->tile_n;
  if (bn != 64 && bn != 128 && bn != 192 && bn != 256 && bn != 512) bn = 0;
  if (bn == 512 && fused_collective) bn = 0;
  const incin::TileChoice pick = incin::choose_tile(d->M, d->N, d->K, (long long)blo * bhi, bn, splits, can_split,
                                                    !fused_collective && in_kind == INCIN_GEMM_IN_BF16, sms);
  bn = pick.bn;
  splits = pick.splits;
  const bool pair = bn == 512;
  const int b_box = pair ? 128 : bn;                      // B rows one CTA loads per k-block

  CUtensorMap ta, tb;
  int rc;
  if (!d->a_mn_major)
    rc = make_operand_map(&ta, d->A, d->K, d->M, d->lda, blo, d->a_stride_lo, bhi, d->a_stride_hi, BK, BM);
  else
    rc = make_operand_map(&ta, d->A, d->M, d->K, d->lda, blo, d->a_stride_lo, bhi, d->a_stride_hi, 64, BK);
  if (rc != INCIN_OK) return rc;
  if (!d->b_mn_major)
    rc = make_operand_map(&tb, d->B, d->K, d->N, d->ldb, blo, d->b_stride_lo, bhi, d->b_stride_hi, BK, b_box);
  else
    rc = make_operand_map(&tb, d->B, d->N, d->K, d->ldb, blo, d->b_stride_lo, bhi, d->b_stride_hi, 64, BK);
  if (rc != INCIN_OK) return rc;

  GemmKernelParams p;
  p.M = d->M;
  p.N = d->N;
  p.K = d->K;
  p.batch_lo = blo;
  p.batch_hi = bhi;
  p.tiles_m = (d->M + BM - 1) / BM;
  p.tiles_n = pair ? (d->N + 255) / 256 : (d->N + bn - 1) / bn;
  p.splits = splits;
  const int tiles_m2 = (d->M + 255) / 256;
  const long long units = (long long)(pair ? tiles_m2 : p.tiles_m) * p.tiles_n * blo * bhi * splits;
  if (units > 0x7fffffffLL) return INCIN_ERR_ARGUMENT;
  p.total_units = (int)units;
  p.C = d->C;
  p.ldc = d->ldc;
  p.c_stride_lo = d->c_stride_lo;
  p.c_stride_hi = d->c_stride_hi;
  p.out_fp32 = d->out_fp32;
  p.accumulate = d->accumulate;
  p.alpha = d->alpha;
  p.alpha_ptr = reinterpret_cast<const float*>(d->alpha_ptr);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(d->bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(d->residual);
  p.act = d->act;
  p.aux = reinterpret_cast<__nv_bfloat16*>(d->aux);
  p.status = reinterpret_cast<int*>(d->status);
  p.in_kind = in_kind;
  static const int wide_io = [] {
    const char* e = std::getenv("INCIN_GEMM_B256");
    return e ? std::atoi(e) : 1;
  }();
  p.wide_io = wide_io;
  p.ag_world = d->ag_world > 1 ? d->ag_world : 0;
  p.ag_own_in_place = 0;
  p.ag_rank = d->ag_rank;
  p.ag_rows_per_rank = d->ag_rows_per_rank;
  p.gemm_ctas = d->ag_world > 1 ? d->ag_copy_ctas : d->rs_copy_ctas;
  p.ag_flags = reinterpret_cast<uint32_t*>(d->ag_flags);
  p.ag_gathered = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(d->A));
  p.rs_world = d->rs_world > 1 ? d->rs_world : 0;
  p.rs_rank = d->rs_rank;
  p.rs_rows_per_rank = d->rs_rows_per_rank;
  p.rs_slot_stride = d->rs_slot_stride;
  p.rs_ready = reinterpret_cast<uint32_t*>(d->rs_ready);
  p.rs_push = (p.rs_world && d->rs_copy_ctas != 0 && d->rs_ready) ? 1 : 0;
  // a negative count of copy CTAs asks for copy warps: one extra warp in every compute CTA moves the data
  // (-n: n operand stages of shared memory become the copy ring; at least three stages stay with the GEMM)
  p.copy_warps = p.ag_world ? (d->ag_copy_ctas < 0 ? -d->ag_copy_ctas : 0) : ((p.rs_push && d->rs_copy_ctas < 0) ? -d->rs_copy_ctas : 0);
  p.ag_flag_target = 1;
  if (p.ag_world && p.copy_warps) p.ag_flag_target = (uint32_t)(((long long)BM * d->K * 2 + 8 * 1024 - 1) / (8 * 1024));
  for (int r = 0; r < 8; ++r) {
    p.ag_src[r] = reinterpret_cast<const __nv_bfloat16*>(d->ag_src[r]);
    p.rs_dst[r] = reinterpret_cast<__nv_bfloat16*>(d->rs_dst[r]);
  }
  if (p.ag_world) {
    if (p.ag_world > 8 || d->a_mn_major || d->lda != d->K || (d->K % 8) || p.ag_rows_per_rank % BM ||
        d->M != p.ag_world * p.ag_rows_per_rank || !p.ag_flags || splits != 1 || blo * bhi != 1)
      return INCIN_ERR_ARGUMENT;
    // a NULL source for this rank's own shard: the caller has already placed those rows in the gathered buffer
    p.ag_own_in_place = p.ag_src[p.ag_rank] ? 0 : 1;
    for (int r = 0; r < p.ag_world; ++r)
      if (!p.ag_src[r] && r != p.ag_rank) return INCIN_ERR_ARGUMENT;
  }
  if (p.rs_world) {
    if (p.rs_world > 8 || d->out_fp32 || p.rs_rows_per_rank % BM || d->M != p.rs_world * p.rs_rows_per_rank ||
        splits != 1 || blo * bhi != 1 || d->residual || d->aux || p.ag_world)
      return INCIN_ERR_ARGUMENT;
    // push mode moves whole 128-row blocks of the staging buffer with bulk copies: rows must be dense and 16-byte sized
    if (p.rs_push && (!d->C || d->ldc != d->N || (d->N % 8))) return INCIN_ERR_ARGUMENT;
    for (int r = 0; r < p.rs_world; ++r)
      if (!p.rs_dst[r]) return INCIN_ERR_ARGUMENT;
  }

  // Output through staged bulk tensor stores where C (and the side output) can be described by a tensor map: 16-byte
  // aligned base and row / batch strides, results written to this GPU's memory (the reduce-scatter modes keep their
  // per-thread stores to peers).  INCIN_GEMM_TMA_OUT is a mask of the output kinds that take the staged path:
  // 1 = bf16 without side output, 2 = bf16 with the pre-activation side output, 4 = fp32 (plain and accumulating),
  // 8 = also for long reductions (otherwise only K / splits <= 1024 and the 128 x 256 tile, whose staging area costs
  // no operand stage).  Default 4.  Measured on one B200: staging bf16 outputs makes an isolated K = 768 product with a
  // cold L2 14 % faster (the epilogue of a 128 x 256 tile drops from about 6 us), but inside the captured GPT-2 training
  // step, where operands come from a warm L2 and the main loop is bound by shared-memory bandwidth, the extra 64 KB of
  // shared-memory traffic per tile made the step 0.3-0.6 ms (3-5 %) slower, with bulk tensor stores and with row-wise
  // stores alike; accumulating fp32 outputs through bulk reduce-adds were 0.05-0.09 ms faster.
  static const int tma_out_mask = [] {
    const char* e = std::getenv("INCIN_GEMM_TMA_OUT");
    return e ? std::atoi(e) : INCIN_GEMM_TMA_OUT_DEFAULT;
  }();
  const bool with_pre = d->aux && (d->act == INCIN_ACT_GELU || d->act == INCIN_ACT_SILU);
  const int out_kind = d->out_fp32 ? 4 : (with_pre ? 2 : 1);
  const bool tma_out_on = (tma_out_mask & out_kind) != 0;
  const bool tma_out_all = (tma_out_mask & 8) != 0;
  CUtensorMap tc = ta, tx = ta;
  p.tma_out = 0;
  const bool short_k = (kb_total + splits - 1) / splits <= 16;
  if (tma_out_on && !p.rs_world && d->C && (short_k || bn == 256 || tma_out_all)) {
    if (d->out_fp32) {
      p.tma_out = (!with_pre && make_f32_reduce_map(&tc, d->C, d->N, d->M, d->ldc, blo, d->c_stride_lo, bhi, d->c_stride_hi, 32) == INCIN_OK) ? 1 : 0;
    } else {   // bf16 rows leave with 16-byte stores: C (and the side output) 16-byte aligned with strides in multiples of 8
      const bool ok16 = !(reinterpret_cast<uintptr_t>(d->C) & 15) && (!with_pre || !(reinterpret_cast<uintptr_t>(d->aux) & 15)) &&
                        d->ldc % 8 == 0 && (blo == 1 || d->c_stride_lo % 8 == 0) && (bhi == 1 || d->c_stride_hi % 8 == 0);
      p.tma_out = ok16 ? 1 : 0;
    }
  }

  if (p.copy_warps) {
    // the copy warps index chunks with 32-bit arithmetic
    if ((long long)p.tiles_m * (((long long)BM * (p.ag_world ? d->K : d->N) * 2 + 8191) / 8192) > 0x3fffffffLL) return INCIN_ERR_ARGUMENT;
    const int stages = (224 * 1024 - ((p.tma_out || bn == 256) ? 32 * 1024 : 0)) / ((BM + bn) * BK * 2);
    if (p.copy_warps > stages - 3) p.copy_warps = stages - 3;
    if (p.copy_warps < 1) return INCIN_ERR_ARGUMENT;
  }
  const bool amn = d->a_mn_major != 0, bmn = d->b_mn_major != 0;
  if (pair) return incin::launch_pair(amn, bmn, ta, tb, tc, tx, p, tiles_m2, sms, stream);
  int rc2;
  if (bn == 64) rc2 = incin::launch_major<64>(amn, bmn, ta, tb, tc, tx, p, sms, stream);
  else if (bn == 128) rc2 = incin::launch_major<128>(amn, bmn, ta, tb, tc, tx, p, sms, stream);
  else if (bn == 192) rc2 = incin::launch_major<192>(amn, bmn, ta, tb, tc, tx, p, sms, stream);
  else rc2 = incin::launch_major<256>(amn, bmn, ta, tb, tc, tx, p, sms, stream);
  return rc2;
}
