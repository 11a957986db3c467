// Attention backward for head_dim 64 with the query tile split in two halves, so that the tensor core and the
// softmax-gradient threads work at the same time.
//
// One CTA owns a 128-row KV tile and walks the query tiles at or below the diagonal, as in flash_bwd_kernel.  Each
// 128-query tile is handled as halves a and b (64 queries each):
//
//   tensor core : S_a dP_a (i) | dV dK dQ (i-1) | S_b dP_b (i) | S_a dP_a (i+1) | ...
//   compute     :      ...  half b (i-1) | half a (i)      | half b (i)   | half a (i+1) ...
//
// The score MMAs of half a of tile i only need the S_a / dP_a columns of tensor memory, which the compute threads
// have finished reading once half a of tile i-1 is done; so while they work on half b, the next half a is already
// being produced, and while they work on half a of tile i the tensor core runs the three gradient products of
// tile i-1.  The shared-memory copy of P^T / dS^T that those products read is therefore still in use when half a of
// the next tile is written: half a is double buffered, half b is not (it is rewritten only after the products that
// read it have been committed).  Buffers sit in shared memory as [a0][b][a1], which lets the dQ product, whose A
// operand is dS in MN-major form with a fixed positive stride between its two 64-query chunks, read (a0, b) for even
// tiles and (b, a1) for odd tiles; for odd tiles the rows of the dQ partial are then the query rows rotated by 64,
// which the drain undoes.
//
// The kernel is persistent: one CTA per SM walks a list of (KV tile, KV head, batch) items, longest first and in
// snake order over the CTAs, so barrier set-up and the tensor-memory allocation are paid once per SM instead of once
// per item (measured at about 10 us per item before), and the causal imbalance between KV tiles evens out.
//
// Tensor memory (512 columns): S^T a|b [0,128), dP^T a|b [128,256), dV [256,320), dK [320,384), dQ partial x2
// [384,512).  All waits are bounded; a timed-out wait unwinds through the common exit.
#pragma once

namespace incin {

struct Fb64 {
  static constexpr int D = 64;
  static constexpr int H = 64;                          // queries per half
  static constexpr int ST = 2;                          // Q / dO stages
  static constexpr int TILE_BYTES = FB_T * D * 2;       // 16 KB: K, V, Q, dO tiles
  static constexpr int CHUNK_BYTES = FB_T * H * 2;      // 16 KB: one half of P^T or dS^T ([128 kv][64 q])
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_Q = 2 * TILE_BYTES;
  static constexpr int OFF_DO = OFF_Q + ST * TILE_BYTES;
  static constexpr int OFF_P = OFF_DO + ST * TILE_BYTES;      // [a0][b][a1]
  static constexpr int OFF_DS = OFF_P + 3 * CHUNK_BYTES;      // [a0][b][a1]
  static constexpr int OFF_STAT = OFF_DS + 3 * CHUNK_BYTES;   // lse[128], delta[128] per stage
  static constexpr int OFF_DQS = OFF_STAT + ST * 2 * FB_T * 4;   // dQ staging: two [128 q][32 fp32] boxes, SWIZZLE_128B
  static constexpr int DQS_BYTES = FB_T * 32 * 4;
  static constexpr int OFF_BAR = OFF_DQS + 2 * DQS_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;                // the window itself is declared 1024-byte aligned
  static_assert(OFF_DQS % 1024 == 0 && SMEM_BYTES <= 227 * 1024, "shared-memory plan");
  static constexpr int COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 320, COL_DQ = 384, TMEM_COLS = 512;
  // byte offset of half h of tile `it` inside a [a0][b][a1] triple
  __device__ static constexpr int chunk_off(int h, int it) { return h ? CHUNK_BYTES : ((it & 1) ? 2 * CHUNK_BYTES : 0); }
};

// PROF: add up clock intervals of the issuing thread and of one compute lane into p.prof (a second instantiation, so
// that the production kernel carries no clock reads).
template <bool PROF>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ FbParams p) {
  using Cfg = Fb64;
  constexpr int D = Cfg::D, ST = Cfg::ST, H = Cfg::H;
  // The plan fills the 227 KB an SM offers, so there is no room to round the base up: the window is declared aligned
  // and the kernel refuses to run (status word, nothing touched) should the base ever not be.
  extern __shared__ __align__(1024) uint8_t smem_aligned[];
  uint8_t* smem = smem_aligned;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kStatusBadArgument);
    return;
  }
  auto now = [] () -> long long {
    if constexpr (PROF) return clock64();
    else return 0ll;
  };
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint8_t* sDS = smem + Cfg::OFF_DS;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;          // 1
  uint64_t* q_full = bars + 1;       // [2]  Q_i, dO_i and their statistics landed
  uint64_t* q_empty = bars + 3;      // [2]  the MMAs that read that stage finished
  uint64_t* sdp = bars + 5;          // [2]  half a / half b of S^T and dP^T are in tensor memory
  uint64_t* pds = bars + 7;          // [2]  half a / half b of P^T and dS^T are in shared memory (one arrival per warp)
  uint64_t* dq_full = bars + 9;      // [2]  dQ partial buffer written (and dV / dK updated)
  uint64_t* dq_drained = bars + 11;  // [2]  dQ partial buffer read out (one arrival per warp)
  uint64_t* kv_empty = bars + 13;    // every product of the current item has been committed: K / V may be replaced
  uint64_t* dkv_drained = bars + 14; // dK / dV of the current item have been read out (one arrival per warp)
  uint64_t* stg_free = bars + 15;    // [2]  per compute group: the previous bulk reduce has read the dQ staging box
  uint64_t* stg_full = bars + 17;    // [2]  per compute group: all 8 warps have written their part of the box
  uint8_t* sDQS = smem + Cfg::OFF_DQS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.Hq / p.Hkv;
  const int heads_batches = p.Hkv * p.batch;
  const int n_items = p.n_tiles * heads_batches;
  // item list: KV tile 0 (most query tiles) first; round r of CTA c takes item r*G + c (even r) or (r+1)*G - 1 - c
  // (odd r), which pairs long and short items on every CTA.  Returns false when this CTA has no item in round r.
  auto item_of = [&](int r, int& kv_tile, int& hkv, int& b) -> bool {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int idx = (r & 1) ? (r + 1) * G - 1 - c : r * G + c;
    if (idx >= n_items) return false;
    kv_tile = idx / heads_batches;
    const int hb = idx % heads_batches;
    hkv = hb % p.Hkv;
    b = hb / p.Hkv;
    return true;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&sdp[s], 1);
      mbar_init(&pds[s], FB_CWARPS / 2);   // each half is produced by its own group of 8 warps
      mbar_init(&dq_full[s], 1);
      mbar_init(&dq_drained[s], FB_CWARPS);
    }
    mbar_init(kv_empty, 1);
    mbar_init(dkv_drained, FB_CWARPS);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&stg_free[s], 1);
      mbar_init(&stg_full[s], FB_CWARPS / 2);
    }
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&p.tm_dq);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();   // tensor memory is held
  pdl_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // (the whole warp walks the loop: warp-uniform waits and address arithmetic; one elected lane issues the copies)
    const bool leader = elect_one() != 0;
    {
      int base = 0;   // query tiles handed to the pipeline so far (all roles count the same way)
      bool ok = true;
      for (int r = 0; ok; ++r) {
        int kv_tile, hkv, b;
        if (!item_of(r, kv_tile, hkv, b)) break;
        const int kv0 = kv_tile * FB_T;
        const int tiles_per_head = p.n_tiles - kv_tile;
        const int n_iters = tiles_per_head * group;
        // K / V of the previous item are still operands until its last product has been committed
        if (r > 0 && !mbar_wait(kv_empty, (r - 1) & 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        if (leader) {
          mbar_expect_tx(kv_full, 2 * Cfg::TILE_BYTES);
          tma_load_4d(sK, &tmK, kv_full, 0, kv0, hkv, b);
          tma_load_4d(sV, &tmV, kv_full, 0, kv0, hkv, b);
        }
        for (int it = 0; it < n_iters; ++it) {
          const int g = base + it, s = g % ST;
          const int hq = hkv * group + it / tiles_per_head;
          const int q0 = (kv_tile + it % tiles_per_head) * FB_T;
          if (!mbar_wait(&q_empty[s], ((g / ST) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          if (leader) {
            mbar_expect_tx(&q_full[s], 2 * Cfg::TILE_BYTES + 2 * FB_T * 4);
            tma_load_4d(sQ + s * Cfg::TILE_BYTES, &tmQ, &q_full[s], 0, q0, hq, b);
            tma_load_4d(sDO + s * Cfg::TILE_BYTES, &tmDO, &q_full[s], 0, q0, hq, b);
            const long long stat = ((long long)b * p.Hq + hq) * p.Tpad + q0;
            bulk_load_1d(sStat + s * 2 * FB_T, p.lse + stat, FB_T * 4, &q_full[s]);
            bulk_load_1d(sStat + s * 2 * FB_T + FB_T, p.delta + stat, FB_T * 4, &q_full[s]);
          }
          __syncwarp();
        }
        base += n_iters;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // (the whole warp walks the loop; one elected lane executes the tcgen05 instructions)
    const bool leader = elect_one() != 0;
    {
      constexpr uint32_t id_half = make_idesc_bf16(FB_T, H, false, false);   // S^T / dP^T of one half: [128 kv] x [64 q]
      constexpr uint32_t id_kmn = make_idesc_bf16(FB_T, D, false, true);     // dV, dK
      constexpr uint32_t id_mnmn = make_idesc_bf16(FB_T, D, true, true);     // dQ
      // Shared-memory descriptors: every operand sits at a compile-time offset from the 1024-byte aligned base, so a
      // descriptor is one add on the low word (address >> 4) plus constants.  The issuing thread is the critical path
      // of the kernel; building descriptors field by field for each product cost more than the products themselves.
      constexpr uint32_t kDescHi = ((1024u >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);   // SBO 1024, version, SWIZZLE_128B
      constexpr uint32_t kLoK = (16u >> 4) << 16;                                       // K-major: LBO 16
      constexpr uint32_t kLoMN = ((uint32_t)(FB_T * 128) >> 4) << 16;                   // MN-major: LBO 16 KB
      static_assert(Cfg::CHUNK_BYTES == FB_T * 128, "one LBO for every MN-major operand");
      auto desc = [&](uint32_t lo16, uint32_t lo_const) -> uint64_t {
        return (static_cast<uint64_t>(kDescHi) << 32) | static_cast<uint64_t>(lo16 + lo_const);
      };
      const uint32_t b16 = (smem_u32(smem) & 0x3FFFF) >> 4;
      const uint32_t k16 = b16 + (Cfg::OFF_K >> 4), v16 = b16 + (Cfg::OFF_V >> 4);
      // score products of half h of the tile in stage s: rows h*64.. of Q / dO are 64 x 128 bytes further on
      auto scores = [&](int h, int s) {
        const uint32_t q16 = b16 + ((Cfg::OFF_Q + s * Cfg::TILE_BYTES + h * (H * 128)) >> 4);
        const uint32_t do16 = b16 + ((Cfg::OFF_DO + s * Cfg::TILE_BYTES + h * (H * 128)) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          if (leader) umma_f16_ss(tmem_base + Cfg::COL_ST + h * H, desc(k16 + kk * 2, kLoK), desc(q16 + kk * 2, kLoK), id_half,
                      kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          if (leader) umma_f16_ss(tmem_base + Cfg::COL_DPT + h * H, desc(v16 + kk * 2, kLoK), desc(do16 + kk * 2, kLoK), id_half,
                      kk > 0 ? 1u : 0u);
        if (leader) umma_commit(&sdp[h]);
      };
      int base = 0;
      bool ok = true;
      long long t_kv = 0, t_q = 0, t_pds0 = 0, t_pds1 = 0, t_dq = 0, t_issue = 0, t_all = now(), tm;
#define PROF_WAIT(acc, expr) (tm = now(), ok_w = (expr), acc += now() - tm, ok_w)
      bool ok_w;
      for (int r = 0; ok; ++r) {
        int kv_tile, hkv, b;
        if (!item_of(r, kv_tile, hkv, b)) break;
        const int n_iters = (p.n_tiles - kv_tile) * group;
        if (!PROF_WAIT(t_kv, mbar_wait(kv_full, r & 1, abort_flag, p.status, kStatusTimeoutFull))) break;
        for (int it = 0; it <= n_iters && ok; ++it) {
          const int g = base + it;
          if (it < n_iters) {
            if (!PROF_WAIT(t_q, mbar_wait(&q_full[g % ST], (g / ST) & 1, abort_flag, p.status, kStatusTimeoutFull))) { ok = false; break; }
            // half a of the previous tile has been read out of tensor memory (across items the previous item's last
            // tile was waited for through pds[1])
            if (it > 0 && !PROF_WAIT(t_pds0, mbar_wait(&pds[0], (g - 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull))) { ok = false; break; }
            tc_fence_after();
            scores(0, g % ST);
          }
          if (it > 0) {
            const int j = it - 1, gj = g - 1, sj = gj % ST, bq = gj & 1;
            if (!PROF_WAIT(t_pds1, mbar_wait(&pds[1], gj & 1, abort_flag, p.status, kStatusTimeoutTmemFull))) { ok = false; break; }
            if (gj >= 2 && !PROF_WAIT(t_dq, mbar_wait(&dq_drained[bq], ((gj >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutTmemEmpty))) {
              ok = false;
              break;
            }
            // the first products of an item overwrite dV / dK: the previous item's must have been read out
            if (j == 0 && r > 0 && !mbar_wait(dkv_drained, (r - 1) & 1, abort_flag, p.status, kStatusTimeoutTmemEmpty)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t q16 = b16 + ((Cfg::OFF_Q + sj * Cfg::TILE_BYTES) >> 4);
            const uint32_t do16 = b16 + ((Cfg::OFF_DO + sj * Cfg::TILE_BYTES) >> 4);
            const uint32_t half_a = Cfg::chunk_off(0, gj) >> 4, half_b = Cfg::chunk_off(1, gj) >> 4;
            const uint32_t p16a = b16 + (Cfg::OFF_P >> 4) + half_a, p16b = b16 + (Cfg::OFF_P >> 4) + half_b;
            const uint32_t ds16a = b16 + (Cfg::OFF_DS >> 4) + half_a, ds16b = b16 + (Cfg::OFF_DS >> 4) + half_b;
            const uint32_t acc0 = j > 0 ? 1u : 0u;
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk)   // dV += P^T dO: reduction over the 128 queries, 16 per step
              if (leader) umma_f16_ss(tmem_base + Cfg::COL_DV, desc((kk < 4 ? p16a : p16b) + (kk & 3) * 2, kLoK),
                          desc(do16 + kk * 128, kLoMN), id_kmn, kk > 0 ? 1u : acc0);
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk)   // dK += dS^T Q
              if (leader) umma_f16_ss(tmem_base + Cfg::COL_DK, desc((kk < 4 ? ds16a : ds16b) + (kk & 3) * 2, kLoK),
                          desc(q16 + kk * 128, kLoMN), id_kmn, kk > 0 ? 1u : acc0);
            // dQ partial = dS K: A = dS in MN-major form, two 64-query chunks CHUNK_BYTES apart starting at the
            // lower of the two addresses: (a0, b) for even tiles, (b, a1) for odd tiles (rows come out rotated by 64)
            const uint32_t dsf16 = b16 + ((Cfg::OFF_DS + (bq ? Cfg::CHUNK_BYTES : 0)) >> 4);
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk)
              if (leader) umma_f16_ss(tmem_base + Cfg::COL_DQ + bq * D, desc(dsf16 + kk * 128, kLoMN), desc(k16 + kk * 128, kLoMN),
                          id_mnmn, kk > 0 ? 1u : 0u);
            if (leader) {
              umma_commit(&q_empty[sj]);
              umma_commit(&dq_full[bq]);
              if (it == n_iters) umma_commit(kv_empty);   // last product of the item: K / V may be replaced
            }
            __syncwarp();
          }
          if (it < n_iters) scores(1, g % ST);   // half b: its columns were read out before pds[1] of the previous tile
        }
        base += n_iters;
      }
#undef PROF_WAIT
      if (PROF && leader) {
        t_all = now() - t_all;
        t_issue = t_all - t_kv - t_q - t_pds0 - t_pds1 - t_dq;
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 0), (unsigned long long)t_all);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 1), (unsigned long long)t_kv);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 2), (unsigned long long)t_q);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 3), (unsigned long long)t_pds0);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 4), (unsigned long long)t_pds1);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 5), (unsigned long long)t_dq);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 6), (unsigned long long)t_issue);
        atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 7), (unsigned long long)base);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax-gradient threads
    // Two groups of 8 warps, one per half of the query tile, run side by side: while group 0 waits for tensor memory
    // or for its barrier, group 1 has work to issue.  Inside a group: warp -> (TMEM lane quarter = 32 KV rows,
    // cb2 = which 32 of the half's 64 query columns).  For the dQ / dK / dV drains all 16 warps split D as before.
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int cb = cw >> 2;            // 0..3: 16-column block of D for the drains
    const int my_half = cw >> 3;       // 0: half a, 1: half b
    const int cb2 = (cw >> 2) & 1;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;

    long long c_wait_sdp = 0, c_wait_dq = 0, c_drain = 0, c_ld0 = 0, c_chunks = 0, c_fence = 0, c_all = now();   // optional profile (see attn_prof_buffer)
    // dQ partial of pipeline slot g (tile `it_j` of the item described by the arguments).  Tensor memory hands every
    // lane one query row, so adding it to global memory from registers would be one 16-byte `red` per lane and row;
    // instead each compute group stages its 32 columns as a [128 q][32] fp32 box in shared memory (128-byte swizzle:
    // conflict free for row-per-lane stores) and one thread adds the box to dq_accum with a bulk tensor reduce.
    const bool elected = (cw == my_half * (FB_CWARPS / 2)) && lane == 0;
    uint8_t* stage_box = sDQS + my_half * Cfg::DQS_BYTES;
    auto drain_dq = [&](int g, int it_j, int kv_tile, int hkv, int b) -> bool {
      const int bq = g & 1;
      const long long tw = now();
      if (!mbar_wait(&dq_full[bq], (g >> 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) return false;
      const long long tb = now();
      c_wait_dq += tb - tw;
      tc_fence_after();
      uint32_t r[16];
      tmem_ld_32x16(tmem_base + Cfg::COL_DQ + bq * D + lane_addr + cb * 16, r);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_drained[bq]);   // the tensor-memory buffer may be overwritten
      // the box is free once the previous reduce of this group has read it
      if (elected) {
        bulk_wait_read_all();
        mbar_arrive(&stg_free[my_half]);
      }
      if (!mbar_wait(&stg_free[my_half], g & 1, abort_flag, p.status, kStatusTimeoutEmpty)) return false;
      const int q_local = bq ? ((row + H) & (FB_T - 1)) : row;   // odd slots: rows are the queries rotated by 64
      uint8_t* srow = stage_box + q_local * 128;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int unit = ((cb & 1) * 4 + u) ^ (q_local & 7);
        *reinterpret_cast<float4*>(srow + unit * 16) =
            make_float4(__uint_as_float(r[u * 4]) * p.scale, __uint_as_float(r[u * 4 + 1]) * p.scale,
                        __uint_as_float(r[u * 4 + 2]) * p.scale, __uint_as_float(r[u * 4 + 3]) * p.scale);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&stg_full[my_half]);
      if (elected) {
        if (!mbar_wait(&stg_full[my_half], g & 1, abort_flag, p.status, kStatusTimeoutFull)) return false;
        const int tiles_per_head = p.n_tiles - kv_tile;
        const int hq_j = hkv * group + it_j / tiles_per_head;
        const int q0 = (kv_tile + it_j % tiles_per_head) * FB_T;
        tma_reduce_add_4d(&p.tm_dq, stage_box, my_half * 32, q0, hq_j, b);   // rows past T are clipped by the map
        bulk_commit();
      }
      c_drain += now() - tb;
      return true;
    };

    int base = 0;
    bool ok = true;
    for (int rnd = 0; ok; ++rnd) {
      int kv_tile, hkv, b;
      if (!item_of(rnd, kv_tile, hkv, b)) break;
      const int kv0 = kv_tile * FB_T;
      const int kv_idx = kv0 + row;
      const bool kv_live = kv_idx < p.T;
      const int tiles_per_head = p.n_tiles - kv_tile;
      const int n_iters = tiles_per_head * group;
      for (int it = 0; it < n_iters && ok; ++it) {
        const int g = base + it, s = g % ST;
        const int q0 = (kv_tile + it % tiles_per_head) * FB_T;
        const bool masked = (q0 < kv0 + FB_T) || (kv0 + FB_T > p.T);   // diagonal tile, or a KV tile with dead rows
        auto half = [&](int h, auto masked_tag) -> bool {
          constexpr bool MASKED = decltype(masked_tag)::value;
          const long long tw = now();
          if (!mbar_wait(&sdp[h], g & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) return false;
          c_wait_sdp += now() - tw;
          tc_fence_after();
          const int off = Cfg::chunk_off(h, g) + row * 128;     // [128 kv rows][64 q] bf16, SWIZZLE_128B
          // 32 query columns per thread in four chunks of 8: the tensor-memory loads of chunk c+1 are in flight while
          // chunk c is computed (one chunk of S^T and dP^T = one 16-byte unit of P^T and of dS^T)
          const int cbase = h * H + cb2 * 32;                   // first of this thread's query columns in the tile
          const float* s_lse = sStat + s * 2 * FB_T + cbase;    // q_full (waited by the issuer) covers the statistics
          const float* s_delta = s_lse + FB_T;
          uint32_t rs[2][8], rd[2][8];
          tmem_ld_32x8(tmem_base + Cfg::COL_ST + lane_addr + cbase, rs[0]);
          tmem_ld_32x8(tmem_base + Cfg::COL_DPT + lane_addr + cbase, rd[0]);
          tmem_ld_wait_on(rs[0], rd[0]);
          const long long t_a = now();
          c_ld0 += t_a - tw;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int cur = c & 1, nxt = cur ^ 1;
            if (c < 3) {
              tmem_ld_32x8(tmem_base + Cfg::COL_ST + lane_addr + cbase + (c + 1) * 8, rs[nxt]);
              tmem_ld_32x8(tmem_base + Cfg::COL_DPT + lane_addr + cbase + (c + 1) * 8, rd[nxt]);
            }
            uint32_t pp[4], dd[4];
#pragma unroll
            for (int gq = 0; gq < 2; ++gq) {
              const float4 l4 = *reinterpret_cast<const float4*>(s_lse + c * 8 + gq * 4);
              const float4 d4 = *reinterpret_cast<const float4*>(s_delta + c * 8 + gq * 4);
              const float lse[4] = {l4.x, l4.y, l4.z, l4.w};
              const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
              float pv[4], dv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = gq * 4 + e;
                float pr = exp2f(fmaf(__uint_as_float(rs[cur][i]), p.scale_log2, -lse[e]));
                if constexpr (MASKED) pr = (kv_live && (q0 + cbase + c * 8 + i >= kv_idx)) ? pr : 0.f;
                pv[e] = pr;
                dv[e] = pr * (__uint_as_float(rd[cur][i]) - dl[e]);   // the softmax scale is applied when dQ / dK leave TMEM
              }
              pp[gq * 2] = pack_bf16x2(pv[0], pv[1]);
              pp[gq * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
              dd[gq * 2] = pack_bf16x2(dv[0], dv[1]);
              dd[gq * 2 + 1] = pack_bf16x2(dv[2], dv[3]);
            }
            const int unit = (cb2 * 4 + c) ^ (row & 7);
            *reinterpret_cast<uint4*>(sP + off + unit * 16) = make_uint4(pp[0], pp[1], pp[2], pp[3]);
            *reinterpret_cast<uint4*>(sDS + off + unit * 16) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
            if (c < 3) tmem_ld_wait_on(rs[nxt], rd[nxt]);
          }
          const long long t_b = now();
          c_chunks += t_b - t_a;
          fence_proxy_async_smem();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&pds[h]);
          c_fence += now() - t_b;
          return true;
        };
        ok = masked ? half(my_half, std::true_type{}) : half(my_half, std::false_type{});
        // the dQ partial of the previous tile of this item: overlaps the products the issuer has just launched
        if (ok && it > 0) ok = drain_dq(g - 1, it - 1, kv_tile, hkv, b);
      }
      if (!ok) break;
      if (!drain_dq(base + n_iters - 1, n_iters - 1, kv_tile, hkv, b)) break;
      // dK and dV of this item (dq_full of its last tile implies both are complete)
      tc_fence_after();
      constexpr int DC = D / 4;
      __nv_bfloat16* dk_row = p.dk + (long long)b * p.dk_stride_b + (long long)kv_idx * p.dk_stride_t +
                              (long long)hkv * p.dk_stride_h + cb * DC;
      __nv_bfloat16* dv_row = p.dv + (long long)b * p.dv_stride_b + (long long)kv_idx * p.dv_stride_t +
                              (long long)hkv * p.dv_stride_h + cb * DC;
      uint32_t rk[16], rv[16];
      tmem_ld_32x16(tmem_base + Cfg::COL_DK + lane_addr + cb * DC, rk);
      tmem_ld_32x16(tmem_base + Cfg::COL_DV + lane_addr + cb * DC, rv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dkv_drained);   // the next item's products may overwrite dV / dK now
      if (kv_live) {
        // this thread's 16 columns of the row are 32 contiguous bytes: one 256-bit store each where the address allows
        uint32_t ka[8], va[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ka[e] = pack_bf16x2(__uint_as_float(rk[e * 2]) * p.scale, __uint_as_float(rk[e * 2 + 1]) * p.scale);
          va[e] = pack_bf16x2(__uint_as_float(rv[e * 2]), __uint_as_float(rv[e * 2 + 1]));
        }
        if (aligned32(dk_row) && aligned32(dv_row)) {
          st_global_b256(dk_row, ka);
          st_global_b256(dv_row, va);
        } else {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            *reinterpret_cast<uint4*>(dk_row + u * 8) = make_uint4(ka[u * 4], ka[u * 4 + 1], ka[u * 4 + 2], ka[u * 4 + 3]);
            *reinterpret_cast<uint4*>(dv_row + u * 8) = make_uint4(va[u * 4], va[u * 4 + 1], va[u * 4 + 2], va[u * 4 + 3]);
          }
        }
      }
      base += n_iters;
    }
    if (elected) bulk_wait_all();   // the staged boxes stay valid until their reduces have completed
    if (PROF && lane == 0 && warp == 2) {
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 12), (unsigned long long)c_ld0);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 13), (unsigned long long)c_chunks);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + 14), (unsigned long long)c_fence);
    }
    if (PROF && lane == 0 && warp == 2) {
      const int o = 8;
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + o), (unsigned long long)(now() - c_all));
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + o + 1), (unsigned long long)c_wait_sdp);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + o + 2), (unsigned long long)c_wait_dq);
      atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + o + 3), (unsigned long long)c_drain);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace incin
