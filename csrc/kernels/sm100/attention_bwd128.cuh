// Attention backward for head_dim 128, pipelined over 64-query steps so that the tensor core and the softmax-gradient
// threads work at the same time.
//
// One CTA owns a 128-row KV tile and walks the queries at or below the diagonal in steps of 64 rows.  With head_dim
// 128 the accumulators dV and dK alone fill half of tensor memory, so a 128-query tile would leave no room for a
// second set of score columns and every step would wait for the one before it (that is flash_bwd_kernel<128>).  With
// 64 queries per step the scores S^T and their gradient dP^T take 64 columns each, two buffers of each fit, and two
// steps are in flight at any time:
//
//   tensor core : S dP (j) | dV dK dQ^T (j-1) | S dP (j+1) | dV dK dQ^T (j) | ...
//   group 0     :     softmax-gradient (j)        | softmax-gradient (j+1)       ...      (8 warps)
//   group 1     :  ... read out dQ^T (j-1), stage, reduce | read out dQ^T (j) ...           (8 warps)
//
// Step j uses buffer j & 1 of everything.  Per step:
//     S^T  = K Q^T   [128 kv x 64 q]      dP^T = V dO^T
//     dV  += P^T dO  [128 kv x 128 d]     dK  += dS^T Q          (reduction over the 64 queries)
//     dQ^T = K^T dS  [128 d  x 64 q]                             (reduction over the 128 kv rows)
// dQ is produced TRANSPOSED: head_dim runs along the tensor-memory lanes, so the 32 lanes of a warp hold 32
// consecutive floats of one dQ row.  The compute group writes the partial as four [64 q][32 fp32] boxes into the
// P^T / dS^T buffers of its step — dead once the step's products have completed, and exactly 32 KB together — and one
// thread adds the boxes to the fp32 accumulator with bulk tensor reduces: the L2 sees whole 128-byte lines instead of
// 8 k scalar atomics per step, which otherwise slowed every other L2 client of the SM (the Q / dO loads waited 8 times
// longer).  The dQ^T partial reuses the dP^T columns of its step, which the compute group has read by then.
//
// Shared memory (224 KB + barriers): K, V 32 KB each; three stages of Q and dO (64 rows, 16 KB each); two buffers of
// P^T and of dS^T (16 KB each); per-stage lse / delta.  Tensor memory (512 columns): S^T x2 [0,128), dP^T / dQ^T x2
// [128,256), dV [256,384), dK [384,512).
//
// The kernel is persistent: one CTA per SM walks (batch, KV head, KV tile) items, head by head, in snake order.
// All waits are bounded; a timed-out wait unwinds through the common exit.  No counterpart in the reference.
#pragma once

namespace incin {

struct Fb128 {
  static constexpr int D = 128;
  static constexpr int TQ = 64;                         // queries per step
  static constexpr int ST = 3;                          // Q / dO stages
  static constexpr int KV_BYTES = FB_T * D * 2;         // 32 KB: K or V tile, two chunks of 64 head-dim columns
  static constexpr int KV_CHUNK = FB_T * 128;           // 16 KB
  static constexpr int Q_BYTES = TQ * D * 2;            // 16 KB: Q or dO of one step, two chunks of 64 columns
  static constexpr int Q_CHUNK = TQ * 128;              // 8 KB
  static constexpr int PT_BYTES = FB_T * TQ * 2;        // 16 KB: P^T or dS^T of one step ([128 kv][64 q])
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_Q = 2 * KV_BYTES;
  static constexpr int OFF_DO = OFF_Q + ST * Q_BYTES;
  static constexpr int OFF_P = OFF_DO + ST * Q_BYTES;
  static constexpr int OFF_DS = OFF_P + 2 * PT_BYTES;
  static constexpr int OFF_STAT = OFF_DS + 2 * PT_BYTES;      // per stage: lse[64], delta[64]
  static constexpr int OFF_BAR = OFF_STAT + ST * 2 * TQ * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;            // the window itself is declared 1024-byte aligned
  static_assert(OFF_Q % 1024 == 0 && OFF_P % 1024 == 0 && OFF_BAR % 8 == 0 && SMEM_BYTES <= 227 * 1024,
                "shared-memory plan");
  static constexpr int COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384, TMEM_COLS = 512;
};

// PROF: a second instantiation that adds up clock intervals of the issuing thread and of one compute lane into p.prof
// (read with incin_attn_prof_read), so that the production kernel carries no clock reads.  p.prof[15] holds
// experiment switches for that instantiation only: bit 0 = leave out the dQ adds, bit 1 = the P^T / dS^T
// shared-memory stores, bit 2 = the dQ^T products, bit 3 = the dV / dK products, bit 4 = the dP^T products (all give
// wrong results; they exist to attribute time).
template <bool PROF>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ FbParams p) {
  using Cfg = Fb128;
  constexpr int D = Cfg::D, ST = Cfg::ST, TQ = Cfg::TQ;
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
  const long long dbg = PROF ? p.prof[15] : 0ll;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint8_t* sDS = smem + Cfg::OFF_DS;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;              // 1
  uint64_t* q_full = bars + 1;           // [3]  Q_j, dO_j and their statistics landed
  uint64_t* q_empty = bars + 4;          // [3]  the products that read that stage finished
  uint64_t* sdp = bars + 7;              // [2]  S^T and dP^T of a step are in tensor memory
  uint64_t* pds = bars + 9;              // [2]  P^T and dS^T of a step are in shared memory (one arrival per warp of the group)
  uint64_t* dq_full = bars + 11;         // [2]  dQ^T partial written (and dV / dK updated)
  uint64_t* dq_drained = bars + 13;      // [2]  dQ^T partial read out (one arrival per warp of the group)
  uint64_t* kv_empty = bars + 15;        // every product of the current item has been committed: K / V may be replaced
  uint64_t* dkv_drained = bars + 16;     // dK / dV of the current item have been read out (one arrival per warp)
  uint64_t* stg_free = bars + 17;        // [2]  per group: the bulk reduces of its previous step have read their boxes
  uint64_t* stg_full = bars + 19;        // [2]  per group: all 8 warps have written their part of the dQ boxes
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.Hq / p.Hkv;
  const int heads_batches = p.Hkv * p.batch;
  const int n_items = p.n_tiles * heads_batches;
  const int n_steps_total = (p.T + TQ - 1) / TQ;     // 64-query steps of the whole sequence
  // Item list: (batch, KV head) outermost, KV tile innermost, so the CTAs that run at the same time work on a handful
  // of heads: their fp32 dQ accumulator (T x D x 4 bytes per head, touched by every KV tile of the head), Q and dO stay
  // in L2 between the KV tiles.  With the KV tile outermost 148 CTAs spread over 148 heads, the accumulator lines were
  // evicted between two adds and every add became a DRAM read-modify-write (twice the accumulator per KV tile).
  // Round r of CTA c takes item r*G + c (even r) or (r+1)*G - 1 - c (odd r): the snake pairs the long items (low KV
  // tiles) of one round with the short ones of the next.  Returns false when this CTA has no item in round r.
  auto item_of = [&](int r, int& kv_tile, int& hkv, int& b) -> bool {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int idx = (r & 1) ? (r + 1) * G - 1 - c : r * G + c;
    if (idx >= n_items) return false;
    kv_tile = idx % p.n_tiles;
    const int hb = idx / p.n_tiles;
    hkv = hb % p.Hkv;
    b = hb / p.Hkv;
    return true;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&sdp[g], 1);
      mbar_init(&pds[g], FB_CWARPS / 2);
      mbar_init(&dq_full[g], 1);
      mbar_init(&dq_drained[g], FB_CWARPS / 2);
    }
    mbar_init(kv_empty, 1);
    mbar_init(dkv_drained, FB_CWARPS);
    for (int g = 0; g < 2; ++g) {
      mbar_init(&stg_free[g], 1);
      mbar_init(&stg_full[g], FB_CWARPS / 2);
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
      int base = 0;   // query steps handed to the pipeline so far (all roles count the same way)
      bool ok = true;
      for (int r = 0; ok; ++r) {
        int kv_tile, hkv, b;
        if (!item_of(r, kv_tile, hkv, b)) break;
        const int kv0 = kv_tile * FB_T;
        const int steps_per_head = n_steps_total - 2 * kv_tile;
        const int n_iters = steps_per_head * group;
        // K / V of the previous item are still operands until its last product has been committed
        if (r > 0 && !mbar_wait(kv_empty, (r - 1) & 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        if (leader) {
          mbar_expect_tx(kv_full, 2 * Cfg::KV_BYTES);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_4d(sK + c * Cfg::KV_CHUNK, &tmK, kv_full, c * 64, kv0, hkv, b);
            tma_load_4d(sV + c * Cfg::KV_CHUNK, &tmV, kv_full, c * 64, kv0, hkv, b);
          }
        }
        for (int it = 0; it < n_iters; ++it) {
          const int g = base + it, s = g % ST;
          const int hq = hkv * group + it / steps_per_head;
          const int q0 = (2 * kv_tile + it % steps_per_head) * TQ;
          if (!mbar_wait(&q_empty[s], ((g / ST) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          if (leader) {
            mbar_expect_tx(&q_full[s], 2 * Cfg::Q_BYTES + 2 * TQ * 4);
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
              tma_load_4d(sQ + s * Cfg::Q_BYTES + c * Cfg::Q_CHUNK, &tmQ, &q_full[s], c * 64, q0, hq, b);
              tma_load_4d(sDO + s * Cfg::Q_BYTES + c * Cfg::Q_CHUNK, &tmDO, &q_full[s], c * 64, q0, hq, b);
            }
            // per-query statistics of this step: two 256-byte bulk copies (rows are padded to the 128-row tile edge)
            const long long stat = ((long long)b * p.Hq + hq) * p.Tpad + q0;
            bulk_load_1d(sStat + s * 2 * TQ, p.lse + stat, TQ * 4, &q_full[s]);
            bulk_load_1d(sStat + s * 2 * TQ + TQ, p.delta + stat, TQ * 4, &q_full[s]);
          }
          __syncwarp();
        }
        base += n_iters;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop (waits, descriptor arithmetic, loop control stay warp-uniform and cheap); only the
    // elected lane executes the tcgen05 instructions.
    const bool leader = elect_one() != 0;
    {
      constexpr uint32_t id_s = make_idesc_bf16(FB_T, TQ, false, false);   // S^T / dP^T: [128 kv] x [64 q], K = head_dim
      constexpr uint32_t id_kmn = make_idesc_bf16(FB_T, D, false, true);   // dV, dK: [128 kv] x [128 d], K = queries
      constexpr uint32_t id_qt = make_idesc_bf16(D, TQ, true, true);       // dQ^T: [128 d] x [64 q], K = kv rows
      // Shared-memory descriptors: every operand sits at a compile-time offset from the 1024-byte aligned base, so a
      // descriptor is one add on the low word (address >> 4) plus constants (the issuing thread is the critical path).
      constexpr uint32_t kDescHi = ((1024u >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);   // SBO 1024, version, SWIZZLE_128B
      constexpr uint32_t kLoK = (16u >> 4) << 16;                                       // K-major: LBO 16
      constexpr uint32_t kLoMNkv = ((uint32_t)Cfg::KV_CHUNK >> 4) << 16;                // MN-major K / V: chunks 16 KB apart
      constexpr uint32_t kLoMNq = ((uint32_t)Cfg::Q_CHUNK >> 4) << 16;                  // MN-major Q / dO: chunks 8 KB apart
      auto desc = [&](uint32_t lo16, uint32_t lo_const) -> uint64_t {
        return (static_cast<uint64_t>(kDescHi) << 32) | static_cast<uint64_t>(lo16 + lo_const);
      };
      const uint32_t b16 = (smem_u32(smem) & 0x3FFFF) >> 4;
      const uint32_t k16 = b16 + (Cfg::OFF_K >> 4), v16 = b16 + (Cfg::OFF_V >> 4);
      // score products of the step in stage s into buffer g; reduction over head_dim: 8 steps of 16, the second four
      // in the second 64-column chunk of each operand
      auto scores = [&](int g, int s) {
        const uint32_t q16 = b16 + ((Cfg::OFF_Q + s * Cfg::Q_BYTES) >> 4);
        const uint32_t do16 = b16 + ((Cfg::OFF_DO + s * Cfg::Q_BYTES) >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          if (leader) umma_f16_ss(tmem_base + Cfg::COL_ST + g * TQ, desc(k16 + (kk >> 2) * (Cfg::KV_CHUNK >> 4) + (kk & 3) * 2, kLoK),
                      desc(q16 + (kk >> 2) * (Cfg::Q_CHUNK >> 4) + (kk & 3) * 2, kLoK), id_s, kk > 0 ? 1u : 0u);
        if (!(PROF && (dbg & 16)))
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          if (leader) umma_f16_ss(tmem_base + Cfg::COL_DPT + g * TQ, desc(v16 + (kk >> 2) * (Cfg::KV_CHUNK >> 4) + (kk & 3) * 2, kLoK),
                      desc(do16 + (kk >> 2) * (Cfg::Q_CHUNK >> 4) + (kk & 3) * 2, kLoK), id_s, kk > 0 ? 1u : 0u);
        if (leader) umma_commit(&sdp[g]);
      };
      int base = 0;
      bool ok = true;
      long long t_kv = 0, t_q = 0, t_drained = 0, t_pds = 0, t_all = now(), tm;
      bool ok_w;
#define PROF_WAIT(acc, expr) (tm = now(), ok_w = (expr), acc += now() - tm, ok_w)
      for (int r = 0; ok; ++r) {
        int kv_tile, hkv, b;
        if (!item_of(r, kv_tile, hkv, b)) break;
        const int n_iters = (n_steps_total - 2 * kv_tile) * group;
        if (!PROF_WAIT(t_kv, mbar_wait(kv_full, r & 1, abort_flag, p.status, kStatusTimeoutFull))) break;
        for (int it = 0; it <= n_iters && ok; ++it) {
          if (it < n_iters) {
            const int gi = base + it, g = gi & 1, s = gi % ST;
            if (!PROF_WAIT(t_q, mbar_wait(&q_full[s], (gi / ST) & 1, abort_flag, p.status, kStatusTimeoutFull))) { ok = false; break; }
            // buffer g: the dQ^T partial of step gi - 2 has been read out (its S^T / dP^T were read before that)
            if (gi >= 2 && !PROF_WAIT(t_drained, mbar_wait(&dq_drained[g], ((gi >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutTmemEmpty))) {
              ok = false;
              break;
            }
            tc_fence_after();
            scores(g, s);
          }
          if (it > 0) {
            const int j = it - 1, gj = base + j, g = gj & 1, s = gj % ST;
            if (!PROF_WAIT(t_pds, mbar_wait(&pds[g], (gj >> 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull))) { ok = false; break; }
            // the first products of an item overwrite dV / dK: the previous item's must have been read out
            if (j == 0 && r > 0 && !mbar_wait(dkv_drained, (r - 1) & 1, abort_flag, p.status, kStatusTimeoutTmemEmpty)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t q16 = b16 + ((Cfg::OFF_Q + s * Cfg::Q_BYTES) >> 4);
            const uint32_t do16 = b16 + ((Cfg::OFF_DO + s * Cfg::Q_BYTES) >> 4);
            const uint32_t p16 = b16 + ((Cfg::OFF_P + g * Cfg::PT_BYTES) >> 4);
            const uint32_t ds16 = b16 + ((Cfg::OFF_DS + g * Cfg::PT_BYTES) >> 4);
            const uint32_t acc0 = j > 0 ? 1u : 0u;
            if (!(PROF && (dbg & 8))) {
#pragma unroll
            for (int kk = 0; kk < TQ / 16; ++kk)   // dV += P^T dO: reduction over the 64 queries, 16 per product
              if (leader) umma_f16_ss(tmem_base + Cfg::COL_DV, desc(p16 + kk * 2, kLoK), desc(do16 + kk * 128, kLoMNq), id_kmn,
                          kk > 0 ? 1u : acc0);
#pragma unroll
            for (int kk = 0; kk < TQ / 16; ++kk)   // dK += dS^T Q
              if (leader) umma_f16_ss(tmem_base + Cfg::COL_DK, desc(ds16 + kk * 2, kLoK), desc(q16 + kk * 128, kLoMNq), id_kmn,
                          kk > 0 ? 1u : acc0);
            }
            if (!(PROF && (dbg & 4)))
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk)   // dQ^T = K^T dS: both operands MN-major, 16 kv rows per product
              if (leader) umma_f16_ss(tmem_base + Cfg::COL_DPT + g * TQ, desc(k16 + kk * 128, kLoMNkv), desc(ds16 + kk * 128, kLoMNkv),
                          id_qt, kk > 0 ? 1u : 0u);
            if (leader) {
              umma_commit(&q_empty[s]);
              umma_commit(&dq_full[g]);
              if (it == n_iters) umma_commit(kv_empty);   // last product of the item: K / V may be replaced
            }
            __syncwarp();
          }
        }
        base += n_iters;
      }
#undef PROF_WAIT
      if (PROF && leader) {
        t_all = now() - t_all;
        auto add = [&](int i, long long v) { atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + i), (unsigned long long)v); };
        add(0, t_all); add(1, t_kv); add(2, t_q); add(3, t_drained); add(4, t_pds);
        add(5, t_all - t_kv - t_q - t_drained - t_pds);   // issuing (the thread is back-pressured: tensor-pipe time)
        add(7, base);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax-gradient threads
    // Two groups of 8 warps with different roles, both working on every step: group 0 turns S^T / dP^T into P^T / dS^T,
    // group 1 reads the dQ^T partial out of tensor memory, stages it and has it added to the accumulator.  Split by
    // role (rather than by step parity) the tail of the read-out — shared-memory stores, fence, the wait for the
    // group's other warps, issuing the reduces — runs beside the next step's softmax-gradient math instead of in
    // front of it.  Inside a group: warp -> (TMEM lane quarter, cb2 = which 32 of the step's 64 query columns).
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int role = cw >> 3;          // 0: softmax-gradient, 1: dQ read-out
    const int cb2 = (cw >> 2) & 1;
    const int cb = cw >> 2;            // 0..3: 32-column block of head_dim for the dK / dV write-out
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool elected = (cw == FB_CWARPS / 2) && lane == 0;   // issues the bulk reduces

    int base = 0;
    bool ok = true;
    long long c_wait_sdp = 0, c_soft = 0, c_wait_dq = 0, c_drain = 0, c_dkv = 0, c_all = now(), c_steps = 0;
    for (int rnd = 0; ok; ++rnd) {
      int kv_tile, hkv, b;
      if (!item_of(rnd, kv_tile, hkv, b)) break;
      const int kv0 = kv_tile * FB_T;
      const int kv_idx = kv0 + row;
      const bool kv_live = kv_idx < p.T;
      const int steps_per_head = n_steps_total - 2 * kv_tile;
      const int n_iters = steps_per_head * group;
      if (role == 0) {
        for (int it = 0; it < n_iters && ok; ++it) {
          const int gi = base + it, s = gi % ST, g = gi & 1;
          const int q0 = (2 * kv_tile + it % steps_per_head) * TQ;
          const bool masked = (q0 < kv0 + FB_T) || (kv0 + FB_T > p.T);   // a diagonal step, or a KV tile with dead rows
          const long long t0 = now();
          if (!mbar_wait(&sdp[g], (gi >> 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
          // P^T / dS^T of this buffer were the dQ boxes of step gi - 2: its reduces must have read them
          if (gi >= 2 && !mbar_wait(&stg_free[g], ((gi >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          const long long t1 = now();
          tc_fence_after();
          auto softmax_grad = [&](auto masked_tag) {
            constexpr bool MASKED = decltype(masked_tag)::value;
            const int off = g * Cfg::PT_BYTES + row * 128;      // [128 kv rows][64 q] bf16, SWIZZLE_128B
            // 32 query columns per thread in four chunks of 8: the tensor-memory loads of chunk c+1 are in flight while
            // chunk c is computed (one chunk of S^T and dP^T = one 16-byte unit of P^T and of dS^T)
            const uint32_t tcol = lane_addr + g * TQ + cb2 * 32;
            const float* s_lse = sStat + s * 2 * TQ + cb2 * 32;      // q_full (waited by the issuer) covers the statistics
            const float* s_delta = s_lse + TQ;
            uint32_t rs[2][8], rd[2][8];
            tmem_ld_32x8(tmem_base + Cfg::COL_ST + tcol, rs[0]);
            tmem_ld_32x8(tmem_base + Cfg::COL_DPT + tcol, rd[0]);
            tmem_ld_wait_on(rs[0], rd[0]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int cur = c & 1, nxt = cur ^ 1;
              if (c < 3) {
                tmem_ld_32x8(tmem_base + Cfg::COL_ST + tcol + (c + 1) * 8, rs[nxt]);
                tmem_ld_32x8(tmem_base + Cfg::COL_DPT + tcol + (c + 1) * 8, rd[nxt]);
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
                  if constexpr (MASKED) pr = (kv_live && (q0 + cb2 * 32 + c * 8 + i >= kv_idx)) ? pr : 0.f;
                  pv[e] = pr;
                  dv[e] = pr * (__uint_as_float(rd[cur][i]) - dl[e]);   // the softmax scale is applied when dQ / dK leave TMEM
                }
                pp[gq * 2] = pack_bf16x2(pv[0], pv[1]);
                pp[gq * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
                dd[gq * 2] = pack_bf16x2(dv[0], dv[1]);
                dd[gq * 2 + 1] = pack_bf16x2(dv[2], dv[3]);
              }
              const int unit = (cb2 * 4 + c) ^ (row & 7);
              if (!(PROF && (dbg & 2))) {
                *reinterpret_cast<uint4*>(sP + off + unit * 16) = make_uint4(pp[0], pp[1], pp[2], pp[3]);
                *reinterpret_cast<uint4*>(sDS + off + unit * 16) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
              }
              if (c < 3) tmem_ld_wait_on(rs[nxt], rd[nxt]);
            }
          };
          if (masked) softmax_grad(std::true_type{});
          else softmax_grad(std::false_type{});
          fence_proxy_async_smem();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&pds[g]);
          if constexpr (PROF) {
            const long long t2 = now();
            c_wait_sdp += t1 - t0; c_soft += t2 - t1; ++c_steps;
          }
        }
      } else {
        for (int it = 0; it < n_iters && ok; ++it) {
          const int gi = base + it, g = gi & 1;
          const int q0 = (2 * kv_tile + it % steps_per_head) * TQ;
          const int hq = hkv * group + it / steps_per_head;
          // the reduces of the previous step have read their boxes: P^T / dS^T of that buffer may be rewritten
          if (elected && gi >= 1) {
            bulk_wait_read_all();
            mbar_arrive(&stg_free[(gi - 1) & 1]);
          }
          // dQ^T partial of this step: lanes are head_dim, columns are the 64 queries; this warp reads 32 lanes x 32
          // queries and stages them as rows of its box; one thread adds the four boxes to the accumulator.  Boxes 0, 1
          // live in the step's P^T buffer, boxes 2, 3 in its dS^T buffer (both dead once dq_full has arrived).
          const long long t2 = now();
          if (!mbar_wait(&dq_full[g], (gi >> 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
          const long long t3 = now();
          tc_fence_after();
          uint32_t r0[16], r1[16];
          const uint32_t tcol = lane_addr + g * TQ + cb2 * 32;
          tmem_ld_32x16(tmem_base + Cfg::COL_DPT + tcol, r0);
          tmem_ld_32x16(tmem_base + Cfg::COL_DPT + tcol + 16, r1);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&dq_drained[g]);   // the buffer may be overwritten by the scores of step gi + 2
          uint8_t* my_box = (quarter < 2 ? sP : sDS) + g * Cfg::PT_BYTES + (quarter & 1) * (TQ * 128);
          if (!(PROF && (dbg & 1))) {
            // row q of box `quarter` = this warp's 32 floats of dQ[q][quarter * 32 ..]: one conflict-free 128-byte row
            // per store instruction (128-byte swizzle: 16-byte unit u of row r sits at u ^ (r & 7))
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int ql = cb2 * 32 + i;
              const float v = __uint_as_float(i < 16 ? r0[i & 15] : r1[i & 15]) * p.scale;
              *reinterpret_cast<float*>(my_box + ql * 128 + ((((lane >> 2) ^ (ql & 7))) << 4) + (lane & 3) * 4) = v;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&stg_full[g]);
          if (elected) {
            if (!mbar_wait(&stg_full[g], (gi >> 1) & 1, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
            if (!(PROF && (dbg & 1))) {
#pragma unroll
              for (int bx = 0; bx < 4; ++bx)   // rows past T are clipped by the tensor map
                tma_reduce_add_4d(&p.tm_dq, (bx < 2 ? sP : sDS) + g * Cfg::PT_BYTES + (bx & 1) * (TQ * 128), bx * 32, q0, hq, b);
            }
            bulk_commit();
          }
          if constexpr (PROF) {
            const long long t4 = now();
            c_wait_dq += t3 - t2; c_drain += t4 - t3;
          }
        }
      }
      if (!ok) break;
      const long long t5 = now();
      // dK and dV of this item: complete once the products of its last step have been committed
      {
        const int gl = base + n_iters - 1;
        if (!mbar_wait(&dq_full[gl & 1], (gl >> 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) break;
      }
      tc_fence_after();
      constexpr int DC = D / 4;   // 32 columns per warp
      __nv_bfloat16* dk_row = p.dk + (long long)b * p.dk_stride_b + (long long)kv_idx * p.dk_stride_t +
                              (long long)hkv * p.dk_stride_h + cb * DC;
      __nv_bfloat16* dv_row = p.dv + (long long)b * p.dv_stride_b + (long long)kv_idx * p.dv_stride_t +
                              (long long)hkv * p.dv_stride_h + cb * DC;
      uint32_t rk[2][16], rv[2][16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld_32x16(tmem_base + Cfg::COL_DK + lane_addr + cb * DC + c * 16, rk[c]);
        tmem_ld_32x16(tmem_base + Cfg::COL_DV + lane_addr + cb * DC + c * 16, rv[c]);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dkv_drained);   // the next item's products may overwrite dV / dK now
      if (kv_live) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          // 16 columns = 32 contiguous bytes per thread: one 256-bit store each where the address allows
          uint32_t ka[8], va[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            ka[e] = pack_bf16x2(__uint_as_float(rk[c][e * 2]) * p.scale, __uint_as_float(rk[c][e * 2 + 1]) * p.scale);
            va[e] = pack_bf16x2(__uint_as_float(rv[c][e * 2]), __uint_as_float(rv[c][e * 2 + 1]));
          }
          if (aligned32(dk_row) && aligned32(dv_row)) {
            st_global_b256(dk_row + c * 16, ka);
            st_global_b256(dv_row + c * 16, va);
          } else {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              *reinterpret_cast<uint4*>(dk_row + c * 16 + u * 8) = make_uint4(ka[u * 4], ka[u * 4 + 1], ka[u * 4 + 2], ka[u * 4 + 3]);
              *reinterpret_cast<uint4*>(dv_row + c * 16 + u * 8) = make_uint4(va[u * 4], va[u * 4 + 1], va[u * 4 + 2], va[u * 4 + 3]);
            }
          }
        }
      }
      base += n_iters;
      c_dkv += now() - t5;
    }
    if (PROF && lane == 0 && (warp == 2 || warp == 2 + FB_CWARPS / 2)) {   // one lane of each role
      auto add = [&](int i, long long v) { atomicAdd(reinterpret_cast<unsigned long long*>(p.prof + i), (unsigned long long)v); };
      if (role == 0) { add(8, now() - c_all); add(9, c_wait_sdp); add(10, c_soft); add(13, c_dkv); add(14, c_steps); }
      else { add(11, c_wait_dq); add(12, c_drain); }
    }
    if (elected) bulk_wait_all();   // the boxes stay valid until their reduces have completed
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
