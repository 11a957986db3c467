// Causal flash attention backward for sm_100a (dQ, dK, dV), GQA-aware.
//
// One CTA owns a 128-row K/V tile of one KV head and walks the query tiles at or below the diagonal
// (for every query head of the group).  Per query tile five tcgen05 GEMMs run, all with M = 128 and
// accumulators in tensor memory:
//     S^T  = K Q^T          dP^T = V dO^T                      (scores and their gradient, transposed)
//     dV  += P^T dO         dK  += dS^T Q                      (accumulate over query tiles in TMEM)
//     dQ_i = dS K                                             (per-tile partial, reduced with fp32 atomics)
// Computing the transposed scores puts the KV index in the TMEM lanes, so the 128 softmax threads
// (one KV row each) produce P^T and dS^T directly in the K-major layout the dV/dK GEMMs consume,
// and the same shared-memory tiles are re-read MN-major for dQ: no transposes anywhere.
// P is recomputed from the forward pass's log-sum-exp (log2 domain); delta = rowsum(O * dO) comes
// from a small preprocess kernel.  dQ partials are added into an fp32 scratch buffer the caller
// provides and converted to bf16 by a final strided cast.
//
// No counterpart in the reference (no attention backward exists there).
#include "ptx.cuh"
#include "launch.cuh"
#include "../../include/incin_b200.h"
#include <math_constants.h>
#include <cstdlib>
#include <type_traits>

namespace incin {

int make_f32_reduce_map(CUtensorMap* out, void* ptr, long long inner, long long rows, long long ld, long long batch_lo,
                        long long stride_lo, long long batch_hi, long long stride_hi, int box_rows);
int make_operand_map(CUtensorMap* out, const void* ptr, long long inner, long long rows, long long ld,
                     long long batch_lo, long long stride_lo, long long batch_hi, long long stride_hi, int box_inner,
                     int box_rows);

constexpr int FB_T = 128;  // tile edge for both the KV tile (TMEM lanes) and the query tile
constexpr int FB_CWARPS = 16;                       // compute warps: 4 TMEM lane quarters x 4 column blocks
constexpr int FB_CTHREADS = FB_CWARPS * 32;
constexpr int FB_THREADS = 64 + FB_CTHREADS;        // + TMA warp + MMA warp

template <int D>
struct FbCfg {
  static constexpr int STAGES = (D == 64) ? 2 : 1;
  static constexpr int TILE_BYTES = FB_T * D * 2;      // K, V, Q, dO tiles
  static constexpr int PT_BYTES = FB_T * FB_T * 2;     // P^T, dS^T tiles
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE_BYTES;
  static constexpr int OFF_Q = 2 * TILE_BYTES;
  static constexpr int OFF_DO = OFF_Q + STAGES * TILE_BYTES;
  static constexpr int OFF_P = OFF_DO + STAGES * TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + PT_BYTES;
  static constexpr int OFF_STAT = OFF_DS + PT_BYTES;   // lse[128], delta[128] per stage
  static constexpr int OFF_BAR = OFF_STAT + STAGES * 2 * FB_T * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // TMEM columns: S^T / dQ partial [0,128), dP^T [128,256), dV [256,256+D), dK [256+D, 256+2D)
  static constexpr int COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 256 + D, TMEM_COLS = 512;
  // D = 64 leaves 128 columns free: two dQ partial buffers of their own, so the dQ drain of tile i-1 and the
  // dV/dK/dQ MMAs of tile i-1 overlap the softmax-gradient math of tile i (PIPELINED).  With D = 128 tensor memory
  // is full and the dQ partial has to reuse the S^T columns, which serialises the iteration.
  static constexpr bool PIPELINED = (D == 64);
  static constexpr int COL_DQ = 256 + 2 * D;
};

struct FbParams {
  alignas(64) CUtensorMap tm_dq;   // fp32 dq_accum as {D, T, Hq, B}, 32 x 128 boxes (head_dim-64 kernel: bulk reduce-adds)
  int T, Hq, Hkv, n_tiles;
  int batch;           // B (the persistent kernel enumerates its work items itself)
  float scale, scale_log2;
  int Tpad;            // T rounded up to the tile edge: row stride of lse / delta
  const float* lse;    // [B, Hq, Tpad] log2 domain, +inf beyond T
  const float* delta;  // [B, Hq, Tpad], 0 beyond T
  float* dq_accum;     // [B, T, Hq, D] fp32, zero-initialised by the caller
  __nv_bfloat16 *dk, *dv;
  long long dk_stride_b, dk_stride_t, dk_stride_h, dv_stride_b, dv_stride_t, dv_stride_h;
  int* status;
  long long* prof;     // optional (INCIN_ATTN_PROF=1): clock counters of the issuer thread and of one compute lane
};

template <int D>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FbParams p) {
  using Cfg = FbCfg<D>;
  constexpr int ST = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDO = smem + Cfg::OFF_DO;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint8_t* sDS = smem + Cfg::OFF_DS;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;            // 1
  uint64_t* q_full = bars + 1;         // [ST]  Q_i and dO_i landed
  uint64_t* q_empty = bars + 1 + ST;   // [ST]  the three consuming MMAs of that stage finished
  uint64_t* sdp_full = bars + 1 + 2 * ST;  // S^T and dP^T in TMEM
  uint64_t* pds_full = sdp_full + 1;       // all compute threads: P^T and dS^T in shared memory
  uint64_t* dq_full = sdp_full + 2;        // [2] dQ partial in TMEM (and dV/dK updated); the serial flow uses [0]
  uint64_t* dq_drained = sdp_full + 4;     // [2] all compute threads: dQ partial read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sdp_full + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int kv0 = kv_tile * FB_T;
  const int first_q_tile = kv_tile;  // causal: query tiles at or below the diagonal
  const int tiles_per_head = p.n_tiles - first_q_tile;
  const int n_iters = tiles_per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, FB_CWARPS);   // one arrival per compute warp
    for (int i = 0; i < 2; ++i) {
      mbar_init(&dq_full[i], 1);
      mbar_init(&dq_drained[i], FB_CWARPS);
    }
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
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
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_4d(sK + c * (FB_T * 128), &tmK, kv_full, c * 64, kv0, hkv, b);
        tma_load_4d(sV + c * (FB_T * 128), &tmV, kv_full, c * 64, kv0, hkv, b);
      }
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % ST;
        const int hq = hkv * group + it / tiles_per_head;
        const int q0 = (first_q_tile + it % tiles_per_head) * FB_T;
        if (!mbar_wait(&q_empty[s], ((it / ST) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        mbar_expect_tx(&q_full[s], 2 * Cfg::TILE_BYTES + 2 * FB_T * 4);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(sQ + s * Cfg::TILE_BYTES + c * (FB_T * 128), &tmQ, &q_full[s], c * 64, q0, hq, b);
          tma_load_4d(sDO + s * Cfg::TILE_BYTES + c * (FB_T * 128), &tmDO, &q_full[s], c * 64, q0, hq, b);
        }
        // per-query statistics of this tile: two 512-byte bulk copies (rows are padded to the tile edge)
        const long long stat = ((long long)b * p.Hq + hq) * p.Tpad + q0;
        bulk_load_1d(sStat + s * 2 * FB_T, p.lse + stat, FB_T * 4, &q_full[s]);
        bulk_load_1d(sStat + s * 2 * FB_T + FB_T, p.delta + stat, FB_T * 4, &q_full[s]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_kk = make_idesc_bf16(FB_T, FB_T, false, false);  // S^T, dP^T
      constexpr uint32_t id_kmn = make_idesc_bf16(FB_T, D, false, true);     // dV, dK
      constexpr uint32_t id_mnmn = make_idesc_bf16(FB_T, D, true, true);     // dQ
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kStatusTimeoutFull);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP), aDS = smem_u32(sDS);
      if constexpr (Cfg::PIPELINED) {
        // one extra pass: pass `it` issues the dV/dK/dQ MMAs of tile it-1 and then the score MMAs of tile it
        for (int it = 0; it <= n_iters && ok; ++it) {
          if (it < n_iters) {
            if (!mbar_wait(&q_full[it % ST], (it / ST) & 1, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
          }
          if (it > 0) {
            const int j = it - 1, sj = j % ST, bq = j & 1;
            const uint32_t aQ = smem_u32(sQ + sj * Cfg::TILE_BYTES), aDO = smem_u32(sDO + sj * Cfg::TILE_BYTES);
            // tile j's P^T / dS^T are in shared memory, and its S^T / dP^T columns have been read
            if (!mbar_wait(pds_full, j & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
            if (j >= 2 && !mbar_wait(&dq_drained[bq], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutTmemEmpty)) {
              ok = false;
              break;
            }
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk) {
              const uint32_t a_off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
              const uint32_t b_off = kk * 2048;
              umma_f16_ss(tmem_base + Cfg::COL_DV, make_smem_desc(aP + a_off, 16, 1024),
                          make_smem_desc(aDO + b_off, FB_T * 128, 1024), id_kmn, (j > 0 || kk > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk) {
              const uint32_t a_off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
              const uint32_t b_off = kk * 2048;
              umma_f16_ss(tmem_base + Cfg::COL_DK, make_smem_desc(aDS + a_off, 16, 1024),
                          make_smem_desc(aQ + b_off, FB_T * 128, 1024), id_kmn, (j > 0 || kk > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < FB_T / 16; ++kk) {
              const uint32_t off = kk * 2048;
              umma_f16_ss(tmem_base + Cfg::COL_DQ + bq * D, make_smem_desc(aDS + off, FB_T * 128, 1024),
                          make_smem_desc(aK + off, FB_T * 128, 1024), id_mnmn, kk > 0 ? 1u : 0u);
            }
            umma_commit(&q_empty[sj]);
            umma_commit(&dq_full[bq]);
          }
          if (it < n_iters) {
            const int s = it % ST;
            const uint32_t aQ = smem_u32(sQ + s * Cfg::TILE_BYTES), aDO = smem_u32(sDO + s * Cfg::TILE_BYTES);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
              umma_f16_ss(tmem_base + Cfg::COL_ST, make_smem_desc(aK + off, 16, 1024), make_smem_desc(aQ + off, 16, 1024),
                          id_kk, kk > 0 ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
              umma_f16_ss(tmem_base + Cfg::COL_DPT, make_smem_desc(aV + off, 16, 1024),
                          make_smem_desc(aDO + off, 16, 1024), id_kk, kk > 0 ? 1u : 0u);
            }
            // arrives once everything issued so far has completed, the previous tile's dV/dK/dQ MMAs included: only
            // then may the compute threads overwrite P^T / dS^T in shared memory
            umma_commit(sdp_full);
          }
        }
      } else {
        for (int it = 0; it < n_iters && ok; ++it) {
          const int s = it % ST;
          const uint32_t aQ = smem_u32(sQ + s * Cfg::TILE_BYTES), aDO = smem_u32(sDO + s * Cfg::TILE_BYTES);
          if (!mbar_wait(&q_full[s], (it / ST) & 1, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
          // the S^T columns double as the dQ partial of the previous iteration: wait until it was read out
          if (!mbar_wait(dq_drained, (it & 1) ^ 1, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
          tc_fence_after();
  #pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
            umma_f16_ss(tmem_base + Cfg::COL_ST, make_smem_desc(aK + off, 16, 1024), make_smem_desc(aQ + off, 16, 1024),
                        id_kk, kk > 0 ? 1u : 0u);
          }
  #pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
            umma_f16_ss(tmem_base + Cfg::COL_DPT, make_smem_desc(aV + off, 16, 1024),
                        make_smem_desc(aDO + off, 16, 1024), id_kk, kk > 0 ? 1u : 0u);
          }
          umma_commit(sdp_full);
          if (!mbar_wait(pds_full, it & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
          tc_fence_after();
  #pragma unroll
          for (int kk = 0; kk < FB_T / 16; ++kk) {  // reduction over the 128 query rows of this tile
            const uint32_t a_off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;  // P^T / dS^T: K-major, K = q
            const uint32_t b_off = kk * 2048;                                  // dO / Q: MN-major, 16 q rows per step
            umma_f16_ss(tmem_base + Cfg::COL_DV, make_smem_desc(aP + a_off, 16, 1024),
                        make_smem_desc(aDO + b_off, FB_T * 128, 1024), id_kmn, (it > 0 || kk > 0) ? 1u : 0u);
          }
  #pragma unroll
          for (int kk = 0; kk < FB_T / 16; ++kk) {
            const uint32_t a_off = (kk >> 2) * (FB_T * 128) + (kk & 3) * 32;
            const uint32_t b_off = kk * 2048;
            umma_f16_ss(tmem_base + Cfg::COL_DK, make_smem_desc(aDS + a_off, 16, 1024),
                        make_smem_desc(aQ + b_off, FB_T * 128, 1024), id_kmn, (it > 0 || kk > 0) ? 1u : 0u);
          }
  #pragma unroll
          for (int kk = 0; kk < FB_T / 16; ++kk) {  // dQ = dS K: reduction over the 128 kv rows
            const uint32_t off = kk * 2048;          // both operands MN-major: 16 kv rows per step
            umma_f16_ss(tmem_base + Cfg::COL_ST, make_smem_desc(aDS + off, FB_T * 128, 1024),
                        make_smem_desc(aK + off, FB_T * 128, 1024), id_mnmn, kk > 0 ? 1u : 0u);
          }
          umma_commit(&q_empty[s]);
          umma_commit(dq_full);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax-gradient threads
    // warp -> (TMEM lane quarter = KV rows, column block = 32 query columns of the tile)
    const int cw = warp - 2;
    const int quarter = warp & 3;
    const int cb = cw >> 2;
    const int row = quarter * 32 + lane;
    const int kv_idx = kv0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool kv_live = kv_idx < p.T;
    // dQ partial of tile j: lanes are query rows of that tile; this warp adds D/4 of the columns into the fp32
    // accumulator.  Pipelined flow: buffer j & 1 of the dedicated dQ columns; serial flow: the S^T columns.
    auto drain_dq = [&](int j) -> bool {
      const int bq = Cfg::PIPELINED ? (j & 1) : 0;
      const uint32_t parity = Cfg::PIPELINED ? ((j >> 1) & 1) : (j & 1);
      if (!mbar_wait(&dq_full[bq], parity, abort_flag, p.status, kStatusTimeoutTmemFull)) return false;
      tc_fence_after();
      const int hq_j = hkv * group + j / tiles_per_head;
      const int q = (first_q_tile + j % tiles_per_head) * FB_T + row;
      constexpr int DC = D / 4;  // columns per warp: 16 (D = 64) or 32 (D = 128)
      const uint32_t col = Cfg::PIPELINED ? (Cfg::COL_DQ + bq * D) : Cfg::COL_ST;
      float* dq_row = p.dq_accum + (((long long)b * p.T + q) * p.Hq + hq_j) * D + cb * DC;
      if constexpr (DC == 16) {
        uint32_t r[16];
        tmem_ld_32x16(tmem_base + col + lane_addr + cb * DC, r);
        tmem_ld_wait();
        if (q < p.T) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq_row + u * 4),
                         "f"(__uint_as_float(r[u * 4]) * p.scale), "f"(__uint_as_float(r[u * 4 + 1]) * p.scale),
                         "f"(__uint_as_float(r[u * 4 + 2]) * p.scale), "f"(__uint_as_float(r[u * 4 + 3]) * p.scale)
                         : "memory");
        }
      } else {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + col + lane_addr + cb * DC, r);
        tmem_ld_wait();
        if (q < p.T) {
#pragma unroll
          for (int u = 0; u < 8; ++u)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq_row + u * 4),
                         "f"(__uint_as_float(r[u * 4]) * p.scale), "f"(__uint_as_float(r[u * 4 + 1]) * p.scale),
                         "f"(__uint_as_float(r[u * 4 + 2]) * p.scale), "f"(__uint_as_float(r[u * 4 + 3]) * p.scale)
                         : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_drained[bq]);
      return true;
    };
    bool ok = true;
    for (int it = 0; it < n_iters; ++it) {
      const int s = it % ST;
      const int q0 = (first_q_tile + it % tiles_per_head) * FB_T;
      const float* s_lse = sStat + s * 2 * FB_T + cb * 32;
      const float* s_delta = s_lse + FB_T;
      // q_full also covers the statistics; the MMA thread waited on it before sdp_full can complete
      if (!mbar_wait(sdp_full, it & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      // Only the diagonal tile needs the causal test and only the last KV tile can hold dead rows: every other tile
      // takes the unmasked instantiation (three instructions fewer per element in an issue-bound loop).
      auto softmax_grad = [&](auto masked_tag) {
        constexpr bool MASKED = decltype(masked_tag)::value;
  #pragma unroll
        for (int hf = 0; hf < 2; ++hf) {  // two halves of 16 query columns keep the register footprint small
          uint32_t rs[16], rd[16];
          tmem_ld_32x16(tmem_base + Cfg::COL_ST + lane_addr + cb * 32 + hf * 16, rs);
          tmem_ld_32x16(tmem_base + Cfg::COL_DPT + lane_addr + cb * 32 + hf * 16, rd);
          tmem_ld_wait();
          uint32_t pp[8], dd[8];
  #pragma unroll
          for (int g = 0; g < 4; ++g) {
            const float4 l4 = *reinterpret_cast<const float4*>(s_lse + hf * 16 + g * 4);
            const float4 d4 = *reinterpret_cast<const float4*>(s_delta + hf * 16 + g * 4);
            const float lse[4] = {l4.x, l4.y, l4.z, l4.w};
            const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
            float pv[4], dv[4];
  #pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = g * 4 + e;
              const int qi = cb * 32 + hf * 16 + i;
              float pr = exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse[e]));
              if constexpr (MASKED) pr = (kv_live && (q0 + qi >= kv_idx)) ? pr : 0.f;
              pv[e] = pr;
              dv[e] = pr * (__uint_as_float(rd[i]) - dl[e]);   // the softmax scale is applied when dQ / dK leave TMEM
            }
            pp[g * 2] = pack_bf16x2(pv[0], pv[1]);
            pp[g * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
            dd[g * 2] = pack_bf16x2(dv[0], dv[1]);
            dd[g * 2 + 1] = pack_bf16x2(dv[2], dv[3]);
          }
          uint8_t* prow = sP + (cb >> 1) * (FB_T * 128) + row * 128;
          uint8_t* drow = sDS + (cb >> 1) * (FB_T * 128) + row * 128;
  #pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int unit = ((cb & 1) * 4 + hf * 2 + u) ^ (row & 7);
            *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(pp[u * 4], pp[u * 4 + 1], pp[u * 4 + 2], pp[u * 4 + 3]);
            *reinterpret_cast<uint4*>(drow + unit * 16) = make_uint4(dd[u * 4], dd[u * 4 + 1], dd[u * 4 + 2], dd[u * 4 + 3]);
          }
        }
      };
      if (q0 < kv0 + FB_T || kv0 + FB_T > p.T) softmax_grad(std::true_type{});
      else softmax_grad(std::false_type{});
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();                          // every lane's writes and fences precede the single arrival of its warp
      if (lane == 0) mbar_arrive(pds_full);
      if constexpr (Cfg::PIPELINED) {
        if (it > 0 && !drain_dq(it - 1)) { ok = false; break; }   // overlaps the MMAs the issuer has just launched
      } else {
        if (!drain_dq(it)) { ok = false; break; }
      }
    }
    if constexpr (Cfg::PIPELINED) {
      if (ok && n_iters > 0) ok = drain_dq(n_iters - 1);
    }
    // final: dK and dV of this KV tile (dq_full of the last iteration implies both are complete)
    if (ok && n_iters > 0) {
      tc_fence_after();
      constexpr int DC = D / 4;
      __nv_bfloat16* dk_row = p.dk + (long long)b * p.dk_stride_b + (long long)kv_idx * p.dk_stride_t +
                              (long long)hkv * p.dk_stride_h + cb * DC;
      __nv_bfloat16* dv_row = p.dv + (long long)b * p.dv_stride_b + (long long)kv_idx * p.dv_stride_t +
                              (long long)hkv * p.dv_stride_h + cb * DC;
#pragma unroll
      for (int c = 0; c < DC / 16; ++c) {
        uint32_t rk[16], rv[16];
        tmem_ld_32x16(tmem_base + Cfg::COL_DK + lane_addr + cb * DC + c * 16, rk);
        tmem_ld_32x16(tmem_base + Cfg::COL_DV + lane_addr + cb * DC + c * 16, rv);
        tmem_ld_wait();
        if (kv_live) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint4 a, bb;
            a.x = pack_bf16x2(__uint_as_float(rk[u * 8 + 0]) * p.scale, __uint_as_float(rk[u * 8 + 1]) * p.scale);
            a.y = pack_bf16x2(__uint_as_float(rk[u * 8 + 2]) * p.scale, __uint_as_float(rk[u * 8 + 3]) * p.scale);
            a.z = pack_bf16x2(__uint_as_float(rk[u * 8 + 4]) * p.scale, __uint_as_float(rk[u * 8 + 5]) * p.scale);
            a.w = pack_bf16x2(__uint_as_float(rk[u * 8 + 6]) * p.scale, __uint_as_float(rk[u * 8 + 7]) * p.scale);
            bb.x = pack_bf16x2(__uint_as_float(rv[u * 8 + 0]), __uint_as_float(rv[u * 8 + 1]));
            bb.y = pack_bf16x2(__uint_as_float(rv[u * 8 + 2]), __uint_as_float(rv[u * 8 + 3]));
            bb.z = pack_bf16x2(__uint_as_float(rv[u * 8 + 4]), __uint_as_float(rv[u * 8 + 5]));
            bb.w = pack_bf16x2(__uint_as_float(rv[u * 8 + 6]), __uint_as_float(rv[u * 8 + 7]));
            *reinterpret_cast<uint4*>(dk_row + c * 16 + u * 8) = a;
            *reinterpret_cast<uint4*>(dv_row + c * 16 + u * 8) = bb;
          }
        }
        __syncwarp();
      }
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

// delta[b, h, t] = sum_d O[b,t,h,d] * dO[b,t,h,d] (0 for the padding rows t >= T).  A row (b, t, h) is D bf16 =
// LPR 16-byte loads, one per lane of a group of LPR = D / 8 lanes; every group takes DELTA_ROWS rows with all their
// loads issued before the first is used, so that a thread keeps 2 x DELTA_ROWS 16-byte loads in flight.
constexpr int DELTA_ROWS = 4;
// IDX is the type of the row / element counters: 32-bit whenever the problem allows, because the 64-bit divisions that
// split a counter into (b, t, h) otherwise cost more than the loads.
template <int LPR, typename IDX>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                  long long B, int T, int Tpad, int H, long long o_sb, long long o_st, long long o_sh,
                  long long do_sb, long long do_st, long long do_sh) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int GROUPS = 256 / LPR;                       // row groups per block
  const int sub = threadIdx.x % LPR;
  const IDX total = (IDX)(B * Tpad * H);
  const IDX first = ((IDX)blockIdx.x * GROUPS + threadIdx.x / LPR) * DELTA_ROWS;
  // (b, t, h) of the first row; the following rows step h, then t, then b
  int h0 = (int)(first % (IDX)H);
  int t0 = (int)((first / (IDX)H) % (IDX)Tpad);
  long long b0 = (long long)(first / ((IDX)H * (IDX)Tpad));
  uint4 a[DELTA_ROWS], c[DELTA_ROWS];
  {
    int h = h0, t = t0;
    long long b = b0;
#pragma unroll
    for (int r = 0; r < DELTA_ROWS; ++r) {
      a[r] = make_uint4(0, 0, 0, 0);
      c[r] = make_uint4(0, 0, 0, 0);
      if (first + (IDX)r < total && t < T) {
        a[r] = *reinterpret_cast<const uint4*>(o + b * o_sb + (long long)t * o_st + (long long)h * o_sh + sub * 8);
        c[r] = *reinterpret_cast<const uint4*>(d_o + b * do_sb + (long long)t * do_st + (long long)h * do_sh + sub * 8);
      }
      if (++h == H) {
        h = 0;
        if (++t == Tpad) {
          t = 0;
          ++b;
        }
      }
    }
  }
  int h = h0, t = t0;
  long long b = b0;
#pragma unroll
  for (int r = 0; r < DELTA_ROWS; ++r) {
    const uint32_t ua[4] = {a[r].x, a[r].y, a[r].z, a[r].w}, uc[4] = {c[r].x, c[r].y, c[r].z, c[r].w};
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = unpack_bf16x2(ua[e]), y = unpack_bf16x2(uc[e]);
      s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (sub == 0 && first + (IDX)r < total) delta[(b * H + h) * Tpad + t] = s;
    if (++h == H) {
      h = 0;
      if (++t == Tpad) {
        t = 0;
        ++b;
      }
    }
  }
}

// dq (bf16, strided) = dq_accum (fp32 [B,T,H,D] contiguous); 8 elements (two 16-byte loads, one 16-byte store) per
// thread and step, two steps in flight
template <typename IDX>
__global__ void __launch_bounds__(256)
attn_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long B, int T,
                    int H, int D, long long sb, long long st, long long sh) {
  pdl_launch_dependents();
  pdl_wait();
  const IDX n8 = (IDX)(B * T * H * D / 8);
  const IDX stride = (IDX)gridDim.x * blockDim.x;
  const IDX d8 = (IDX)(D / 8);
  auto store = [&](IDX i, const float4& v0, const float4& v1) {
    const int d = (int)(i % d8) * 8;
    const IDX row = i / d8;                       // (b, t, h)
    const int h = (int)(row % (IDX)H);
    const IDX bt = row / (IDX)H;
    const int t = (int)(bt % (IDX)T);
    const long long b = (long long)(bt / (IDX)T);
    uint4 o;
    o.x = pack_bf16x2(v0.x, v0.y);
    o.y = pack_bf16x2(v0.z, v0.w);
    o.z = pack_bf16x2(v1.x, v1.y);
    o.w = pack_bf16x2(v1.z, v1.w);
    *reinterpret_cast<uint4*>(dq + b * sb + (long long)t * st + (long long)h * sh + d) = o;
  };
  const float4* src = reinterpret_cast<const float4*>(acc);
  IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < n8; i += 2 * stride) {
    const float4 a0 = src[2 * (long long)i], a1 = src[2 * (long long)i + 1];
    const float4 b0 = src[2 * (long long)(i + stride)], b1 = src[2 * (long long)(i + stride) + 1];
    store(i, a0, a1);
    store(i + stride, b0, b1);
  }
  if (i < n8) store(i, src[2 * (long long)i], src[2 * (long long)i + 1]);
}

// Where the backward spends its time: with INCIN_ATTN_PROF=1 the head_dim-64 kernel adds up, per launch, the clock
// cycles its MMA issuer spends waiting on each barrier and issuing, and those one compute lane spends waiting and
// computing.  Read (and cleared) with incin_attn_prof_read.  Off by default: the pointer is null.
static long long* attn_prof_buffer() {
  static long long* buf = [] () -> long long* {
    const char* e = std::getenv("INCIN_ATTN_PROF");
    if (!(e && e[0] == '1')) return nullptr;
    long long* b = nullptr;
    if (cudaMalloc(&b, 16 * sizeof(long long)) != cudaSuccess) return nullptr;
    cudaMemset(b, 0, 16 * sizeof(long long));
    return b;
  }();
  return buf;
}

}  // namespace incin
#include "attention_bwd64.cuh"
#include "attention_bwd128.cuh"
namespace incin {

template <int D>
static int launch_bwd(const incin_attn_desc* d, cudaStream_t stream) {
  using Cfg = FbCfg<D>;
  // head_dim 64 runs the half-split kernel and head_dim 128 the kernel pipelined over 64-query steps (tensor core and
  // softmax-gradient threads overlap in both); INCIN_ATTN_BWD_SPLIT=0 selects the one-tile-at-a-time kernel instead
  static const bool split_on = [] {
    const char* e = std::getenv("INCIN_ATTN_BWD_SPLIT");
    return !(e && e[0] == '0');
  }();
  const bool use_split = (D == 64) && split_on;
  const bool use_steps = (D == 128) && split_on;
  const int q_box_rows = use_steps ? Fb128::TQ : FB_T;   // rows of one Q / dO load
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_operand_map(&tq, d->q, D, d->T, d->q_stride_t, d->Hq, d->q_stride_h, d->B, d->q_stride_b, 64, q_box_rows);
  if (rc) return rc;
  rc = make_operand_map(&tk, d->k, D, d->T, d->k_stride_t, d->Hkv, d->k_stride_h, d->B, d->k_stride_b, 64, FB_T);
  if (rc) return rc;
  rc = make_operand_map(&tv, d->v, D, d->T, d->v_stride_t, d->Hkv, d->v_stride_h, d->B, d->v_stride_b, 64, FB_T);
  if (rc) return rc;
  rc = make_operand_map(&tdo, d->d_o, D, d->T, d->do_stride_t, d->Hq, d->do_stride_h, d->B, d->do_stride_b, 64, q_box_rows);
  if (rc) return rc;
  // O is read and dQ written 16 bytes at a time
  if ((reinterpret_cast<uintptr_t>(d->o) & 15) || (reinterpret_cast<uintptr_t>(d->dq) & 15) || (d->o_stride_t % 8) ||
      (d->o_stride_h % 8) || (d->o_stride_b % 8) || (d->dq_stride_t % 8) || (d->dq_stride_h % 8) || (d->dq_stride_b % 8))
    return INCIN_ERR_ALIGNMENT;
  const bool prof = (use_split || use_steps) && attn_prof_buffer() != nullptr;
  auto kern = use_split ? (prof ? flash_bwd64_kernel<true> : flash_bwd64_kernel<false>)
                        : (use_steps ? (prof ? flash_bwd128_kernel<true> : flash_bwd128_kernel<false>) : flash_bwd_kernel<D>);
  const int smem_bytes = use_split ? Fb64::SMEM_BYTES : (use_steps ? Fb128::SMEM_BYTES : Cfg::SMEM_BYTES);
  static PerDeviceFlags attr[5];
  const int which = use_split ? (prof ? 2 : 1) : (use_steps ? (prof ? 4 : 3) : 0);
  if (!ensure_dynamic_smem(kern, smem_bytes, attr[which])) return INCIN_ERR_LAUNCH;
  const long long rows = (long long)d->B * d->T * d->Hq;
  const int Tpad = (d->T + FB_T - 1) / FB_T * FB_T;
  const long long prow = (long long)d->B * Tpad * d->Hq;
  const bool idx32 = prow * D < (1ll << 30);   // row and element counters (and their strides) fit 32 bits
  {
    constexpr int LPR = D / 8, ROWS_PER_BLOCK = 256 / LPR * DELTA_ROWS;
    auto go = [&](auto kern) {
      return launch_pdl(kern, dim3((unsigned)((prow + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK)), dim3(256), 0, stream,
                        (const __nv_bfloat16*)d->o, (const __nv_bfloat16*)d->d_o, d->delta, (long long)d->B, (int)d->T, Tpad,
                        (int)d->Hq, (long long)d->o_stride_b, (long long)d->o_stride_t, (long long)d->o_stride_h,
                        (long long)d->do_stride_b, (long long)d->do_stride_t, (long long)d->do_stride_h);
    };
    if ((idx32 ? go(attn_delta_kernel<LPR, unsigned>) : go(attn_delta_kernel<LPR, long long>)) != cudaSuccess)
      return INCIN_ERR_LAUNCH;
  }
  if (cudaMemsetAsync(d->dq_accum, 0, sizeof(float) * rows * D, stream) != cudaSuccess) return INCIN_ERR_LAUNCH;
  FbParams p;
  p.T = d->T;
  p.Hq = d->Hq;
  p.Hkv = d->Hkv;
  p.n_tiles = (d->T + FB_T - 1) / FB_T;
  p.batch = d->B;
  p.Tpad = Tpad;
  p.scale = d->scale;
  p.scale_log2 = d->scale * 1.4426950408889634f;
  p.lse = d->lse;
  p.delta = d->delta;
  p.dq_accum = d->dq_accum;
  if (use_split || use_steps) {   // dQ partials leave through bulk tensor reduces of 32-column boxes
    rc = make_f32_reduce_map(&p.tm_dq, d->dq_accum, D, d->T, (long long)d->Hq * D, d->Hq, D, d->B,
                             (long long)d->T * d->Hq * D, use_steps ? Fb128::TQ : FB_T);
    if (rc) return rc;
  }
  p.dk = (__nv_bfloat16*)d->dk;
  p.dv = (__nv_bfloat16*)d->dv;
  p.dk_stride_b = d->dk_stride_b;
  p.dk_stride_t = d->dk_stride_t;
  p.dk_stride_h = d->dk_stride_h;
  p.dv_stride_b = d->dv_stride_b;
  p.dv_stride_t = d->dv_stride_t;
  p.dv_stride_h = d->dv_stride_h;
  p.status = (int*)d->status;
  p.prof = attn_prof_buffer();
  dim3 grid(p.n_tiles, d->Hkv, d->B);
  if (use_split || use_steps) {   // persistent: one CTA per SM (or per item when there are fewer items)
    const long long items = (long long)p.n_tiles * d->Hkv * d->B;
    static const int sms = [] { int dev = 0, n = 148; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); return n; }();
    grid = dim3((unsigned)(items < sms ? items : sms), 1, 1);
  }
  if (launch_pdl<true>(kern, grid, dim3(FB_THREADS), smem_bytes, stream, tq, tk, tv, tdo, p) != cudaSuccess) return INCIN_ERR_LAUNCH;
  long long n8 = rows * D / 8;
  long long blocks = (n8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  auto cast = [&](auto kern) {
    return launch_pdl(kern, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)d->dq_accum, (__nv_bfloat16*)d->dq,
                      (long long)d->B, (int)d->T, (int)d->Hq, D, (long long)d->dq_stride_b, (long long)d->dq_stride_t,
                      (long long)d->dq_stride_h);
  };
  if ((idx32 ? cast(attn_dq_cast_kernel<unsigned>) : cast(attn_dq_cast_kernel<long long>)) != cudaSuccess)
    return INCIN_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace incin

// Experiment switches of the profiling instantiation of the head_dim-128 backward (slot 15 of the profile buffer);
// only has an effect with INCIN_ATTN_PROF=1.
extern "C" int incin_attn_prof_flags(long long flags) {
  long long* b = incin::attn_prof_buffer();
  if (!b) return INCIN_ERR_UNSUPPORTED;
  return cudaMemcpy(b + 15, &flags, sizeof(long long), cudaMemcpyHostToDevice) == cudaSuccess ? INCIN_OK : INCIN_ERR_DRIVER;
}

extern "C" int incin_attn_prof_read(long long* out16) {
  long long* b = incin::attn_prof_buffer();
  if (!b || !out16) return INCIN_ERR_UNSUPPORTED;
  if (cudaMemcpy(out16, b, 16 * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess) return INCIN_ERR_DRIVER;
  cudaMemset(b, 0, 15 * sizeof(long long));   // slot 15 holds the experiment switches
  return INCIN_OK;
}

extern "C" int incin_flash_attn_bwd(const incin_attn_desc* d, void* stream) {
  if (!d || !d->q || !d->k || !d->v || !d->o || !d->d_o || !d->lse || !d->delta || !d->dq_accum || !d->dq ||
      !d->dk || !d->dv || d->B <= 0 || d->T <= 0 || d->Hq <= 0 || d->Hkv <= 0 || d->Hq % d->Hkv != 0)
    return INCIN_ERR_ARGUMENT;
  if (d->D == 64) return incin::launch_bwd<64>(d, (cudaStream_t)stream);
  if (d->D == 128) return incin::launch_bwd<128>(d, (cudaStream_t)stream);
  return INCIN_ERR_UNSUPPORTED;
}
