// Causal online-softmax (flash) attention forward for sm_100a, GQA-aware.
//
// One CTA owns a 128-row query tile of one head.  K/V tiles stream in by TMA (local memory, no
// multicast); S = Q K^T is a tcgen05.mma into tensor memory; 128 softmax threads (one query row
// each, so row max / row sum need no shuffles) read S with tcgen05.ld, keep the running max and sum
// in the log2 domain, write P as bf16 into 128B-swizzled shared memory, and a second tcgen05.mma
// accumulates O += P V in tensor memory.  O is only rescaled when the running max grew by more than
// 2^8 (the final division by the row sum makes the result exact either way), and the rescale is a
// tcgen05.ld / tcgen05.st round trip over the 128 accumulator lanes.  Two CTAs fit per SM (96 KB
// shared memory, 256 TMEM columns each) so one CTA's exponentials overlap the other's MMAs.  Inside a CTA the
// next score product S_{j+1} is issued as soon as the softmax threads hold S_j in registers (barrier s_free), and
// O += P_j V_j signals its own barrier (pv_done), so both products run under the softmax math of the next tile.
//
// The reference has no attention kernel in use: its CPU path materialises softmax(QK^T s + mask) V
// (crates/incin-backends/src/cpu/ops/shape_ops.rs:1245-1269) and CUDA reports SDPA as unsupported;
// flash_attention_lite.cu there is dead code with one thread per query row.
#include "ptx.cuh"
#include "launch.cuh"
#include "../../include/incin_b200.h"
#include <math_constants.h>

namespace incin {

int make_operand_map(CUtensorMap* out, const void* ptr, long long inner, long long rows, long long ld,
                     long long batch_lo, long long stride_lo, long long batch_hi, long long stride_hi, int box_inner,
                     int box_rows);

constexpr int FA_BM = 128;
constexpr int FA_THREADS = 192;

template <int D, int BN>
struct FaCfg {
  static constexpr int Q_BYTES = FA_BM * D * 2;
  static constexpr int K_BYTES = BN * D * 2;
  static constexpr int V_BYTES = BN * D * 2;
  static constexpr int P_BYTES = FA_BM * BN * 2;
  static constexpr int K_STAGES = 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + K_STAGES * K_BYTES;
  static constexpr int OFF_P = OFF_V + V_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 256;  // S: [0, BN), O: [BN, BN + D)
};

struct FaParams {
  int T, Hq, Hkv, n_q_tiles;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* O;
  long long o_stride_b, o_stride_t, o_stride_h;
  float* lse;  // [B, Hq, Tpad], log2 domain; rows in [T, Tpad) are written as +inf
  int Tpad;
  int* status;
  int tile_major;   // 1: grid = (heads, batch, query tiles), else (query tiles, heads, batch)
};

template <int D, int BN>
__global__ void __launch_bounds__(FA_THREADS, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  using Cfg = FaCfg<D, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;         // 1
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]
  uint64_t* v_full = bars + 5;     // 1
  uint64_t* v_empty = bars + 6;    // 1
  uint64_t* s_full = bars + 7;     // 1: S_j is in tensor memory
  uint64_t* p_full = bars + 8;     // one arrival per softmax warp: P_j in shared memory, O rescaled
  uint64_t* s_free = bars + 9;     // one arrival per softmax warp: S_j has been read into registers
  uint64_t* pv_done = bars + 10;   // 1: O += P_j V_j has finished (P_j's shared memory and O may be touched again)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks are dispatched x-fastest.  Heavy (late) query tiles go first either way.  When K / V of all heads together
  // fit L2 (tile_major), the query tile is the slowest index: ALL heads' heaviest tiles start first and the light ones
  // fill the gaps at the end (longest-processing-time order over the whole launch; GPT-2 layer 0.050 -> 0.038 ms).
  // Otherwise a head's tiles stay together so that its K / V are read from DRAM once (with B 8, H 32, S 4096, D 128
  // the global order cost 19 %).
  const int q_tile = p.n_q_tiles - 1 - (int)(p.tile_major ? blockIdx.z : blockIdx.x);
  const int hq = p.tile_major ? blockIdx.x : blockIdx.y, b = p.tile_major ? blockIdx.y : blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = q_tile * FA_BM;
  int last_kv = q0 + FA_BM - 1;
  if (last_kv > p.T - 1) last_kv = p.T - 1;
  const int n_tiles = last_kv / BN + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);   // one arrival per softmax warp
    mbar_init(s_free, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + BN;
  pdl_launch_dependents();   // tensor memory is held; a successor may be scheduled as CTAs retire
  pdl_wait();                // no global memory was touched above

  if (warp == 0) {
    // producer: the whole warp walks the loop (warp-uniform waits and address arithmetic), one elected lane issues
    const bool leader = elect_one() != 0;
    {
      if (leader) {
        mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_4d(sQ + c * (FA_BM * 128), &tmQ, q_full, c * 64, q0, hq, b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int ks = j & 1;
        if (!mbar_wait(&k_empty[ks], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        if (leader) {
          mbar_expect_tx(&k_full[ks], Cfg::K_BYTES);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(sK + ks * Cfg::K_BYTES + c * (BN * 128), &tmK, &k_full[ks], c * 64, j * BN, hkv, b);
        }
        if (!mbar_wait(v_empty, (j & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        if (leader) {
          mbar_expect_tx(v_full, Cfg::V_BYTES);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) tma_load_4d(sV + c * (BN * 128), &tmV, v_full, c * 64, j * BN, hkv, b);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // issuer: the whole warp walks the loop, one elected lane executes the tcgen05 instructions
    const bool leader = elect_one() != 0;
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(FA_BM, BN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(FA_BM, D, false, true);
      // S_{j+1} = Q K_{j+1}^T is issued as soon as the softmax threads have S_j in registers, so it and O += P_j V_j
      // run while they work on the exponentials of tile j+1; the chain of a tile is then the softmax math alone.
      auto issue_s = [&](int j) -> bool {
        const int ks = j & 1;
        if (!mbar_wait(&k_full[ks], (j >> 1) & 1, abort_flag, p.status, kStatusTimeoutFull)) return false;
        if (j > 0 && !mbar_wait(s_free, (j - 1) & 1, abort_flag, p.status, kStatusTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK + ks * Cfg::K_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t ad = make_smem_desc(aq + (kk >> 2) * (FA_BM * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(bk + (kk >> 2) * (BN * 128) + (kk & 3) * 32, 16, 1024);
          if (leader) umma_f16_ss(tmem_S, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
        }
        if (leader) {
          umma_commit(&k_empty[ks]);
          umma_commit(s_full);
        }
        __syncwarp();
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusTimeoutFull);
      ok = ok && issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
        if (!mbar_wait(v_full, j & 1, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ap = smem_u32(sP), bv = smem_u32(sV);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t ad = make_smem_desc(ap + (kk >> 2) * (FA_BM * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(bv + kk * 2048, BN * 128, 1024);  // V^T: MN-major, 16 kv rows per step
          if (leader) umma_f16_ss(tmem_O, ad, bd, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        if (leader) {
          umma_commit(v_empty);
          umma_commit(pv_done);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // row inside the tile == TMEM lane
    const int q_idx = q0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_ref = -CUDART_INF_F, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN - 1 > q0) || (kv0 + BN > p.T);
      // whole S row into registers with back-to-back TMEM loads and a single wait
      uint32_t r[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c)
        tmem_ld_32x32(tmem_S + lane_addr + c * 32, reinterpret_cast<uint32_t(&)[32]>(r[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);   // the next score product may overwrite S
      if (need_mask) {  // masked scores become -inf, so the code below needs no further tests
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int kv = kv0 + i;
          if (!(kv <= q_idx && kv < p.T)) r[i] = __float_as_uint(-CUDART_INF_F);
        }
      }
      // row maximum with four independent chains
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(r[i]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(r[i + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(r[i + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(r[i + 3]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      // lazy rescale: only move the reference when the maximum grew by more than 2^8
      const bool need = mx > m_ref + 8.0f;
      float alpha = 1.0f;
      if (need) {
        alpha = exp2f(m_ref - mx);  // 0 on the first tile
        m_ref = mx;
        l_sum *= alpha;
      }
      // P = exp2(s * scale - m_ref) as packed bf16, kept in registers (in place of the scores they came from) while
      // O += P_{j-1} V_{j-1} may still be running; four independent sum chains
      const float neg_m = -m_ref;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < BN; i += 2) {
        const float e0 = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, neg_m));
        const float e1 = exp2f(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, neg_m));
        ls4[i & 3] += e0;
        ls4[(i & 3) + 1] += e1;
        r[i >> 1] = pack_bf16x2(e0, e1);
      }
      // that product must have finished before O is rescaled or P's shared memory is written again
      if (j > 0 && !mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_O + lane_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem_O + lane_addr + c * 32, o);
        }
        tmem_st_wait();
      }
      // P into 128B-swizzled shared memory: 16-byte unit ^ (row % 8)
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint8_t* prow = sP + (c >> 1) * (FA_BM * 128) + row * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int w0 = (c * 32 + u * 8) >> 1;
          const int unit = ((c & 1) * 4 + u) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + unit * 16) = make_uint4(r[w0], r[w0 + 1], r[w0 + 2], r[w0 + 3]);
        }
      }
      l_sum += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();                        // every lane's writes and fences precede the single arrival of its warp
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(pv_done, (n_tiles - 1) & 1, abort_flag, p.status, kStatusTimeoutTmemFull)) {
      tc_fence_after();
      const float inv = 1.0f / l_sum;
      const bool live_row = q_idx < p.T;
      __nv_bfloat16* orow = p.O + (long long)b * p.o_stride_b + (long long)q_idx * p.o_stride_t +
                            (long long)hq * p.o_stride_h;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_O + lane_addr + c * 32, r);
        tmem_ld_wait();
        if (live_row && aligned32(orow)) {   // 32 bytes per store: whole sectors of the row
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint32_t o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              o[e] = pack_bf16x2(__uint_as_float(r[u * 16 + e * 2]) * inv, __uint_as_float(r[u * 16 + e * 2 + 1]) * inv);
            st_global_b256(orow + c * 32 + u * 16, o);
          }
        } else if (live_row) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[u * 8 + 0]) * inv, __uint_as_float(r[u * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[u * 8 + 2]) * inv, __uint_as_float(r[u * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[u * 8 + 4]) * inv, __uint_as_float(r[u * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[u * 8 + 6]) * inv, __uint_as_float(r[u * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = o;
          }
        }
        __syncwarp();
      }
      p.lse[((long long)b * p.Hq + hq) * p.Tpad + q_idx] = live_row ? m_ref + log2f(l_sum) : CUDART_INF_F;
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

template <int D, int BN>
static int launch_fwd(const incin_attn_desc* d, cudaStream_t stream) {
  using Cfg = FaCfg<D, BN>;
  CUtensorMap tq, tk, tv;
  int rc = make_operand_map(&tq, d->q, D, d->T, d->q_stride_t, d->Hq, d->q_stride_h, d->B, d->q_stride_b, 64, FA_BM);
  if (rc) return rc;
  rc = make_operand_map(&tk, d->k, D, d->T, d->k_stride_t, d->Hkv, d->k_stride_h, d->B, d->k_stride_b, 64, BN);
  if (rc) return rc;
  rc = make_operand_map(&tv, d->v, D, d->T, d->v_stride_t, d->Hkv, d->v_stride_h, d->B, d->v_stride_b, 64, BN);
  if (rc) return rc;
  auto kern = flash_fwd_kernel<D, BN>;
  static PerDeviceFlags attr;
  if (!ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, attr)) return INCIN_ERR_LAUNCH;
  FaParams p;
  p.T = d->T;
  p.Hq = d->Hq;
  p.Hkv = d->Hkv;
  p.n_q_tiles = (d->T + FA_BM - 1) / FA_BM;
  p.scale_log2 = d->scale * 1.4426950408889634f;
  p.O = (__nv_bfloat16*)d->o;
  p.o_stride_b = d->o_stride_b;
  p.o_stride_t = d->o_stride_t;
  p.o_stride_h = d->o_stride_h;
  p.lse = d->lse;
  p.Tpad = p.n_q_tiles * FA_BM;
  p.status = (int*)d->status;
  // K and V of every (batch, kv head) against half of the 126 MB L2
  p.tile_major = ((long long)d->B * d->Hkv * d->T * D * 2 * 2 <= (48ll << 20)) ? 1 : 0;
  dim3 grid = p.tile_major ? dim3(d->Hq, d->B, p.n_q_tiles) : dim3(p.n_q_tiles, d->Hq, d->B);
  if (launch_pdl<true>(kern, grid, dim3(FA_THREADS), Cfg::SMEM_BYTES, stream, tq, tk, tv, p) != cudaSuccess) return INCIN_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? INCIN_OK : INCIN_ERR_LAUNCH;
}

}  // namespace incin

extern "C" int incin_flash_attn_fwd(const incin_attn_desc* d, void* stream) {
  if (!d || !d->q || !d->k || !d->v || !d->o || !d->lse || d->B <= 0 || d->T <= 0 || d->Hq <= 0 || d->Hkv <= 0 ||
      d->Hq % d->Hkv != 0)
    return INCIN_ERR_ARGUMENT;
  if ((d->o_stride_t % 8) || (d->o_stride_h % 8) || (d->o_stride_b % 8) || (reinterpret_cast<uintptr_t>(d->o) & 15))
    return INCIN_ERR_ALIGNMENT;
  if (d->D == 64) return incin::launch_fwd<64, 128>(d, (cudaStream_t)stream);
  if (d->D == 128) return incin::launch_fwd<128, 64>(d, (cudaStream_t)stream);
  return INCIN_ERR_UNSUPPORTED;
}
