// Definitions shared by the single-CTA and the CTA-pair tcgen05 GEMM kernels: tile constants, kernel parameters,
// the persistent tile order, and the fused epilogue of one 32-column accumulator chunk.
#pragma once
#include "ptx.cuh"
#include "launch.cuh"
#include "../../include/incin_b200.h"

namespace incin {

constexpr int BM = 128;
constexpr int BK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;  // warp0: TMA, warp1: MMA + TMEM owner, warps 2-9: epilogue (two per TMEM lane quarter)
constexpr int SMEM_BUDGET = 224 * 1024;   // of the 227 KB a CTA may use; the rest holds barriers and alignment slack
// Output staging: every epilogue warp owns 32 rows x 128 bytes (64 bf16 or 32 fp32 columns) of shared memory, written
// row-per-lane in the 128-byte swizzle and sent to global memory by one bulk tensor store (or reduce-add) per box.
constexpr int EPI_WARPS = 8;
constexpr int STG_WARP_BYTES = 32 * 128;
constexpr int STG_BYTES = EPI_WARPS * STG_WARP_BYTES;   // 32 KB
// Fused-collective launches of the single-CTA kernel may carry one more warp per CTA that moves the collective's data
// (see the copy warp in gemm_tcgen05.cu); every other launch runs with GEMM_THREADS.
constexpr int GEMM_COPY_WARP = 2 + EPI_WARPS;
constexpr int GEMM_THREADS_COPY = GEMM_THREADS + 32;

// STG: the variant with the 32 KB output staging area (one operand stage fewer for every tile but 128 x 256, whose
// four 48 KB stages leave that much room anyway)
template <int BN, bool STG = true>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (SMEM_BUDGET - (STG ? STG_BYTES : 0)) / STAGE_BYTES;
  static constexpr int ACC_STRIDE = (BN <= 64) ? 64 : (BN <= 128 ? 128 : 256);
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr int STG_OFF = STAGES * STAGE_BYTES;                  // 1024-byte aligned (stages are multiples of 8 KB)
  static constexpr int BAR_OFF = STG_OFF + (STG ? STG_BYTES : 0);
  static constexpr int SMEM_BYTES = BAR_OFF + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmKernelParams {
  int M, N, K;
  int batch_lo, batch_hi;
  int tiles_m, tiles_n, splits, total_units;
  void* C;
  long long ldc, c_stride_lo, c_stride_hi;
  int out_fp32, accumulate;
  float alpha;
  const float* alpha_ptr;   // optional device scalar multiplied into alpha (an upstream gradient that lives on the GPU)
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int act;
  __nv_bfloat16* aux;
  int* status;
  int in_kind;            // operands: 0 bf16, 1 fp16, 2 fp32 multiplied as tf32 (K counted in 2-byte units)
  // all-gather -> GEMM
  int ag_world, ag_rank, ag_rows_per_rank, gemm_ctas;  // gemm_ctas: CTAs [0, gemm_ctas) compute, the rest copy
  const __nv_bfloat16* ag_src[8];
  uint32_t* ag_flags;
  __nv_bfloat16* ag_gathered;
  // GEMM -> reduce-scatter
  int rs_world, rs_rank, rs_rows_per_rank;
  int rs_push;            // 1: remote tiles go to the local staging buffer C and copy CTAs push them to their owners
  __nv_bfloat16* rs_dst[8];
  long long rs_slot_stride;
  uint32_t* rs_ready;     // push mode: per 128-row block, epilogue warps that have finished writing it
  // n > 0: the collective's data is moved by one extra warp in every compute CTA (chunks of 8 KB through a ring made
  // of the last n operand stages) instead of by dedicated copy CTAs; ag_flags then count chunks per 128-row tile
  int wide_io;   // 1: 256-bit global loads / stores in the epilogue where the address allows (INCIN_GEMM_B256, default 1)
  int copy_warps;
  uint32_t ag_flag_target;   // value of ag_flags[tile] at which the tile is complete
  int ag_own_in_place;       // 1: this rank's own rows are already in the gathered buffer (nothing copies or waits for them)
  // 1: the epilogue stages its output in shared memory and writes C (and the pre-activation side output) with bulk
  // tensor stores / reduce-adds through the tensor maps passed beside the operands' (dense rows, aligned base)
  int tma_out;
};

struct Unit {
  int m_blk, n_blk, b_lo, b_hi, kb0, kb1;
};

__device__ __forceinline__ Unit decode_unit(const GemmKernelParams& p, int u) {
  Unit w;
  const int split = u % p.splits;
  int t = u / p.splits;
  int b;
  if (p.ag_world > 1) {
    // tiles of one 128-row block are consecutive (one flag wait serves them all) and the row blocks are visited
    // in arrival order: own shard first, then the peers' shards in the order the copy CTAs fetch them
    w.n_blk = t % p.tiles_n;
    t /= p.tiles_n;
    const int mi = t % p.tiles_m;
    w.m_blk = (mi + p.ag_rank * (p.ag_rows_per_rank / BM)) % p.tiles_m;
    b = t / p.tiles_m;
  } else if (p.rs_push) {
    // row blocks owned by the next rank first, own rows last: the copy CTAs push finished blocks while the
    // remaining ones are still being computed, and nothing has to leave this GPU after the last tile
    w.n_blk = t % p.tiles_n;
    t /= p.tiles_n;
    const int mi = t % p.tiles_m;
    w.m_blk = (mi + (p.rs_rank + 1) * (p.rs_rows_per_rank / BM)) % p.tiles_m;
    b = t / p.tiles_m;
  } else {
    w.m_blk = t % p.tiles_m;
    t /= p.tiles_m;
    w.n_blk = t % p.tiles_n;
    b = t / p.tiles_n;
  }
  w.b_lo = b % p.batch_lo;
  w.b_hi = b / p.batch_lo;
  const int kb_total = (p.K + BK - 1) / BK;
  w.kb0 = static_cast<int>((static_cast<long long>(split) * kb_total) / p.splits);
  w.kb1 = static_cast<int>((static_cast<long long>(split + 1) * kb_total) / p.splits);
  return w;
}

// Values of one accumulator chunk: thread = one output row, r = its 32 consecutive fp32 accumulator columns starting
// at column nc.  alpha, bias, GELU / SiLU, activation-gradient masks, residual.  With STAGE_PRE the pre-activation
// (the side output kept for the backward pass) is returned in pre[] for the caller to store; otherwise it is written
// to p.aux here with per-thread stores.  row_ok = false (a row beyond M) skips every per-row global access.
template <bool STAGE_PRE>
__device__ __forceinline__ void epilogue_values(const GemmKernelParams& p, const uint32_t (&r)[32], long long cbase, int nc,
                                                bool vec_ok, float alpha, bool row_ok, float (&v)[32], float (&pre)[32]) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
        const bool full = (nc + 32 <= p.N) && vec_ok;
        if (p.bias) {
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 bb = *reinterpret_cast<const uint4*>(p.bias + nc + q * 8);
              const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = unpack_bf16x2(bw[e]);
                v[q * 8 + e * 2] += f.x;
                v[q * 8 + e * 2 + 1] += f.y;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) v[j] += __bfloat162float(p.bias[nc + j]);
          }
        }
        if (p.act == INCIN_ACT_GELU || p.act == INCIN_ACT_SILU) {
          if (STAGE_PRE) {
#pragma unroll
            for (int j = 0; j < 32; ++j) pre[j] = v[j];
          } else if (p.aux && row_ok) {  // keep the pre-activation for the backward pass
            __nv_bfloat16* ax = p.aux + cbase + nc;
            if (full && p.wide_io && aligned32(ax)) {
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                uint32_t o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = pack_bf16x2(v[q * 16 + e * 2], v[q * 16 + e * 2 + 1]);
                st_global_b256(ax + q * 16, o);
              }
            } else if (full) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
                *reinterpret_cast<uint4*>(ax + q * 8) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) ax[j] = __float2bfloat16(v[j]);
            }
          }
          if (p.act == INCIN_ACT_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
          }
        } else if ((p.act == INCIN_ACT_DGELU || p.act == INCIN_ACT_DSILU) && row_ok) {
          // multiply by act'(pre-activation): fuses the activation backward into the data-gradient GEMM
          const __nv_bfloat16* ax = p.aux + cbase + nc;
          if (full && p.wide_io && aligned32(ax)) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint32_t bw[8];
              ld_global_b256(ax + q * 16, bw);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float2 f = unpack_bf16x2(bw[e]);
                if (p.act == INCIN_ACT_DGELU) {
                  v[q * 16 + e * 2] *= gelu_erf_grad(f.x);
                  v[q * 16 + e * 2 + 1] *= gelu_erf_grad(f.y);
                } else {
                  v[q * 16 + e * 2] *= silu_grad(f.x);
                  v[q * 16 + e * 2 + 1] *= silu_grad(f.y);
                }
              }
            }
          } else if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 bb = *reinterpret_cast<const uint4*>(ax + q * 8);
              const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = unpack_bf16x2(bw[e]);
                if (p.act == INCIN_ACT_DGELU) {
                  v[q * 8 + e * 2] *= gelu_erf_grad(f.x);
                  v[q * 8 + e * 2 + 1] *= gelu_erf_grad(f.y);
                } else {
                  v[q * 8 + e * 2] *= silu_grad(f.x);
                  v[q * 8 + e * 2 + 1] *= silu_grad(f.y);
                }
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (nc + j < p.N) {
                const float x = __bfloat162float(ax[j]);
                v[j] *= (p.act == INCIN_ACT_DGELU) ? gelu_erf_grad(x) : silu_grad(x);
              }
            }
          }
        }
        if (p.residual && row_ok) {
          const __nv_bfloat16* rs = p.residual + cbase + nc;
          if (full && p.wide_io && aligned32(rs)) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint32_t bw[8];
              ld_global_b256(rs + q * 16, bw);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float2 f = unpack_bf16x2(bw[e]);
                v[q * 16 + e * 2] += f.x;
                v[q * 16 + e * 2 + 1] += f.y;
              }
            }
          } else if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 bb = *reinterpret_cast<const uint4*>(rs + q * 8);
              const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = unpack_bf16x2(bw[e]);
                v[q * 8 + e * 2] += f.x;
                v[q * 8 + e * 2 + 1] += f.y;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) v[j] += __bfloat162float(rs[j]);
          }
        }
}

// Epilogue of one accumulator chunk with per-thread global stores: the values above, then a bf16 or fp32 store
// (plain, or atomic for split-K and gradient accumulation).  The caller has checked that the row exists.
__device__ __forceinline__ void epilogue_chunk(const GemmKernelParams& p, const uint32_t (&r)[32], void* c_ptr,
                                               long long cbase, int nc, bool vec_ok, float alpha) {
        float v[32], pre_unused[32];
        epilogue_values<false>(p, r, cbase, nc, vec_ok, alpha, true, v, pre_unused);
        const bool full = (nc + 32 <= p.N) && vec_ok;
        if (p.out_fp32) {
          float* out = reinterpret_cast<float*>(c_ptr) + cbase + nc;
          if (p.accumulate) {
            if (full) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + q * 4), "f"(v[q * 4]),
                             "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                             : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) atomicAdd(out + j, v[j]);
            }
          } else {
            if (full && p.wide_io && aligned32(out)) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint32_t o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(v[q * 8 + e]);
                st_global_b256(out + q * 8, o);
              }
            } else if (full) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(out + q * 4) =
                    make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nc + j < p.N) out[j] = v[j];
            }
          }
        } else {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(c_ptr) + cbase + nc;
          if (full && p.wide_io && aligned32(out)) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              uint32_t o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = pack_bf16x2(v[q * 16 + e * 2], v[q * 16 + e * 2 + 1]);
              st_global_b256(out + q * 16, o);
            }
          } else if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(out + q * 8) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nc + j < p.N) out[j] = __float2bfloat16(v[j]);
          }
        }
}

// ---------------------------------------------------------------------------------------------------------------
// Staged epilogue of one warp for one output tile: its 32 rows x `ncols` columns starting at column n_first, read from
// tensor memory at taddr (lane quarter and accumulator offset included), written through this warp's 4 KB staging box.
// Per step the warp handles 128 bytes of every row (64 bf16 or 32 fp32 columns): values -> shared memory (row per lane,
// 16-byte units XOR-swizzled by the row, so the 32 lanes of a store hit 32 different bank groups) -> global memory.
// fp32 boxes leave through one bulk tensor store, or reduce-add for accumulating outputs, issued by lane 0 (the box is
// reused once that operation has read it; rows beyond M and columns beyond N are clipped by the tensor map).  bf16
// boxes are read back and stored row-wise (see write_rows).
// Why: with per-thread stores every store instruction touches 32 different rows (16 bytes each) and the epilogue of a
// 128 x 256 tile took about 6 us, as long as the main loop of a K = 768 product; staged, the memory system sees whole
// 128-byte rows.
__device__ __forceinline__ void epilogue_staged(const GemmKernelParams& p, const CUtensorMap* tmC, const CUtensorMap* tmAux,
                                                uint32_t taddr, uint8_t* stg, int row0, int n_first, int ncols, int b_lo,
                                                int b_hi, long long cbase, bool row_ok, float alpha, int lane) {
  const bool want_pre = p.aux && (p.act == INCIN_ACT_GELU || p.act == INCIN_ACT_SILU);
  uint8_t* my_row = stg + lane * 128;
  const int sw = lane & 7;
  auto box_free = [&]() {   // the previous bulk operation of this warp has read the box
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
  };
  auto send = [&](const CUtensorMap* tm, int n, bool reduce) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (reduce) tma_reduce_add_4d(tm, stg, n, row0, b_lo, b_hi);
      else tma_store_4d(tm, stg, n, row0, b_lo, b_hi);
      bulk_commit();
    }
  };
  auto pack32 = [](const float (&v)[32], uint32_t (&pk)[16]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
  };
  auto put_bf16 = [&](const uint32_t (&pk)[16], int half) {   // 32 columns = 16-byte units 4*half .. 4*half+3 of the row
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<uint4*>(my_row + (((half * 4 + q) ^ sw) << 4)) = make_uint4(pk[q * 4], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
  };
  // bf16 boxes leave with ordinary stores, read back so that one store instruction covers four whole 128-byte rows
  // (8 lanes x 16 bytes per row) instead of 16 bytes of 32 different rows.  (Bulk tensor stores of these 4 KB boxes
  // measured slower inside a training step: sixteen of them per tile share the SM's copy engine with the operand loads.)
  const long long tile_base = (long long)b_lo * p.c_stride_lo + (long long)b_hi * p.c_stride_hi + (long long)row0 * p.ldc;
  auto write_rows = [&](__nv_bfloat16* dst, int n, int valid_cols) {
    __syncwarp();
    const int u = lane & 7, col = n + u * 8;
    if (u * 8 < valid_cols && col < p.N) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = i * 4 + (lane >> 3);
        if (row0 + row < p.M) {
          const uint4 val = *reinterpret_cast<const uint4*>(stg + row * 128 + ((u ^ (row & 7)) << 4));
          __nv_bfloat16* o = dst + tile_base + (long long)row * p.ldc + col;
          if (col + 8 <= p.N) {
            *reinterpret_cast<uint4*>(o) = val;
          } else {
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&val);
            for (int j = 0; j < 8 && col + j < p.N; ++j) o[j] = e[j];
          }
        }
      }
    }
    __syncwarp();   // the box may be overwritten
  };
  if (p.out_fp32) {
    for (int c = 0; c < ncols; c += 32) {
      const int nc = n_first + c;
      if (nc >= p.N) break;
      uint32_t r[32];
      tmem_ld_32x32(taddr + c, r);
      tmem_ld_wait();
      float v[32], pre[32];
      epilogue_values<false>(p, r, cbase, nc, true, alpha, row_ok, v, pre);
      box_free();
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(my_row + ((q ^ sw) << 4)) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      send(tmC, nc, p.accumulate != 0);
    }
  } else {
    for (int c = 0; c < ncols; c += 64) {
      const int nc = n_first + c;
      if (nc >= p.N) break;
      const bool second = (c + 32 < ncols) && (nc + 32 < p.N);
      uint32_t out[2][16];   // the C values, packed, until the box is free for them
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !second) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c + h * 32, r);
        tmem_ld_wait();
        float v[32], pre[32];
        if (want_pre) {
          epilogue_values<true>(p, r, cbase, nc + h * 32, true, alpha, row_ok, v, pre);
          uint32_t pk[16];
          pack32(pre, pk);
          put_bf16(pk, h);
        } else {
          epilogue_values<false>(p, r, cbase, nc + h * 32, true, alpha, row_ok, v, pre);
        }
        pack32(v, out[h]);
      }
      const int valid_cols = second ? 64 : 32;
      if (want_pre) write_rows(p.aux, nc, valid_cols);
      put_bf16(out[0], 0);
      if (second) put_bf16(out[1], 1);
      write_rows(reinterpret_cast<__nv_bfloat16*>(p.C), nc, valid_cols);
    }
  }
}

}  // namespace incin
