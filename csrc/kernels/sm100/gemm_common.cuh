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

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int ACC_STRIDE = (BN <= 64) ? 64 : (BN <= 128 ? 128 : 256);
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
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

// Epilogue of one accumulator chunk: thread = one output row, r = its 32 consecutive fp32 accumulator columns
// starting at column nc.  alpha, bias, GELU / SiLU (+ pre-activation side output), activation-gradient masks,
// residual, then a bf16 or fp32 store (plain, read-modify-write, or atomic for split-K).
__device__ __forceinline__ void epilogue_chunk(const GemmKernelParams& p, const uint32_t (&r)[32], void* c_ptr,
                                               long long cbase, int nc, bool vec_ok, float alpha) {
        float v[32];
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
          if (p.aux) {  // keep the pre-activation for the backward pass
            __nv_bfloat16* ax = p.aux + cbase + nc;
            if (full) {
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
        } else if (p.act == INCIN_ACT_DGELU || p.act == INCIN_ACT_DSILU) {
          // multiply by act'(pre-activation): fuses the activation backward into the data-gradient GEMM
          const __nv_bfloat16* ax = p.aux + cbase + nc;
          if (full) {
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
        if (p.residual) {
          const __nv_bfloat16* rs = p.residual + cbase + nc;
          if (full) {
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
            if (full) {
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
          if (full) {
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

}  // namespace incin
