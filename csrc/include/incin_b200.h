/* C ABI of the sm_100a kernel library (libincin_sm100.so).
 *
 * Every entry point takes raw device pointers plus the CUDA stream to launch on
 * (a cudaStream_t passed as void*), returns an incin_status code and never
 * synchronises the device.  Unless a function says otherwise it allocates
 * nothing: outputs and scratch buffers are owned by the caller (the Python
 * layer hands in torch-allocated storage), so every launch is capturable in a
 * CUDA graph and replays with no host work.
 *
 * bf16 tensors are `uint16_t`-sized elements in device memory; fp32 tensors are
 * `float`.  "rows" always means the flattened leading dimensions.
 */
#ifndef INCIN_B200_H
#define INCIN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum incin_status {
  INCIN_OK = 0,
  INCIN_ERR_ARGUMENT = 1,
  INCIN_ERR_ALIGNMENT = 2,
  INCIN_ERR_DRIVER = 3,
  INCIN_ERR_TENSOR_MAP = 4,
  INCIN_ERR_LAUNCH = 5,
  INCIN_ERR_UNSUPPORTED = 6,
  INCIN_ERR_TOO_LARGE = 7,
  INCIN_ERR_PEER = 8
} incin_status;

/* epilogue activations of incin_gemm_bf16 */
enum {
  INCIN_ACT_NONE = 0,
  INCIN_ACT_GELU = 1,  /* exact erf GELU; optional pre-activation copy to aux */
  INCIN_ACT_SILU = 2,
  INCIN_ACT_DGELU = 3, /* multiply by GELU'(aux): activation backward fused into a data-gradient GEMM */
  INCIN_ACT_DSILU = 4
};

/* C[b][m][n] = epi(alpha * sum_k A[b][m][k] * B[b][n][k]); all strides in elements.
 * a_mn_major = 0: A is stored [M][lda] (k contiguous);  1: stored [K][lda] (m contiguous).
 * b_mn_major = 0: B is stored [N][ldb] (k contiguous);  1: stored [K][ldb] (n contiguous).
 * batch index b in [0, batch_lo*batch_hi) splits into (b % batch_lo, b / batch_lo) with one
 * stride each, so heads inside a [B, T, 3, H, D] buffer are addressable without a copy. */
typedef struct incin_gemm_desc {
  const void* A;
  const void* B;
  void* C;
  int M, N, K;
  long long lda, ldb, ldc;
  int a_mn_major, b_mn_major;
  int batch_lo, batch_hi;
  long long a_stride_lo, a_stride_hi, b_stride_lo, b_stride_hi, c_stride_lo, c_stride_hi;
  int out_fp32;    /* C is float instead of bf16 */
  int accumulate;  /* fp32 only: C += result (atomic), needed for split-K */
  float alpha;
  const void* bias;     /* bf16 [N] or NULL */
  const void* residual; /* bf16, same layout as C, or NULL */
  int act;
  void* aux;     /* bf16, same layout as C: GELU/SILU pre-activation out, DGELU/DSILU pre-activation in */
  int splits;    /* split-K factor (>1 requires out_fp32 && accumulate) */
  int tile_n;    /* 0 = heuristic, else 64/128/192/256 */
  int max_ctas;  /* 0 = all SMs; smaller leaves SMs to a concurrent communication kernel */
  void* status;  /* optional int32 device word: receives a KernelStatus code if a wait timed out */
  /* --- fused all-gather -> GEMM (tensor-parallel column layer).  ag_world > 1 switches it on: A must then be
   * the LOCAL gathered buffer [ag_world * ag_rows_per_rank][lda] with lda == K, and ag_src[r] is rank r's
   * shard [ag_rows_per_rank][K] (a peer-mapped pointer for r != ag_rank).  ag_copy_ctas CTAs of the same launch
   * pull the shards into the gathered buffer with bulk copies (each remote byte crosses NVLink once) and
   * publish one flag per 128-row tile in ag_flags (uint32[tiles_m], zeroed by the caller before the launch);
   * the GEMM CTAs consume tiles in the order they arrive, own shard first.  ag_rows_per_rank % 128 == 0.
   * ag_src[ag_rank] == NULL: the caller has already written this rank's own rows into the gathered buffer; they are
   * neither copied nor waited for.
   * ag_copy_ctas = -n asks for copy warps instead: every compute CTA carries one more warp that moves its share of the
   * shards in 8 KB bulk copies (no SM is taken from the GEMM; n operand stages of shared memory become the copy ring,
   * at least three stay with the GEMM); ag_flags then count the completed chunks of a tile. */
  int ag_world, ag_rank, ag_rows_per_rank, ag_copy_ctas;
  const void* ag_src[8];
  void* ag_flags;
  /* --- fused GEMM -> reduce-scatter (row layer).  rs_world > 1: the epilogue stores each 128-row tile of the
   * partial product as bf16 into the slot of this rank inside the OWNER rank's slot buffer
   * rs_dst[owner] = [rs_world][rs_rows_per_rank][ldc] over peer stores; C is ignored.  The owner sums the
   * slots afterwards (incin_slot_reduce) once a peer barrier has passed.
   * With rs_copy_ctas > 0 and rs_ready != NULL the transfer is done by copy CTAs instead: the epilogue writes
   * tiles owned by other ranks into the local staging buffer C ([M][ldc], ldc == N), counts finished epilogue
   * warps per 128-row block in rs_ready (uint32[tiles_m], zeroed by the caller), and rs_copy_ctas CTAs of the
   * same launch push each completed block to its owner in 32 KB bulk copies while later blocks are computed.
   * rs_copy_ctas = -n: the blocks are pushed by one copy warp in every compute CTA instead (see ag_copy_ctas). */
  int rs_world, rs_rank, rs_rows_per_rank, rs_copy_ctas;
  void* rs_dst[8];
  long long rs_slot_stride;
  void* rs_ready;
  /* --- operand type: INCIN_GEMM_IN_BF16 (0), INCIN_GEMM_IN_FP16 or INCIN_GEMM_IN_TF32 (A and B are fp32, multiplied
   * as tf32; K-contiguous operands only, lda / ldb multiples of 4).  The last two require out_fp32 and take no fused
   * epilogue (bias, residual, activation), no CTA-pair tile and no fused collective. */
  int in_dtype;
  /* --- optional device scalar (fp32) multiplied into alpha when the epilogue runs: lets a gradient that only exists
   * on the GPU (the upstream gradient of a loss) scale a product without a launch of its own. */
  const void* alpha_ptr;
} incin_gemm_desc;

enum { INCIN_GEMM_IN_BF16 = 0, INCIN_GEMM_IN_FP16 = 1, INCIN_GEMM_IN_TF32 = 2 };

int incin_gemm_bf16(const incin_gemm_desc* desc, void* stream);

/* ---- normalisation ------------------------------------------------------------------------ */
/* y = (x - mean) * rstd * gamma + beta over the last dim C; bf16 io, fp32 statistics.
 * beta may be NULL.  mean/rstd are fp32 [rows] and are kept for the backward pass. */
int incin_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                        long long rows, int C, float eps, void* stream);
/* dx = LN'(dy) (+ dx_add when not NULL: the residual-stream gradient, fused);
 * dgamma/dbeta are fp32 and are ACCUMULATED into (they are slices of the flat gradient buffer).
 * scratch: fp32, at least incin_layernorm_bwd_scratch_floats(rows, C) elements. */
long long incin_layernorm_bwd_scratch_floats(long long rows, int C);
int incin_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                        const void* dx_add, void* dx, float* dgamma, float* dbeta, float* scratch, long long rows,
                        int C, void* stream);
/* RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gamma */
int incin_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, long long rows, int C, float eps,
                      void* stream);
/* LayerNorm backward that also adds the column sums of the dx it writes (dx_add included) into dxsum[C] (fp32): the
 * bias gradient of the linear layer whose output entered the residual stream in front of this norm.  One-pass kernel
 * only: C % 8 == 0 and C <= 1024, dgamma required; scratch of incin_layernorm_bwd_colsum_scratch_floats(rows, C) floats. */
long long incin_layernorm_bwd_colsum_scratch_floats(long long rows, int C);
int incin_layernorm_bwd_colsum(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                               const void* dx_add, void* dx, float* dgamma, float* dbeta, float* dxsum, float* scratch,
                               long long rows, int C, void* stream);
int incin_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, const void* dx_add,
                      void* dx, float* dgamma, float* scratch, long long rows, int C, void* stream);

/* ---- embedding ------------------------------------------------------------------------------ */
/* out[b,t,:] = wte[tok[b,t],:] + wpe[t,:] (wpe may be NULL); tokens are int64 */
int incin_embedding_fwd(const int64_t* tokens, const void* wte, const void* wpe, void* out, long long B, int T, int C,
                        void* stream);
/* dwte/dwpe are fp32 and accumulated into with atomics */
int incin_embedding_bwd(const void* dout, const int64_t* tokens, float* dwte, float* dwpe, long long B, int T, int C,
                        void* stream);

/* ---- softmax cross-entropy -------------------------------------------------------------------- */
/* logits: bf16 [rows][ld], only the first V columns are classes.  Writes per-row loss and log-sum-exp. */
int incin_xent_fwd(const void* logits, const int64_t* targets, float* loss, float* lse, long long rows, int V,
                   long long ld, void* stream);
/* dlogits = (softmax - onehot) * (*dloss) * scale, written in place over logits (columns >= V get 0) */
int incin_xent_bwd(void* logits, const int64_t* targets, const float* lse, const float* dloss, float scale,
                   long long rows, int V, long long ld, void* stream);
/* loss, log-sum-exp and gradient in one launch: logits are overwritten by (softmax - onehot) * scale (columns >= V get
 * 0, rows whose target is out of range get 0); the upstream gradient of the loss is left to the consumer
 * (incin_gemm_desc.alpha_ptr). */
int incin_xent_fused(void* logits, const int64_t* targets, float* loss, float* lse, float scale, long long rows, int V,
                     long long ld, void* stream);
/* out[0] = mean(x[0..n)) : deterministic single-block tree reduction */
int incin_mean_f32(const float* x, float* out, long long n, void* stream);

/* ---- causal softmax for the composed (materialised-scores) attention path ---------------------- */
/* in place over bf16 scores [batch][T][T]: p = softmax(scale * s + causal mask) */
int incin_causal_softmax_fwd(void* scores, long long batch, int T, float scale, void* stream);
/* in place over dP given P: dS = P * (dP - sum(dP * P)) * scale, zero above the diagonal */
int incin_causal_softmax_bwd(void* dp, const void* p, long long batch, int T, float scale, void* stream);

/* ---- reductions / misc ------------------------------------------------------------------------- */
/* dbias[n] += sum_m dy[m][n]  (fp32 accumulate into the flat gradient buffer) */
int incin_colsum_accum(const void* dy, float* dbias, long long rows, int N, long long ld, void* stream);
/* out[0] += sum(x^2); out[1] = 1.0 if any element is NaN/Inf (device-side gradient check, no D2H of tensors) */
int incin_sumsq_nonfinite_f32(const float* x, long long n, float* out, void* stream);
int incin_fill_f32(float* x, float value, long long n, void* stream);
int incin_cast_f32_to_bf16(const float* x, void* y, long long n, void* stream);
int incin_cast_bf16_to_f32(const void* x, float* y, long long n, void* stream);
/* y = act'(pre) * dy,  y = act(x) elementwise (bf16) for modules that do not fuse into a GEMM */
int incin_act_fwd(const void* x, void* y, long long n, int act, void* stream);
int incin_act_bwd(const void* dy, const void* pre, void* dx, long long n, int act, void* stream);
/* SwiGLU: y = silu(gate) * up, inputs are the two halves [rows][2F] -> [rows][F] */
int incin_swiglu_fwd(const void* gate_up, void* y, long long rows, int F, void* stream);
int incin_swiglu_bwd(const void* dy, const void* gate_up, void* dgate_up, long long rows, int F, void* stream);
/* rotary embedding in place on [B][T][H][D] slices with row stride `ld`; inverse=1 applies the transpose (backward) */
int incin_rope(void* x, long long B, int T, int H, int D, long long stride_b, long long stride_t, long long stride_h,
               float theta, int inverse, void* stream);

/* ---- optimiser --------------------------------------------------------------------------------- */
/* hyper (device, 8 floats): {lr, beta1, beta2, eps, weight_decay, step, grad_scale, unused}.
 * Bias-corrected, decoupled weight decay on the first n_decay elements only.
 * Updates fp32 master weights and moments and writes the bf16 shadow copy used by the forward pass. */
int incin_adamw_flat(float* master, float* m, float* v, const float* grad, void* shadow_bf16, long long n,
                     long long n_decay, const float* hyper, void* stream);
/* hyper: {lr, momentum, unused, unused, weight_decay, ...}; mom may be NULL */
int incin_sgd_flat(float* master, float* mom, const float* grad, void* shadow_bf16, long long n, long long n_decay,
                   const float* hyper, void* stream);

/* ---- device RNG (Philox4x32-10) ---------------------------------------------------------------- */
int incin_philox_uniform_f32(float* out, long long n, uint64_t seed, uint64_t offset, void* stream);
int incin_philox_normal_f32(float* out, long long n, uint64_t seed, uint64_t offset, float mean, float std,
                            void* stream);
int incin_philox_normal_bf16(void* out, long long n, uint64_t seed, uint64_t offset, float mean, float std,
                             void* stream);
/* y = x * mask / (1-p), mask regenerated from (seed, offset) in the backward pass, never stored */
int incin_dropout_bf16(const void* x, void* y, long long n, float p, uint64_t seed, uint64_t offset, void* stream);

/* ---- flash attention (causal, online softmax, GQA) ------------------------------------------------ */
/* q/o/do/dq: [B, T, Hq, D]; k/v/dk/dv: [B, T, Hkv, D]; every tensor has its own (b, t, h) strides in elements
 * so packed QKV buffers need no copies.  D is 64 or 128.  lse: fp32 [B, Hq, Tpad] in the log2 domain
 * (max*scale*log2e + log2(sum)) with Tpad = T rounded up to 128 (padding rows hold +inf).  The backward needs
 * delta (fp32 [B, Hq, Tpad]) and dq_accum (fp32 [B, T, Hq, D])
 * as caller-provided scratch; it zeroes dq_accum itself. */
typedef struct incin_attn_desc {
  const void *q, *k, *v;
  void* o;
  float* lse;
  int B, T, Hq, Hkv, D;
  float scale;
  long long q_stride_b, q_stride_t, q_stride_h;
  long long k_stride_b, k_stride_t, k_stride_h;
  long long v_stride_b, v_stride_t, v_stride_h;
  long long o_stride_b, o_stride_t, o_stride_h;
  /* backward only */
  const void* d_o;
  long long do_stride_b, do_stride_t, do_stride_h;
  void *dq, *dk, *dv;
  long long dq_stride_b, dq_stride_t, dq_stride_h;
  long long dk_stride_b, dk_stride_t, dk_stride_h;
  long long dv_stride_b, dv_stride_t, dv_stride_h;
  float* delta;
  float* dq_accum;
  void* status;
} incin_attn_desc;
int incin_flash_attn_fwd(const incin_attn_desc* desc, void* stream);
int incin_flash_attn_bwd(const incin_attn_desc* desc, void* stream);

/* ---- tensor-parallel helpers -------------------------------------------------------------------- */
/* out[r][n] = sum_s slots[s][r][n] (+ residual[r][n]) in fp32, written as bf16; slots: bf16 [world][rows][ld] */
int incin_slot_reduce(const void* slots, long long slot_stride, int world, const void* residual, void* out,
                      long long rows, int N, long long ld, void* stream);

/* ---- library info ------------------------------------------------------------------------------ */
const char* incin_sm100_version(void);
/* ---- reductions (reduce.cu) ------------------------------------------------------------------ */
/* op: 0 sum, 1 mean, 2 max, 3 min, 4 prod, 5 argmax, 6 argmin.  x is dense, viewed as [outer][reduce][inner];
 * values keep the input dtype (bf16 or fp32, fp32 accumulation), arg* write int64 indices into idx_out. */
int incin_reduce_axis(const void* x, void* out, long long* idx_out, long long outer, long long reduce, long long inner,
                      int op, int is_bf16, void* stream);
/* Whole-tensor reduction in ONE launch with a fixed combine order (bitwise reproducible); result is fp32 (or int64).
 * Uses one file-scope partial buffer per device: launches must be ordered on one stream. */
int incin_reduce_all(const void* x, float* out, long long* idx_out, long long n, int op, int is_bf16, void* stream);
int incin_cumsum(const void* x, void* out, long long outer, long long n, long long inner, int is_bf16, void* stream);

/* ---- data movement (shape.cu) ---------------------------------------------------------------- */
/* dst[sum i_d * dst_strides[d]] = src[sum i_d * src_strides[d]] over shape[0..rank), rank <= 6, strides in elements
 * (0 = broadcast): transpose, narrow, paste, broadcast, concat and pad are all this one copy. */
int incin_strided_copy(const void* src, void* dst, int rank, const long long* shape, const long long* src_strides,
                       const long long* dst_strides, int elem_bytes, void* stream);
/* Indexed ops check every index: an out-of-range one is skipped and *err_flag (device int, may be NULL) is set. */
int incin_gather_rows(const void* src, const long long* index, void* out, long long n_idx, long long row_elems,
                      long long src_rows, int elem_bytes, int* err_flag, void* stream);
int incin_scatter_add_rows(const void* src, const long long* index, float* dst, long long n_idx, long long row_elems,
                           long long dst_rows, int src_is_bf16, int* err_flag, void* stream);
int incin_gather_last(const void* src, const long long* index, void* out, long long rows, long long n_src, long long n_idx,
                      int elem_bytes, int* err_flag, void* stream);
int incin_scatter_last(const void* src, const long long* index, void* dst, long long rows, long long n_dst, long long n_idx,
                       int elem_bytes, int* err_flag, void* stream);
int incin_masked_fill(const void* x, const uint8_t* mask, void* out, float value, long long n, int is_bf16, void* stream);
int incin_where(const uint8_t* cond, const void* a, const void* b, void* out, long long n, int elem_bytes, void* stream);
int incin_tri(const void* x, void* out, long long batch, long long rows, long long cols, long long diagonal, int upper,
              int elem_bytes, void* stream);

/* ---- convolution helpers, pooling, batch norm (spatial.cu); NCHW ------------------------------ */
typedef struct incin_conv_geom {
  int N, C, H, W, KH, KW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
} incin_conv_geom;
int incin_conv_out_hw(const incin_conv_geom* g, int* oh, int* ow);
/* cols = [N*OH*OW][C*KH*KW]: the K-major A operand of the convolution GEMM */
int incin_im2col(const void* x, void* cols, const incin_conv_geom* g, int is_bf16, void* stream);
/* dx = fold(cols): a gather per input pixel (no atomics, deterministic) */
int incin_col2im(const void* cols, void* dx, const incin_conv_geom* g, int is_bf16, void* stream);
int incin_maxpool2d_fwd(const void* x, void* y, int* argmax, const incin_conv_geom* g, int is_bf16, void* stream);
int incin_maxpool2d_bwd(const void* dy, const int* argmax, void* dx, const incin_conv_geom* g, int is_bf16, void* stream);
int incin_avgpool2d(const void* in, void* out, const incin_conv_geom* g, int backward, int is_bf16, void* stream);
int incin_batchnorm_train_fwd(const void* x, const float* gamma, const float* beta, void* y, float* save_mean, float* save_rstd,
                              float* running_mean, float* running_var, int N, int C, long long HW, float eps, float momentum,
                              int is_bf16, void* stream);
int incin_batchnorm_eval(const void* x, const float* gamma, const float* beta, const float* mean, const float* var, void* y,
                         int N, int C, long long HW, float eps, int is_bf16, void* stream);
/* adaptive average pooling over `planes` = N*C planes of H x W -> OH x OW (backward: in = dy, out = dx; a gather) */
int incin_adaptive_avgpool2d(const void* in, void* out, long long planes, int H, int W, int OH, int OW, int backward,
                             int is_bf16, void* stream);
/* softmax over the last axis of [rows, C] (bf16 or fp32 io, fp32 arithmetic); backward: dx = y * (dy - sum(dy * y)) */
int incin_softmax_lastdim_fwd(const void* x, void* y, long long rows, int C, int is_bf16, void* stream);
int incin_softmax_lastdim_bwd(const void* dy, const void* y, void* dx, long long rows, int C, int is_bf16, void* stream);
/* dgamma / dbeta are ACCUMULATED into (fp32) */
int incin_batchnorm_bwd(const void* dy, const void* x, const float* gamma, const float* save_mean, const float* save_rstd,
                        void* dx, float* dgamma, float* dbeta, int N, int C, long long HW, int is_bf16, void* stream);

/* ---- Q8_0 and deterministic embedding backward (quant_embed.cu) ------------------------------- */
int incin_quantize_q8_0(const void* x, void* packed, long long n, int is_bf16, void* stream);
int incin_dequantize_q8_0(const void* packed, void* out, long long n, int out_bf16, void* stream);
/* order: positions sorted by token id; segment s = sorted positions [seg_start[s], seg_start[s+1]) of token
 * seg_token[s] (seg_start has n_segments + 1 entries).  dwte / dwpe (may be NULL) are accumulated into. */
int incin_embedding_bwd_sorted(const void* dout, const long long* order, const long long* seg_start, const long long* seg_token,
                               long long n_segments, float* dwte, float* dwpe, long long B, int T, int C, long long vocab,
                               void* stream);

int incin_sm100_num_sms(void);

#ifdef __cplusplus
}
#endif
#endif /* INCIN_B200_H */
