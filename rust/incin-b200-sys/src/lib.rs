// Generated from csrc/include/*.h by `python -m incin_b200 ffi`; do not edit by hand.
#![allow(non_camel_case_types, non_snake_case)]

use core::ffi::{c_char, c_int, c_longlong, c_uint, c_void};

pub const INCIN_OK: c_int = 0;
pub const INCIN_ERR_ARGUMENT: c_int = 1;
pub const INCIN_ERR_ALIGNMENT: c_int = 2;
pub const INCIN_ERR_DRIVER: c_int = 3;
pub const INCIN_ERR_TENSOR_MAP: c_int = 4;
pub const INCIN_ERR_LAUNCH: c_int = 5;
pub const INCIN_ERR_UNSUPPORTED: c_int = 6;
pub const INCIN_ERR_TOO_LARGE: c_int = 7;
pub const INCIN_ERR_PEER: c_int = 8;
pub const INCIN_ACT_NONE: c_int = 0;
pub const INCIN_ACT_GELU: c_int = 1;
pub const INCIN_ACT_SILU: c_int = 2;
pub const INCIN_ACT_DGELU: c_int = 3;
pub const INCIN_ACT_DSILU: c_int = 4;
pub const INCIN_GEMM_IN_BF16: c_int = 0;
pub const INCIN_GEMM_IN_FP16: c_int = 1;
pub const INCIN_GEMM_IN_TF32: c_int = 2;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct incin_gemm_desc {
    pub A: *const c_void,
    pub B: *const c_void,
    pub C: *mut c_void,
    pub M: c_int,
    pub N: c_int,
    pub K: c_int,
    pub lda: c_longlong,
    pub ldb: c_longlong,
    pub ldc: c_longlong,
    pub a_mn_major: c_int,
    pub b_mn_major: c_int,
    pub batch_lo: c_int,
    pub batch_hi: c_int,
    pub a_stride_lo: c_longlong,
    pub a_stride_hi: c_longlong,
    pub b_stride_lo: c_longlong,
    pub b_stride_hi: c_longlong,
    pub c_stride_lo: c_longlong,
    pub c_stride_hi: c_longlong,
    pub out_fp32: c_int,
    pub accumulate: c_int,
    pub alpha: f32,
    pub bias: *const c_void,
    pub residual: *const c_void,
    pub act: c_int,
    pub aux: *mut c_void,
    pub splits: c_int,
    pub tile_n: c_int,
    pub max_ctas: c_int,
    pub status: *mut c_void,
    pub ag_world: c_int,
    pub ag_rank: c_int,
    pub ag_rows_per_rank: c_int,
    pub ag_copy_ctas: c_int,
    pub ag_src: [*const c_void; 8],
    pub ag_flags: *mut c_void,
    pub rs_world: c_int,
    pub rs_rank: c_int,
    pub rs_rows_per_rank: c_int,
    pub rs_copy_ctas: c_int,
    pub rs_dst: [*mut c_void; 8],
    pub rs_slot_stride: c_longlong,
    pub rs_ready: *mut c_void,
    pub in_dtype: c_int,
    pub alpha_ptr: *const c_void,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct incin_attn_desc {
    pub q: *const c_void,
    pub k: *const c_void,
    pub v: *const c_void,
    pub o: *mut c_void,
    pub lse: *mut f32,
    pub B: c_int,
    pub T: c_int,
    pub Hq: c_int,
    pub Hkv: c_int,
    pub D: c_int,
    pub scale: f32,
    pub q_stride_b: c_longlong,
    pub q_stride_t: c_longlong,
    pub q_stride_h: c_longlong,
    pub k_stride_b: c_longlong,
    pub k_stride_t: c_longlong,
    pub k_stride_h: c_longlong,
    pub v_stride_b: c_longlong,
    pub v_stride_t: c_longlong,
    pub v_stride_h: c_longlong,
    pub o_stride_b: c_longlong,
    pub o_stride_t: c_longlong,
    pub o_stride_h: c_longlong,
    pub d_o: *const c_void,
    pub do_stride_b: c_longlong,
    pub do_stride_t: c_longlong,
    pub do_stride_h: c_longlong,
    pub dq: *mut c_void,
    pub dk: *mut c_void,
    pub dv: *mut c_void,
    pub dq_stride_b: c_longlong,
    pub dq_stride_t: c_longlong,
    pub dq_stride_h: c_longlong,
    pub dk_stride_b: c_longlong,
    pub dk_stride_t: c_longlong,
    pub dk_stride_h: c_longlong,
    pub dv_stride_b: c_longlong,
    pub dv_stride_t: c_longlong,
    pub dv_stride_h: c_longlong,
    pub delta: *mut f32,
    pub dq_accum: *mut f32,
    pub status: *mut c_void,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct incin_conv_geom {
    pub N: c_int,
    pub C: c_int,
    pub H: c_int,
    pub W: c_int,
    pub KH: c_int,
    pub KW: c_int,
    pub stride_h: c_int,
    pub stride_w: c_int,
    pub pad_h: c_int,
    pub pad_w: c_int,
    pub dil_h: c_int,
    pub dil_w: c_int,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct incin_dp_desc {
    pub grads: [*mut c_void; 64],
    pub shadows: [*mut c_void; 64],
    pub pads: [*mut c_void; 64],
    pub master: *mut c_void,
    pub m: *mut c_void,
    pub v: *mut c_void,
    pub hyper: *const c_void,
    pub lo: c_longlong,
    pub hi: c_longlong,
    pub n_decay: c_longlong,
    pub world: c_int,
    pub rank: c_int,
    pub slot: c_int,
    pub ctas: c_int,
    pub status: *mut c_void,
}

extern "C" {
    pub fn incin_act_bwd(dy: *const c_void, pre: *const c_void, dx: *mut c_void, n: c_longlong, act: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_act_fwd(x: *const c_void, y: *mut c_void, n: c_longlong, act: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_adamw_flat(master: *mut f32, m: *mut f32, v: *mut f32, grad: *const f32, shadow_bf16: *mut c_void, n: c_longlong, n_decay: c_longlong, hyper: *const f32, stream: *mut c_void) -> c_int;
    pub fn incin_adaptive_avgpool2d(r#in: *const c_void, out: *mut c_void, planes: c_longlong, H: c_int, W: c_int, OH: c_int, OW: c_int, backward: c_int, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_avgpool2d(r#in: *const c_void, out: *mut c_void, g: *const incin_conv_geom, backward: c_int, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_barrier_pad_bytes() -> c_int;
    pub fn incin_batchnorm_bwd(dy: *const c_void, x: *const c_void, gamma: *const f32, save_mean: *const f32, save_rstd: *const f32, dx: *mut c_void, dgamma: *mut f32, dbeta: *mut f32, N: c_int, C: c_int, HW: c_longlong, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_batchnorm_eval(x: *const c_void, gamma: *const f32, beta: *const f32, mean: *const f32, var: *const f32, y: *mut c_void, N: c_int, C: c_int, HW: c_longlong, eps: f32, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_batchnorm_train_fwd(x: *const c_void, gamma: *const f32, beta: *const f32, y: *mut c_void, save_mean: *mut f32, save_rstd: *mut f32, running_mean: *mut f32, running_var: *mut f32, N: c_int, C: c_int, HW: c_longlong, eps: f32, momentum: f32, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_can_access_peer(dev: c_int, peer: c_int) -> c_int;
    pub fn incin_cast_bf16_to_f32(x: *const c_void, y: *mut f32, n: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_cast_f32_to_bf16(x: *const f32, y: *mut c_void, n: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_causal_softmax_bwd(dp: *mut c_void, p: *const c_void, batch: c_longlong, T: c_int, scale: f32, stream: *mut c_void) -> c_int;
    pub fn incin_causal_softmax_fwd(scores: *mut c_void, batch: c_longlong, T: c_int, scale: f32, stream: *mut c_void) -> c_int;
    pub fn incin_col2im(cols: *const c_void, dx: *mut c_void, g: *const incin_conv_geom, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_coll_all_gather(bufs: *const *mut c_void, world: c_int, rank: c_int, offset_bytes: c_longlong, bytes: c_longlong, out: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn incin_coll_all_to_all(bufs: *const *mut c_void, world: c_int, rank: c_int, offset_bytes: c_longlong, chunk_bytes: c_longlong, out: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn incin_coll_reduce(bufs: *const *mut c_void, world: c_int, offset_bytes: c_longlong, first_elem: c_longlong, n: c_longlong, op: c_int, is_bf16: c_int, out: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn incin_colsum_accum(dy: *const c_void, dbias: *mut f32, rows: c_longlong, N: c_int, ld: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_conv_out_hw(g: *const incin_conv_geom, oh: *mut c_int, ow: *mut c_int) -> c_int;
    pub fn incin_cpu_adamw_f32(w: *mut f32, m: *mut f32, v: *mut f32, g: *const f32, n: i64, lr: f32, b1: f32, b2: f32, eps: f32, wd: f32, step: c_int);
    pub fn incin_cpu_attention_f32(q: *const f32, k: *const f32, v: *const f32, o: *mut f32, heads: i64, T: i64, D: i64, scale: f32, causal: c_int);
    pub fn incin_cpu_cross_entropy_f32(logits: *const f32, targets: *const i64, dlogits: *mut f32, rows: i64, V: i64) -> f32;
    pub fn incin_cpu_dequantize_q8_0(r#in: *const u8, y: *mut f32, n: i64);
    pub fn incin_cpu_gemm_f32(A: *const f32, B: *const f32, C: *mut f32, batch: i64, M: i64, N: i64, K: i64, a_bs: i64, a_rs: i64, a_cs: i64, b_bs: i64, b_rs: i64, b_cs: i64, c_bs: i64, c_rs: i64, alpha: f32, beta: f32);
    pub fn incin_cpu_layernorm_f32(x: *const f32, g: *const f32, b: *const f32, y: *mut f32, rows: i64, C: i64, eps: f32, rms: c_int);
    pub fn incin_cpu_mlp_train(steps: c_int, batch: c_int, n_in: c_int, n_hidden: c_int, n_out: c_int, lr: f32, seed: u64, losses_out: *mut f32, final_params_out: *mut f32) -> c_int;
    pub fn incin_cpu_philox_normal_f32(out: *mut f32, n: i64, seed: u64, offset: u64, mean: f32, std_: f32);
    pub fn incin_cpu_philox_uniform_f32(out: *mut f32, n: i64, seed: u64, offset: u64);
    pub fn incin_cpu_q8_0_bytes(n: i64) -> i64;
    pub fn incin_cpu_quantize_q8_0(x: *const f32, out: *mut u8, n: i64);
    pub fn incin_cpu_sgd_f32(w: *mut f32, g: *const f32, n: i64, lr: f32);
    pub fn incin_cpu_softmax_f32(x: *const f32, y: *mut f32, rows: i64, C: i64, log_softmax: c_int);
    pub fn incin_cpu_unary_f32(x: *const f32, y: *mut f32, n: i64, op: c_int);
    pub fn incin_cumsum(x: *const c_void, out: *mut c_void, outer: c_longlong, n: c_longlong, inner: c_longlong, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_dequantize_q8_0(packed: *const c_void, out: *mut c_void, n: c_longlong, out_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_digest_bytes(state: u64, data: *const c_void, n: i64) -> u64;
    pub fn incin_digest_field(state: u64, data: *const c_void, n: i64) -> u64;
    pub fn incin_digest_init() -> u64;
    pub fn incin_digest_number(state: u64, v: u64) -> u64;
    pub fn incin_dp_pad_bytes() -> c_int;
    pub fn incin_dp_reduce_adamw(desc: *const incin_dp_desc, stream: *mut c_void) -> c_int;
    pub fn incin_dp_reduce_adamw_mc(desc: *const incin_dp_desc, mc_grads: *mut c_void, mc_shadows: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn incin_dropout_bf16(x: *const c_void, y: *mut c_void, n: c_longlong, p: f32, seed: u64, offset: u64, stream: *mut c_void) -> c_int;
    pub fn incin_embedding_bwd(dout: *const c_void, tokens: *const i64, dwte: *mut f32, dwpe: *mut f32, B: c_longlong, T: c_int, C: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_embedding_bwd_sorted(dout: *const c_void, order: *const c_longlong, seg_start: *const c_longlong, seg_token: *const c_longlong, n_segments: c_longlong, dwte: *mut f32, dwpe: *mut f32, B: c_longlong, T: c_int, C: c_int, vocab: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_embedding_fwd(tokens: *const i64, wte: *const c_void, wpe: *const c_void, out: *mut c_void, B: c_longlong, T: c_int, C: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_file_read_ranges(path: *const c_char, n: i64, offsets: *const i64, sizes: *const i64, dst: *const *mut c_void, threads: c_int) -> c_int;
    pub fn incin_fill_f32(x: *mut f32, value: f32, n: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_flash_attn_bwd(desc: *const incin_attn_desc, stream: *mut c_void) -> c_int;
    pub fn incin_flash_attn_fwd(desc: *const incin_attn_desc, stream: *mut c_void) -> c_int;
    pub fn incin_fnv1a64(data: *const c_void, n: i64) -> u64;
    pub fn incin_gather_last(src: *const c_void, index: *const c_longlong, out: *mut c_void, rows: c_longlong, n_src: c_longlong, n_idx: c_longlong, elem_bytes: c_int, err_flag: *mut c_int, stream: *mut c_void) -> c_int;
    pub fn incin_gather_rows(src: *const c_void, index: *const c_longlong, out: *mut c_void, n_idx: c_longlong, row_elems: c_longlong, src_rows: c_longlong, elem_bytes: c_int, err_flag: *mut c_int, stream: *mut c_void) -> c_int;
    pub fn incin_gemm_bf16(desc: *const incin_gemm_desc, stream: *mut c_void) -> c_int;
    pub fn incin_im2col(x: *const c_void, cols: *mut c_void, g: *const incin_conv_geom, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_layernorm_bwd(dy: *const c_void, x: *const c_void, gamma: *const c_void, mean: *const f32, rstd: *const f32, dx_add: *const c_void, dx: *mut c_void, dgamma: *mut f32, dbeta: *mut f32, scratch: *mut f32, rows: c_longlong, C: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_layernorm_bwd_colsum(dy: *const c_void, x: *const c_void, gamma: *const c_void, mean: *const f32, rstd: *const f32, dx_add: *const c_void, dx: *mut c_void, dgamma: *mut f32, dbeta: *mut f32, dxsum: *mut f32, scratch: *mut f32, rows: c_longlong, C: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_layernorm_bwd_colsum_scratch_floats(rows: c_longlong, C: c_int) -> c_longlong;
    pub fn incin_layernorm_bwd_noalloc(dy: *const c_void, x: *const c_void, gamma: *const c_void, mean: *const f32, rstd: *const f32, dx_add: *const c_void, dx: *mut c_void, dgamma: *mut f32, dbeta: *mut f32, rows: c_longlong, C: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_layernorm_bwd_scratch_floats(rows: c_longlong, C: c_int) -> c_longlong;
    pub fn incin_layernorm_fwd(x: *const c_void, gamma: *const c_void, beta: *const c_void, y: *mut c_void, mean: *mut f32, rstd: *mut f32, rows: c_longlong, C: c_int, eps: f32, stream: *mut c_void) -> c_int;
    pub fn incin_loader_create(a: *const c_void, row_bytes_a: i64, b: *const c_void, row_bytes_b: i64, n_rows: i64, batch: i64, shuffle: c_int, drop_last: c_int, seed: u64, workers: c_int, depth: c_int) -> i64;
    pub fn incin_loader_destroy(h: i64);
    pub fn incin_loader_next(h: i64, out_a: *mut c_void, out_b: *mut c_void, rows_out: *mut i64) -> c_int;
    pub fn incin_loader_order(h: i64, out: *mut i64) -> c_int;
    pub fn incin_loader_start(h: i64, epoch: u64) -> i64;
    pub fn incin_masked_fill(x: *const c_void, mask: *const u8, out: *mut c_void, value: f32, n: c_longlong, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_maxpool2d_bwd(dy: *const c_void, argmax: *const c_int, dx: *mut c_void, g: *const incin_conv_geom, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_maxpool2d_fwd(x: *const c_void, y: *mut c_void, argmax: *mut c_int, g: *const incin_conv_geom, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_mean_f32(x: *const f32, out: *mut f32, n: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_memplan_first_fit(n: i64, sizes: *const i64, first: *const i64, last: *const i64, skip: *const u8, offsets_out: *mut i64) -> i64;
    pub fn incin_p2p_send(peer_dst: *mut c_void, src: *const c_void, bytes: c_longlong, peer_flag: *mut c_void, seq: c_uint, stream: *mut c_void) -> c_int;
    pub fn incin_p2p_wait(local_flag: *const c_void, seq: c_uint, status: *mut c_void, timeout_ms: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_peer_barrier(pads: *const *mut c_void, world: c_int, rank: c_int, slot: c_int, status: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn incin_peer_sum_ranges(bases: *const *mut c_void, world: c_int, ranges: *const c_void, n_ranges: c_int, scratch: *mut c_void, stage: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_philox_normal_bf16(out: *mut c_void, n: c_longlong, seed: u64, offset: u64, mean: f32, std: f32, stream: *mut c_void) -> c_int;
    pub fn incin_philox_normal_f32(out: *mut f32, n: c_longlong, seed: u64, offset: u64, mean: f32, std: f32, stream: *mut c_void) -> c_int;
    pub fn incin_philox_uniform_f32(out: *mut f32, n: c_longlong, seed: u64, offset: u64, stream: *mut c_void) -> c_int;
    pub fn incin_quantize_q8_0(x: *const c_void, packed: *mut c_void, n: c_longlong, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_rdv_abort(h: i64, code: c_int, timeout_ms: c_int) -> c_int;
    pub fn incin_rdv_allgather(h: i64, mine: *const c_void, bytes: c_int, all: *mut c_void, timeout_ms: c_int) -> c_int;
    pub fn incin_rdv_connect(rank: c_int, world: c_int, addr: *const c_char, run_id: *const c_char, local_device: i64, timeout_ms: c_int, handle_out: *mut i64) -> c_int;
    pub fn incin_rdv_destroy(h: i64);
    pub fn incin_rdv_ensure_active(h: i64) -> c_int;
    pub fn incin_rdv_failure_code(h: i64) -> c_int;
    pub fn incin_rdv_invalidate(h: i64, code: c_int);
    pub fn incin_rdv_peer_device(h: i64, rank: c_int) -> i64;
    pub fn incin_rdv_shutdown(h: i64, timeout_ms: c_int) -> c_int;
    pub fn incin_rdv_state(h: i64) -> c_int;
    pub fn incin_rdv_wait_for_peer(h: i64, timeout_ms: c_int, kind: *mut c_int, code: *mut c_int, from: *mut c_int) -> c_int;
    pub fn incin_reduce_all(x: *const c_void, out: *mut f32, idx_out: *mut c_longlong, n: c_longlong, op: c_int, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_reduce_axis(x: *const c_void, out: *mut c_void, idx_out: *mut c_longlong, outer: c_longlong, reduce: c_longlong, inner: c_longlong, op: c_int, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_ref_all_gather(r#in: *const *const c_void, out: *const *mut c_void, world: c_int, n: i64, dtype: c_int) -> c_int;
    pub fn incin_ref_all_reduce(r#in: *const *const c_void, out: *const *mut c_void, world: c_int, n: i64, dtype: c_int, op: c_int) -> c_int;
    pub fn incin_ref_all_to_all(r#in: *const *const c_void, out: *const *mut c_void, world: c_int, n: i64, dtype: c_int) -> c_int;
    pub fn incin_ref_reduce_scatter(r#in: *const *const c_void, out: *const *mut c_void, world: c_int, n: i64, dtype: c_int, op: c_int) -> c_int;
    pub fn incin_ref_send_recv(r#in: *const *const c_void, out: *const *mut c_void, world: c_int, n: i64, dtype: c_int, src: c_int, dst: c_int) -> c_int;
    pub fn incin_rmsnorm_bwd(dy: *const c_void, x: *const c_void, gamma: *const c_void, rstd: *const f32, dx_add: *const c_void, dx: *mut c_void, dgamma: *mut f32, scratch: *mut f32, rows: c_longlong, C: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_rmsnorm_fwd(x: *const c_void, gamma: *const c_void, y: *mut c_void, rstd: *mut f32, rows: c_longlong, C: c_int, eps: f32, stream: *mut c_void) -> c_int;
    pub fn incin_rope(x: *mut c_void, B: c_longlong, T: c_int, H: c_int, D: c_int, stride_b: c_longlong, stride_t: c_longlong, stride_h: c_longlong, theta: f32, inverse: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_scatter_add_rows(src: *const c_void, index: *const c_longlong, dst: *mut f32, n_idx: c_longlong, row_elems: c_longlong, dst_rows: c_longlong, src_is_bf16: c_int, err_flag: *mut c_int, stream: *mut c_void) -> c_int;
    pub fn incin_scatter_last(src: *const c_void, index: *const c_longlong, dst: *mut c_void, rows: c_longlong, n_dst: c_longlong, n_idx: c_longlong, elem_bytes: c_int, err_flag: *mut c_int, stream: *mut c_void) -> c_int;
    pub fn incin_sgd_flat(master: *mut f32, mom: *mut f32, grad: *const f32, shadow_bf16: *mut c_void, n: c_longlong, n_decay: c_longlong, hyper: *const f32, stream: *mut c_void) -> c_int;
    pub fn incin_slot_reduce(slots: *const c_void, slot_stride: c_longlong, world: c_int, residual: *const c_void, out: *mut c_void, rows: c_longlong, N: c_int, ld: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_sm100_num_sms() -> c_int;
    pub fn incin_sm100_version() -> *const c_char;
    pub fn incin_softmax_lastdim_bwd(dy: *const c_void, y: *const c_void, dx: *mut c_void, rows: c_longlong, C: c_int, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_softmax_lastdim_fwd(x: *const c_void, y: *mut c_void, rows: c_longlong, C: c_int, is_bf16: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_strided_copy(src: *const c_void, dst: *mut c_void, rank: c_int, shape: *const c_longlong, src_strides: *const c_longlong, dst_strides: *const c_longlong, elem_bytes: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_sumsq_nonfinite_f32(x: *const f32, n: c_longlong, out: *mut f32, stream: *mut c_void) -> c_int;
    pub fn incin_swiglu_bwd(dy: *const c_void, gate_up: *const c_void, dgate_up: *mut c_void, rows: c_longlong, F: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_swiglu_fwd(gate_up: *const c_void, y: *mut c_void, rows: c_longlong, F: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_symm_alloc(bytes: c_longlong, ptr_out: *mut *mut c_void, handle_out: *mut u8) -> c_int;
    pub fn incin_symm_close(peer_ptr: *mut c_void) -> c_int;
    pub fn incin_symm_free(ptr: *mut c_void) -> c_int;
    pub fn incin_symm_open(handle: *const u8, ptr_out: *mut *mut c_void) -> c_int;
    pub fn incin_tape_backward(root: i64) -> c_int;
    pub fn incin_tape_cross_entropy(logits: i64, targets: *const i64) -> i64;
    pub fn incin_tape_depth() -> i64;
    pub fn incin_tape_grad(h: i64, out: *mut f32) -> c_int;
    pub fn incin_tape_linear(x: i64, w: i64, b: i64) -> i64;
    pub fn incin_tape_read(h: i64, out: *mut f32) -> c_int;
    pub fn incin_tape_relu(x: i64) -> i64;
    pub fn incin_tape_reset();
    pub fn incin_tape_set_grad_mode(on: c_int);
    pub fn incin_tape_set_nan_policy(p: c_int);
    pub fn incin_tape_tensor(data: *const f32, rows: i64, cols: i64, requires_grad: c_int) -> i64;
    pub fn incin_tape_tensor_id(h: i64) -> u64;
    pub fn incin_telemetry_close(h: i64) -> i64;
    pub fn incin_telemetry_flush(h: i64) -> i64;
    pub fn incin_telemetry_memory(h: i64, device: c_int, allocated: i64, reserved: i64, step: i64) -> c_int;
    pub fn incin_telemetry_open(path: *const c_char, capacity: i64) -> i64;
    pub fn incin_telemetry_raw(h: i64, json_line: *const c_char) -> c_int;
    pub fn incin_telemetry_scalar(h: i64, name: *const c_char, value: f64, step: i64) -> c_int;
    pub fn incin_tri(x: *const c_void, out: *mut c_void, batch: c_longlong, rows: c_longlong, cols: c_longlong, diagonal: c_longlong, upper: c_int, elem_bytes: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_where(cond: *const u8, a: *const c_void, b: *const c_void, out: *mut c_void, n: c_longlong, elem_bytes: c_int, stream: *mut c_void) -> c_int;
    pub fn incin_xent_bwd(logits: *mut c_void, targets: *const i64, lse: *const f32, dloss: *const f32, scale: f32, rows: c_longlong, V: c_int, ld: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_xent_fused(logits: *mut c_void, targets: *const i64, loss: *mut f32, lse: *mut f32, scale: f32, rows: c_longlong, V: c_int, ld: c_longlong, stream: *mut c_void) -> c_int;
    pub fn incin_xent_fwd(logits: *const c_void, targets: *const i64, loss: *mut f32, lse: *mut f32, rows: c_longlong, V: c_int, ld: c_longlong, stream: *mut c_void) -> c_int;
}
