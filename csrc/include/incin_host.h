/* C ABI of libincin_host.so: CPU oracle kernels, tape autograd, N-rank TCP rendezvous, the reference
 * (in-process, host-memory) collective transport and the host runtime (digest, batch loader, telemetry sink).
 * Every function is plain C, thread-compatible, and allocates only what its result needs. */
#ifndef INCIN_HOST_H
#define INCIN_HOST_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif


/* ---- CPU oracle (fp32 reference of every op; Philox identical to the device generator) ---- */
void incin_cpu_gemm_f32(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t a_bs, int64_t a_rs, int64_t a_cs, int64_t b_bs, int64_t b_rs, int64_t b_cs, int64_t c_bs, int64_t c_rs, float alpha, float beta);
void incin_cpu_unary_f32(const float* x, float* y, int64_t n, int op);
void incin_cpu_softmax_f32(const float* x, float* y, int64_t rows, int64_t C, int log_softmax);
void incin_cpu_layernorm_f32(const float* x, const float* g, const float* b, float* y, int64_t rows, int64_t C, float eps, int rms);
float incin_cpu_cross_entropy_f32(const float* logits, const int64_t* targets, float* dlogits, int64_t rows, int64_t V);
void incin_cpu_sgd_f32(float* w, const float* g, int64_t n, float lr);
void incin_cpu_adamw_f32(float* w, float* m, float* v, const float* g, int64_t n, float lr, float b1, float b2, float eps, float wd, int step);
void incin_cpu_attention_f32(const float* q, const float* k, const float* v, float* o, int64_t heads, int64_t T, int64_t D, float scale, int causal);
int64_t incin_cpu_q8_0_bytes(int64_t n);
void incin_cpu_quantize_q8_0(const float* x, uint8_t* out, int64_t n);
void incin_cpu_dequantize_q8_0(const uint8_t* in, float* y, int64_t n);
void incin_cpu_philox_uniform_f32(float* out, int64_t n, uint64_t seed, uint64_t offset);
void incin_cpu_philox_normal_f32(float* out, int64_t n, uint64_t seed, uint64_t offset, float mean, float std_);

/* ---- tape autograd and the native MLP training loop ---- */
int64_t incin_tape_tensor(const float* data, int64_t rows, int64_t cols, int requires_grad);
int64_t incin_tape_linear(int64_t x, int64_t w, int64_t b);
int64_t incin_tape_relu(int64_t x);
int64_t incin_tape_cross_entropy(int64_t logits, const int64_t* targets);
int incin_tape_backward(int64_t root);
int incin_tape_read(int64_t h, float* out);
int incin_tape_grad(int64_t h, float* out);
int64_t incin_tape_depth(void);
void incin_tape_set_grad_mode(int on);
void incin_tape_set_nan_policy(int p);
void incin_tape_reset(void);
uint64_t incin_tape_tensor_id(int64_t h);
int incin_cpu_mlp_train(int steps, int batch, int n_in, int n_hidden, int n_out, float lr, uint64_t seed, float* losses_out, float* final_params_out);

/* ---- rendezvous (TCP, 160-byte frames, plan-hash preflight) ---- */
int incin_rdv_connect(int rank, int world, const char* addr, const char* run_id, int64_t local_device, int timeout_ms, int64_t* handle_out);
int incin_rdv_state(int64_t h);
int incin_rdv_failure_code(int64_t h);
void incin_rdv_invalidate(int64_t h, int code);
int incin_rdv_ensure_active(int64_t h);
int incin_rdv_abort(int64_t h, int code, int timeout_ms);
int incin_rdv_wait_for_peer(int64_t h, int timeout_ms, int* kind, int* code, int* from);
int incin_rdv_shutdown(int64_t h, int timeout_ms);
int incin_rdv_allgather(int64_t h, const void* mine, int bytes, void* all, int timeout_ms);
int64_t incin_rdv_peer_device(int64_t h, int rank);
void incin_rdv_destroy(int64_t h);

/* ---- reference transport (collective semantics on host memory) ---- */
int incin_ref_all_reduce(const void* const* in, void* const* out, int world, int64_t n, int dtype, int op);
int incin_ref_all_gather(const void* const* in, void* const* out, int world, int64_t n, int dtype);
int incin_ref_reduce_scatter(const void* const* in, void* const* out, int world, int64_t n, int dtype, int op);
int incin_ref_all_to_all(const void* const* in, void* const* out, int world, int64_t n, int dtype);
int incin_ref_send_recv(const void* const* in, void* const* out, int world, int64_t n, int dtype, int src, int dst);

/* ---- runtime: digest (FNV-1a 64: plan hashes, mesh ids, autotune identities) ---- */
uint64_t incin_digest_init(void);
uint64_t incin_digest_bytes(uint64_t state, const void* data, int64_t n);
uint64_t incin_digest_number(uint64_t state, uint64_t v);
uint64_t incin_digest_field(uint64_t state, const void* data, int64_t n);
uint64_t incin_fnv1a64(const void* data, int64_t n);

/* ---- runtime: batch loader (worker threads, ordered delivery, bounded prefetch ring) ---- */
int64_t incin_loader_create(const void* a, int64_t row_bytes_a, const void* b, int64_t row_bytes_b, int64_t n_rows, int64_t batch, int shuffle, int drop_last, uint64_t seed, int workers, int depth);
int64_t incin_loader_start(int64_t h, uint64_t epoch);
int incin_loader_next(int64_t h, void* out_a, void* out_b, int64_t* rows_out);
int incin_loader_order(int64_t h, int64_t* out);
void incin_loader_destroy(int64_t h);

/* ---- runtime: arena planning by liveness (greedy first fit; skip[i] != 0 leaves buffer i out, offset -1) ---- */
int64_t incin_memplan_first_fit(int64_t n, const int64_t* sizes, const int64_t* first, const int64_t* last, const uint8_t* skip, int64_t* offsets_out);

/* ---- runtime: parallel positional reads of byte ranges of one file into caller buffers (0 ok, 1 open, 2 read, 3 args) ---- */
int incin_file_read_ranges(const char* path, int64_t n, const int64_t* offsets, const int64_t* sizes, void* const* dst, int threads);

/* ---- runtime: telemetry sink (JSON lines, bounded queue, background writer) ---- */
int64_t incin_telemetry_open(const char* path, int64_t capacity);
int incin_telemetry_scalar(int64_t h, const char* name, double value, int64_t step);
int incin_telemetry_memory(int64_t h, int device, int64_t allocated, int64_t reserved, int64_t step);
int incin_telemetry_raw(int64_t h, const char* json_line);
int64_t incin_telemetry_flush(int64_t h);
int64_t incin_telemetry_close(int64_t h);

#ifdef __cplusplus
}
#endif
#endif
