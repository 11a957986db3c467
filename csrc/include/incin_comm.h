/* C ABI of the communication layer: peer-mapped ("symmetric") buffers and the fused
 * compute+collective kernels that run over them.  One process per GPU; buffers are exchanged as
 * CUDA IPC handles over any side channel (torch.distributed object collectives or the incin
 * rendezvous all-gather).  Kernels address peers with plain loads and stores. */
#ifndef INCIN_COMM_H
#define INCIN_COMM_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define INCIN_MAX_PEERS 8
#define INCIN_DP_MAX_SLOTS 64
#define INCIN_IPC_HANDLE_BYTES 64

/* cudaMalloc'ed, zero-filled buffer plus its IPC handle (these two allocate; call them at set-up). */
int incin_symm_alloc(long long bytes, void** ptr_out, uint8_t handle_out[INCIN_IPC_HANDLE_BYTES]);
int incin_symm_open(const uint8_t handle[INCIN_IPC_HANDLE_BYTES], void** ptr_out);
int incin_symm_close(void* peer_ptr);
int incin_symm_free(void* ptr);
/* 1 if `dev` can map `peer`'s memory (NVLink/NVSwitch or PCIe P2P) */
int incin_can_access_peer(int dev, int peer);

typedef struct incin_dp_desc {
  void* grads[INCIN_MAX_PEERS];   /* fp32 flat gradient buffer of every rank (own entry = local pointer) */
  void* shadows[INCIN_MAX_PEERS]; /* bf16 flat parameter buffer of every rank */
  void* pads[INCIN_MAX_PEERS];    /* signal pad of every rank, incin_dp_pad_bytes() each, zero-initialised */
  void *master, *m, *v;           /* local fp32 master weights and Adam moments (full length) */
  const void* hyper;              /* device, 8 floats: lr, beta1, beta2, eps, weight_decay, step, grad_scale, - */
  long long lo, hi, n_decay;      /* bucket [lo, hi) in elements, both multiples of 8 */
  int world, rank;
  int slot;                       /* signal slot of this bucket (< INCIN_DP_MAX_SLOTS), one per bucket */
  int ctas;                       /* grid size; small grids leave the SMs to overlapping compute */
  void* status;                   /* optional int32 device word set when a peer wait timed out */
} incin_dp_desc;

/* reduce-scatter(mean) of the bucket over peer memory + AdamW on the owned slice + all-gather of the new
 * bf16 weights, in one kernel.  Every rank must launch it for the same buckets in the same order. */
int incin_dp_reduce_adamw(const incin_dp_desc* desc, void* stream);
int incin_dp_pad_bytes(void);
/* The same kernel over NVSwitch multicast memory: `mc_grads` / `mc_shadows` are the MULTICAST addresses of the
 * gradient and parameter buffers (every rank's buffer bound at the same offset of one multicast object; the unicast
 * pointers in `desc` still name the same memory and carry the handshake pads).  The owned slice is summed inside the
 * switch with multimem.ld_reduce (1/world of the bucket crosses this GPU's links instead of (world-1)/world of it)
 * and the new bf16 weights leave once with multimem.st.  Only for groups whose ranks all stay alive while the
 * buffers are bound: a rank that exits while bound can fault its peers. */
int incin_dp_reduce_adamw_mc(const incin_dp_desc* desc, void* mc_grads, void* mc_shadows, void* stream);

/* Barrier across the GPUs of a group, as one tiny kernel per GPU: every rank signals every peer's pad and waits
 * (bounded) for theirs.  When it has completed on a GPU, every peer has reached the same point of its stream, i.e.
 * every kernel the peers enqueued before their barrier has finished.  pads[r] = rank r's pad (incin_barrier_pad_bytes()
 * bytes, zero-initialised, one pad per group); `slot` picks one of 64 independent barriers in the pad. */
int incin_peer_barrier(void* const* pads, int world, int rank, int slot, void* status, void* stream);
int incin_barrier_pad_bytes(void);

/* In-place all-reduce(sum) of fp32 ranges over a peer group, for the few tensors a tensor-parallel job keeps
 * replicated inside a sub-group.  Two launches around a barrier: stage 0 sums the peers' ranges into `scratch`
 * (local, fp32, at least total length), stage 1 copies scratch back.  ranges = int64 [n_ranges][2] (offset, length)
 * in device memory, offsets relative to each rank's base pointer. */
int incin_peer_sum_ranges(void* const* bases, int world, const void* ranges, int n_ranges, void* scratch, int stage,
                          void* stream);

/* ---- stand-alone collectives over peer-mapped buffers (collectives.cu) -------------------------------------
 * bufs[r] = rank r's symmetric buffer as mapped here (HOST array of `world` pointers).  Sizes and offsets are
 * multiples of 16 bytes.  Bracket each call with incin_peer_barrier on the same stream. */
/* out[r * bytes ..] = bufs[r][offset .. offset + bytes) */
int incin_coll_all_gather(void* const* bufs, int world, int rank, long long offset_bytes, long long bytes, void* out,
                          void* stream);
/* out[r * chunk ..] = bufs[r][offset + rank * chunk .. + chunk) */
int incin_coll_all_to_all(void* const* bufs, int world, int rank, long long offset_bytes, long long chunk_bytes, void* out,
                          void* stream);
/* out[i] = reduce_r bufs[r][offset + first_elem + i], i < n; op 0 sum, 1 mean, 2 max, 3 min; fp32 or bf16 elements.
 * reduce-scatter: first_elem = rank * n; all-reduce: first_elem = 0 and n = whole length.  Rank order is fixed,
 * so every rank gets bitwise the same sums. */
int incin_coll_reduce(void* const* bufs, int world, long long offset_bytes, long long first_elem, long long n, int op,
                      int is_bf16, void* out, void* stream);
/* Pipeline transfers: copy `bytes` into the receiver's buffer, then release `seq` into the receiver's flag word.
 * The receiver's wait spins on its own flag for at most timeout_ms (<= 10 s) and records status 5 when it gives up. */
int incin_p2p_send(void* peer_dst, const void* src, long long bytes, void* peer_flag, unsigned seq, void* stream);
int incin_p2p_wait(const void* local_flag, unsigned seq, void* status, long long timeout_ms, void* stream);

#ifdef __cplusplus
}
#endif
#endif
