/* Allocation-free LayerNorm backward.
 *
 * This entry point has no counterpart in the reference project.
 *
 * Who it is for: code that must not, or cannot, reach the CUDA allocator at the moment it needs a
 * LayerNorm backward pass -- a host thread that runs while another thread is capturing work, a
 * plugin that was handed a stream and raw pointers but owns no memory pool, a real-time loop that
 * may not block on the allocator's locks, or a C caller that links this library without PyTorch and
 * therefore has no caching allocator behind it.  The regular incin_layernorm_bwd() asks such a caller
 * to bring an fp32 scratch buffer for the dgamma/dbeta partial sums; this variant brings its own.
 *
 * How: the scratch lives in a fixed array in the library's device data segment
 * (INCIN_LN_NOALLOC_MAX_FLOATS floats = 4 MiB).  Every GPU that loads the library holds that array
 * until the process exits, whether or not this function is ever called.  The function itself calls
 * no cudaMalloc/cudaFree and no allocating library routine.
 *
 * Limits and rules:
 *   - incin_layernorm_bwd_scratch_floats(rows, C) must not exceed INCIN_LN_NOALLOC_MAX_FLOATS
 *     (that is C <= 8192 for any row count); larger problems return INCIN_ERR_TOO_LARGE and launch
 *     nothing.
 *   - The first call on each device looks up the device address of the array (one
 *     cudaGetSymbolAddress with that device current).  Make that first call outside any stream
 *     capture; later calls on the same device only launch kernels.
 *   - All calls on one device share the one array, and it keeps whatever the previous call left in
 *     it.  The kernels overwrite every element they later read, so nothing needs clearing between
 *     calls, but two calls that overlap on the GPU (different streams, no dependency) race on it
 *     and produce wrong dgamma/dbeta.  Order them on one stream or with events.
 *   - Inputs, outputs and semantics are exactly those of incin_layernorm_bwd(): dgamma/dbeta are
 *     accumulated into, dx_add may be NULL.
 */
#ifndef INCIN_B200_NOALLOC_H
#define INCIN_B200_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define INCIN_LN_NOALLOC_MAX_FLOATS (64LL * 2 * 8192)

int incin_layernorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean,
                                const float* rstd, const void* dx_add, void* dx, float* dgamma, float* dbeta,
                                long long rows, int C, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INCIN_B200_NOALLOC_H */
