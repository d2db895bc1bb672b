/* LayerNorm / RMSNorm backward for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference: the reference's norms are
 * compositions of host tensor ops (nn/norm.go:50-148) and own no device memory.
 *
 * Who needs it.  gb_norm_bwd (norm.cu) wants a scratch buffer for the per-CTA partial
 * sums of the weight and bias gradients, and its usual caller gets that buffer from
 * PyTorch's caching allocator.  Some callers have no allocator to ask: a host program
 * that links the shared object directly and hands over raw device pointers; a serving
 * or training loop whose memory plan is fixed before the first step, where a late
 * cudaMalloc could fail or would stall every stream of the device while it runs; code
 * running in a callback where the CUDA runtime forbids allocation.  For them the scratch
 * lives inside the library: a file-scope __device__ array of
 * 148 * 2 * 4096 floats (about 4.6 MiB) that every GPU loading the library holds until
 * the process exits.
 *
 * Contract.
 *  - Same arguments as gb_norm_bwd minus the scratch pair.  The caller still passes all
 *    inputs and outputs (x, dy, weight, mean, rstd -> dx, dgamma, dbeta).
 *  - D (row width) may be at most gb_norm_bwd_noalloc_max_dim() = 4096; larger rows are
 *    rejected with status -5 and a message from gb_last_error().
 *  - Neither this call nor anything it calls uses cudaMalloc, cudaFree or an allocating
 *    library routine.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first
 *    call during start-up, before any stream capture begins on the device.  Two host
 *    threads that make the first call on one device at the same time both store the same
 *    address, so that is harmless.
 *  - All calls on a device share the one array, and it keeps whatever the previous call
 *    left there.  The kernels overwrite every partial row before reading it, so no
 *    clearing is needed; but two calls that can run at the same time on the GPU (two
 *    streams, or two host threads) race on the array.  Serialise them on one stream.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

/* kind: 0 LayerNorm, 1 RMSNorm (mean may be null).  dtype / wdtype: 0 bf16, 1 fp16,
 * 2 fp32 for x/dy/dx and for weight/dgamma/dbeta.  dgamma / dbeta may be null.
 * Returns 0 on success. */
int gb_norm_bwd_noalloc(int kind, int dtype, int wdtype, const void* x, const void* dy,
                        const void* w, const float* mean, const float* rstd, void* dx,
                        void* dgamma, void* dbeta, long long rows, int D, void* stream);

/* Largest row width gb_norm_bwd_noalloc accepts. */
int gb_norm_bwd_noalloc_max_dim(void);

#ifdef __cplusplus
}
#endif
