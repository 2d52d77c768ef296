/* kwu_rmsnorm_bwd_noalloc — RMSNorm backward that never asks for memory.
 *
 * This entry point has no counterpart in the reference project; it exists for hosts of this library
 * that are not allowed to allocate on the device. Examples: a plugin running inside a serving or
 * training runtime that owns the whole memory pool and hands the plugin only its input and output
 * tensors; code running where an allocation would be an error or a stall (inside another framework's
 * captured region, in a real-time loop, under a fixed memory budget checked by an auditor); bindings
 * for languages that have no device allocator of their own. Such callers can still pass the
 * operands, because those already exist, but they have nowhere to get the temporary buffer that
 * kwu_rmsnorm_bwd needs for the weight-gradient partial sums.
 *
 * What it computes is exactly what kwu_rmsnorm_bwd computes:
 *     dx = rstd * (dy*w_eff - xhat * mean(dy*w_eff*xhat)) [+ dres],   dw (+)= sum_rows dy * xhat
 * with x, dy, dres, dx in bf16 (rows x cols, contiguous), w, rstd, dw in fp32. w, dres and dw may be
 * null (no scale / no residual gradient / no weight gradient wanted).
 *
 * Contract
 *  - The temporary lives in an array of KWU_NOALLOC_MAX_BLOCKS x KWU_NOALLOC_MAX_COLS floats
 *    (2.3 MiB) that is part of the library image. Every GPU on which the library is loaded holds that
 *    array until the process ends, whether or not this function is ever called.
 *  - cols must be a multiple of 8 and at most KWU_NOALLOC_MAX_COLS; anything larger is refused with
 *    a non-zero return code and a message available from kwu_last_error(). rows is unlimited.
 *  - No cudaMalloc / cudaFree / allocating library routine is called, on any path.
 *  - The first call on each device looks up the device address of the array (one
 *    cudaGetSymbolAddress, with that device current) and remembers it. Make that first call outside
 *    of any stream capture; later calls only launch kernels on the given stream.
 *  - All calls on one device share the one array, and it keeps whatever the last call left in it.
 *    Nothing needs to be cleared between calls (each call overwrites every entry it later reads),
 *    but two calls whose kernels can run at the same time on one GPU (different streams, different
 *    threads) would overwrite each other's partial sums: serialise them, e.g. by using one stream.
 *  - Returns 0 on success.
 */
#ifndef KWU_NOALLOC_H_
#define KWU_NOALLOC_H_

#define KWU_NOALLOC_MAX_COLS 4096
#define KWU_NOALLOC_MAX_BLOCKS 148

#ifdef __cplusplus
extern "C" {
#endif

int kwu_rmsnorm_bwd_noalloc(const void* x, const float* w, const float* rstd, const void* dy,
                            const void* dres, void* dx, float* dw, int rows, int cols, int one_plus,
                            int accumulate_dw, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* KWU_NOALLOC_H_ */
