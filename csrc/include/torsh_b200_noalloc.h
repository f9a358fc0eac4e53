/* Allocation-free entry point of libtorsh_b200_cuda.so.
 *
 * This entry point has no counterpart in the reference framework (cool-japan/torsh): it exists for
 * callers of THIS library that are not allowed to allocate device memory at the moment they call -
 * code between cudaStreamBeginCapture and cudaStreamEndCapture, latency-critical serving loops
 * that forbid allocator traffic, and C / FFI hosts that have no device allocator of their own.
 *
 * tb_norm_bwd_static computes exactly what tb_norm_bwd computes (LayerNorm / RMSNorm backward:
 * dx, and dgamma / dbeta ACCUMULATED into the given fp32 buffers) but takes its scratch memory from a
 * fixed 8 MiB device array inside the library instead of from the caller.
 *
 *  - Inputs and outputs are still the caller's buffers.
 *  - A problem is accepted when tb_norm_bwd_workspace(rows, H) <= tb_norm_bwd_static_capacity()
 *    (both in floats); otherwise the call returns TB_E_TOO_LARGE (-4) and tb_last_error() says why.
 *  - All calls on a device share the one array: calls whose kernels may overlap on the GPU race.
 *    Keep them on one stream or order them with events.
 *  - The first call on each device resolves the array's device address (with that device current),
 *    and the first call of every host thread selects the device for that thread (cudaSetDevice, which
 *    creates the device's context if the process has none yet). Make one call per host thread and
 *    device before any stream capture starts.
 *  - No cudaMalloc, cudaFree or other allocating routine is called, on any path.
 */
#ifndef TORSH_B200_NOALLOC_H
#define TORSH_B200_NOALLOC_H

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Capacity of the built-in scratch array, in floats. */
long tb_norm_bwd_static_capacity(void);

/* dtype: 0 = bf16, 1 = fp32 (x, dy, dx, gamma). rms: 0 = LayerNorm, 1 = RMSNorm (mean may be NULL).
 * dres (optional) is added to dx. dbeta may be NULL. Returns 0 on success. */
int tb_norm_bwd_static(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                       const void* dres, void* dx, float* dgamma, float* dbeta, int rows, int H, int rms,
                       int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
