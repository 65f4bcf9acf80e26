/* Entry points of libpb200_kernels.so that allocate no device memory.
 *
 * This has no counterpart in the reference project; it exists for users of this
 * library whose call site cannot allocate: a host that runs inside a memory pool
 * owning the whole GPU, a server or real-time loop that fixes its memory plan
 * before it starts, or a plug-in that receives only its input and output buffers.
 *
 * pb_rmsnorm_bwd_noalloc is pb_rmsnorm_bwd (RMSNorm backward: dx, and dw summed over
 * rows in a fixed order) with the per-CTA partial sums kept in a fixed device array
 * inside the library instead of a caller-provided scratch buffer.
 *
 *   dy, h   bf16 [rows, d]   upstream gradient and the normalised input
 *   w       fp32 [d]         norm weight          rstd  fp32 [rows]  saved 1/rms
 *   dres    bf16 [rows, d] or NULL: gradient of the residual stream, added to dx
 *   dx      bf16 [rows, d]   out                  dw    fp32 [d]     out (+= if accumulate)
 *
 * Returns 0 on success, a CUDA error code, or 3 (bad argument) when d is not a
 * multiple of 8 or exceeds pb_rmsnorm_bwd_noalloc_max_d() (2048): nothing is
 * launched in that case. The array costs about 2.3 MiB on every GPU that loads the
 * library, for the life of the process. The first call on a device resolves the
 * array's address; make it before starting a stream capture on that device. All
 * calls on a device share the array, so calls that overlap on the GPU race:
 * issue them on one stream or order them with events.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int pb_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const void* rstd,
                           const void* dres, void* dx, void* dw, int accumulate, int rows, int d,
                           cudaStream_t stream);
int pb_rmsnorm_bwd_noalloc_max_d(void);

#ifdef __cplusplus
}
#endif
