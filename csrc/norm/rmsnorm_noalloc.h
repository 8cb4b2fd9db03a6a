// Allocation-free RMSNorm backward.
//
// This entry point has no counterpart in the reference; it exists for callers that must not touch
// the device allocator when they call into this library: code running inside a CUDA-graph
// stream capture (where cudaMalloc is illegal), callers that own a fixed memory budget and hand
// out every byte themselves, and real-time or signal-adjacent paths in which an allocator lock
// or an implicit device synchronisation is unacceptable.  `b200_rmsnorm_bwd` needs a
// caller-provided scratch buffer for its per-block partial sums of the weight gradient; this
// variant keeps that scratch inside the library instead.
//
// The scratch is one file-scope `__device__` array of
//     B200_NOALLOC_MAX_BLOCKS x B200_NOALLOC_MAX_H floats  (592 x 2048 x 4 B = 4.6 MiB),
// which every GPU that loads this library holds until the process exits.  Nothing is allocated or
// freed by the call, neither with cudaMalloc/cudaFree nor through any allocating library routine.
//
// Set-up: the first call on a device looks up the array's device address (once per device, with
// that device current).  Make that first call outside of any stream capture; later calls only
// enqueue two kernels on `stream`.
//
// Sharing: all calls on a device use the same array.  Every launch overwrites exactly the part of
// it that it later reads, so no clearing is needed between calls and old contents never leak into
// a result - but two calls whose kernels can overlap on the GPU (different streams without an
// ordering between them) race on the array.  Serialise them.
//
// Limits: H must be a multiple of 8 and at most B200_NOALLOC_MAX_H; larger or odd sizes are
// rejected with B200_NOALLOC_ERR_SIZE before anything is enqueued.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_NOALLOC_MAX_H 2048
#define B200_NOALLOC_MAX_BLOCKS 592

#define B200_NOALLOC_OK 0
#define B200_NOALLOC_ERR_SIZE (-1)    /* H not a multiple of 8, H > B200_NOALLOC_MAX_H, or T < 0 */
#define B200_NOALLOC_ERR_SETUP (-2)   /* the scratch array's address could not be obtained */
#define B200_NOALLOC_ERR_LAUNCH (-3)  /* a kernel launch was refused */
#define B200_NOALLOC_ERR_ARG (-4)     /* a required pointer is null */
#define B200_NOALLOC_ERR_PRIOR (-5)   /* an earlier CUDA error is still pending on this thread; nothing enqueued */

// dx[T,H] (bf16) = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dres);   dw_out[H] (fp32) (+)= sum_t dy*xhat
//   dy, x, dx : bf16 [T, H]      rstd : fp32 [T]      w : fp32 [H]
//   dres      : bf16 [T, H] or null (a second gradient to add into dx)
//   dw_accumulate != 0 adds into dw_out instead of overwriting it.
// Same arithmetic and the same summation order as b200_rmsnorm_bwd.
int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* rstd, const float* w, const void* dres,
                             void* dx, float* dw_out, int dw_accumulate, int T, int H, cudaStream_t stream);

// Human-readable text for a return code of the function above.
const char* b200_rmsnorm_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
