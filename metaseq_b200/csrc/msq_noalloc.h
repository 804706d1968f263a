// Entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference (facebookresearch/metaseq): there every helper
// that needs temporary device memory gets it from PyTorch's allocator.
//
// Who needs it.  Side threads of a training or serving process -- the asynchronous
// checkpoint writer that wants the norm of a shard it is about to serialise, a failure
// watchdog that samples a gradient norm, a C or C++ host program that links this library
// without PyTorch -- run while the main thread's caching allocator already holds nearly all
// of the GPU's memory.  For them a cudaMalloc can fail although the process as a whole has
// room, and both cudaMalloc and cudaFree make the whole device wait, which stalls the step
// that is running on the main thread.  They also cannot borrow PyTorch's allocator: it is
// not theirs to call from a foreign thread, and a plain C caller does not have it at all.
//
// What it does.  msq_sumsq_noalloc computes out[0] (+)= sum(g[i]^2) over n elements, the
// same result as msq_sumsq, but keeps its per-CTA partial sums in a fixed array that lives
// inside the library image instead of in a caller-provided buffer.  It calls no cudaMalloc,
// cudaFree or any allocating routine.
//
// Limits and rules.
//   * n must satisfy 0 <= n <= MSQ_NOALLOC_MAX_ELEMS; anything else is rejected with
//     MSQ_NOALLOC_ERR_SIZE and a message on stderr, and nothing is launched.
//   * The partial-sum array has MSQ_NOALLOC_MAX_PARTS floats (4 KiB).  Every GPU that loads
//     the library holds its own copy until the process exits.
//   * The first call on a device looks up the device address of that array (once per
//     device, with that device current).  Make that first call at start-up, outside any
//     stream capture.
//   * All calls on a device share the array and it keeps whatever the previous call left
//     in it.  Each call overwrites every slot it later reads, so nothing has to be cleared,
//     but two calls whose kernels can overlap on the GPU (different streams, no ordering
//     between them) race on it: order them on one stream or with events.
//   * g and out are device pointers on the current device; `stream` belongs to it too.
#pragma once

#include <cuda_runtime.h>

#define MSQ_NOALLOC_MAX_PARTS 1024
#define MSQ_NOALLOC_MAX_ELEMS (1LL << 31)

#define MSQ_NOALLOC_OK 0
#define MSQ_NOALLOC_ERR_SIZE (-20)    // n outside [0, MSQ_NOALLOC_MAX_ELEMS]
#define MSQ_NOALLOC_ERR_DTYPE (-21)   // dtype not 0 (fp16), 1 (bf16) or 2 (fp32)
#define MSQ_NOALLOC_ERR_SYMBOL (-22)  // the device address of the scratch array could not be obtained
#define MSQ_NOALLOC_ERR_LAUNCH (-23)  // a kernel launch failed
#define MSQ_NOALLOC_ERR_ARG (-24)     // null pointer with n > 0, or misaligned g

#ifdef __cplusplus
extern "C"
#endif
int msq_sumsq_noalloc(const void* g, long long n, int dtype, float* out, int accumulate, cudaStream_t stream);
