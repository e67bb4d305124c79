// sllm_noalloc.h: the library's one entry point that allocates nothing.
//
// This entry point has no counterpart in the reference project.  It exists for callers that
// cannot allocate device memory at the moment they need a product: code running inside a
// region where the allocator must stay untouched (another framework's memory pool being
// measured or frozen, a real-time loop that may not block on the driver's allocation lock),
// or a host that hands this library raw device pointers from its own arena and forbids
// cudaMalloc altogether.  The engine's normal path is unaffected and does not use it.
//
//   int sllm_linear_stream_noalloc(x, W, bias, out, M, N, K, splits, stream)
//
//   out[M, N] (float32) = x[M, K] (bfloat16) * W[N, K]^T (bfloat16) + bias[N] (float32 or null),
//   by the k-split weight-streaming kernel: `splits` slices of K are multiplied by different
//   CTAs and added up afterwards.  The caller passes inputs and output; the partial sums,
//   which the ordinary entry point (sllm_linear_stream) wants in scratch memory supplied by
//   the caller, live here in an array compiled into the library.
//
// Limits and rules:
//   * M <= 64 (what the kernel takes; the engine's own dispatch sends it at most 32 rows, because
//     beyond that another kernel is faster), K a multiple of 128, and
//     splits' x M x N <= SLLM_NOALLOC_SCRATCH_FLOATS, where
//     splits' = sllm_linear_stream_splits(K, splits).  Larger requests are refused with an
//     error code and a message (sllm_last_error); nothing is launched.
//   * The array costs SLLM_NOALLOC_SCRATCH_FLOATS * 4 bytes (8 MiB) of device memory on every
//     GPU that loads the library, from load to process exit, used or not.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress)
//     and remembers it.  Make that first call before any stream capture begins.
//   * All calls share the one array.  Two calls whose kernels can overlap on the GPU (different
//     streams, or one stream per thread) race on it; keep calls on one stream, or order them
//     with events.  The array keeps the last call's partial sums; a call overwrites every
//     element it later reads, so nothing has to be cleared between calls.
//   * It calls no cudaMalloc, cudaFree or any allocating routine, and returns 0 on success.
#pragma once

#include <cuda_runtime.h>

#define SLLM_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int sllm_linear_stream_noalloc(const void* x, const void* W, const float* bias, float* out, int M, int N, int K,
                               int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
