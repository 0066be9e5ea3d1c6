// An entry point for callers that are not allowed to allocate device memory.
//
// This function has no counterpart in the reference (Cambricon CATCH); it exists
// only in this library.
//
// Who needs it: code that runs where cudaMalloc / cudaFree (or a framework
// allocator that may fall through to them) must not be called -- for example a
// latency-critical service thread whose rules forbid calls that can synchronise
// the whole device, a plugin running inside another program's memory budget, or
// a caller that has handed all of its device memory to a different allocator.
// The regular batch-norm statistics path (b200_bn_stats + b200_bn_finalize) asks
// its caller for a zero-filled fp64 scratch buffer of 2*C doubles; this variant
// keeps that scratch in a fixed array inside the library instead, so the caller
// passes only its input and its two outputs.
#pragma once
#include "kernels_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Largest channel count the built-in scratch array can serve.  The array holds
// 2 * B200_NOALLOC_BN_MAX_CHANNELS doubles (64 KiB) and is resident on every GPU
// that loads the library until the process exits.
#define B200_NOALLOC_BN_MAX_CHANNELS 4096

// Per-channel batch statistics of x, a dense [rows, C] tensor (channels
// innermost, dtype B200_F32 / B200_BF16 / B200_F16):
//     mean[c]   = average of x[:, c]
//     invstd[c] = 1 / sqrt(biased variance of x[:, c] + eps)
// `mean` and `invstd` are caller-owned fp32 device arrays of C elements.
//
// * Allocates nothing: no cudaMalloc / cudaFree and no allocating library call.
// * C must be a multiple of 4 (fp32) or 8 (16-bit types) and at most
//   B200_NOALLOC_BN_MAX_CHANNELS; larger C returns cudaErrorInvalidValue (1)
//   without launching anything.
// * The first call on a device looks up the scratch array's device address
//   (once per device, with that device current).  Make that first call before
//   starting any stream capture.
// * All calls share the one scratch array.  The function clears the part it uses
//   at the start of every call, so results do not depend on earlier calls, but
//   two calls whose kernels overlap on the GPU (different streams, no ordering
//   between them) race on it: order such calls yourself.
// Returns 0 or a CUDA error code (see b200_error_string).
B200_API int b200_bn_batch_stats_noalloc(const void* x, int x_dtype, long long rows, int C, float eps, float* mean,
                                         float* invstd, void* stream);

#ifdef __cplusplus
}
#endif
