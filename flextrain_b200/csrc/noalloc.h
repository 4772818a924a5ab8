// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for embedders that run
// inside an environment where cudaMalloc / cudaFree are off limits at call time: code executing under a
// fixed memory budget that was carved up in advance, plugins of a host application that owns the
// allocator and forbids foreign allocations, and latency-critical loops where an allocation could
// synchronise the device.  Such callers can still pass their own input and output buffers, but they
// cannot provide (or do not want to size) the kernel's internal workspace.
//
// The regular entry point, ftb_rmsnorm_bwd (elementwise.cu), needs a caller-provided fp32 workspace of
// (blocks x D) for the two-stage weight-gradient reduction.  ftb_rmsnorm_bwd_noalloc computes the same
// results but keeps that workspace in a file-scope __device__ array inside the library
// (FTB_NOALLOC_MAX_BLOCKS x FTB_NOALLOC_MAX_D floats = 4.6 MiB, held by every GPU that loads the
// library until the process exits).
//
// Contract
//   * Inputs and outputs are the caller's: dy, x, dx (T x D, bf16), w (D, fp32) or NULL, rstd (T, fp32), optional
//     dx_add / y_out (T x D, bf16), optional dw (D, fp32; accumulated when dw_accumulate != 0).
//   * Every tensor pointer (dy, x, dx, dx_add, y_out, w, dw) must be 16-byte aligned (rows move as 16-byte vectors);
//     a misaligned or missing required pointer is rejected with FTB_NOALLOC_ERR_BAD_POINTER before any launch.
//     Without w the normalisation has no gain; asking for dw without w is rejected with the same code.
//   * `stream` must belong to the device that is current when the call is made: the workspace address is looked up for
//     the current device.  Host threads may call concurrently (the address cache is benign to race on), but see the
//     last point about calls that overlap on the GPU.
//   * D must be a multiple of 8 and at most FTB_NOALLOC_MAX_D; larger D is rejected with
//     FTB_NOALLOC_ERR_TOO_LARGE and nothing is launched.  ftb_noalloc_strerror() turns a code into text.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any call.
//   * The first call on each device resolves the device address of the workspace
//     (cudaGetSymbolAddress, with that device current).  Make that first call outside of any stream
//     capture; later calls only launch kernels.
//   * All calls share the one workspace and it keeps whatever the previous call left in it.  The kernels
//     overwrite every element they later read, so nothing has to be cleared, but two calls that overlap on
//     the GPU (different streams, no ordering between them) race on it.  Order them with events or use
//     one stream.
#pragma once
#include <cuda_runtime.h>

#define FTB_NOALLOC_MAX_D 8192
#define FTB_NOALLOC_MAX_BLOCKS 148

#define FTB_NOALLOC_ERR_TOO_LARGE (-3)
#define FTB_NOALLOC_ERR_BAD_SHAPE (-2)
#define FTB_NOALLOC_ERR_SYMBOL (-4)
#define FTB_NOALLOC_ERR_BAD_POINTER (-5)

#ifdef __cplusplus
extern "C" {
#endif

int ftb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const void* dx_add,
                            void* dx, void* y_out, float* dw, int dw_accumulate, int T, int D, cudaStream_t stream);

const char* ftb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
