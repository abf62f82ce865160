// Entry points of libfsb200 that never allocate memory.
//
// These have no counterpart in the reference library; they exist for callers that must not allocate while
// they run: code between cudaStreamBeginCapture and cudaStreamEndCapture, a process whose allocator is
// owned by another runtime and must not be re-entered, or a tight loop that cannot afford an allocator's
// synchronisation.  Such callers cannot hand the kernel a workspace from torch or cudaMalloc, so the
// workspace lives inside the library as a fixed device array.  (They still launch kernels: do not call them
// from a host function enqueued on a stream, where CUDA forbids runtime calls altogether.)
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of columns fsb_colsum_static accepts.  The built-in workspace holds 48 strips of this many
// fp32 partial sums (1.5 MiB per device).
#define FSB_COLSUM_STATIC_MAX_H 8192

// Return codes of fsb_colsum_static (0 = launched).
#define FSB_NOALLOC_ERR_SHAPE (-1)       // H is not a multiple of 8
#define FSB_NOALLOC_ERR_TOO_LARGE (-2)   // H exceeds FSB_COLSUM_STATIC_MAX_H: use fsb_colsum with your own workspace
#define FSB_NOALLOC_ERR_DEVICE (-3)      // current device ordinal is outside the table kept by the library (64)
#define FSB_NOALLOC_ERR_SYMBOL (-4)      // the runtime could not resolve the workspace on this device

// out[c] = sum over r of x[r, c], for a bf16 matrix x[rows, H] in device memory; out is bf16 [H].
// Same arithmetic and the same result as fsb_colsum, but without a caller-provided workspace and without
// any allocation: no cudaMalloc, no cudaFree, no library routine that allocates.
//
//  * The first call on each device looks up the address of the built-in workspace (cudaGetSymbolAddress,
//    with that device current).  Make that first call outside of any stream capture; later calls on the
//    same device only launch two kernels on `stream`.
//  * The workspace is one array per device, shared by every caller and never cleared: it still holds the
//    partial sums of the previous call.  Nothing in it needs to start at zero, since each call overwrites
//    every element that it later reads.  Two calls that may run at the same time on one device (different
//    streams, or different host threads) race on it; order them with events or use fsb_colsum instead.
//  * H > FSB_COLSUM_STATIC_MAX_H is refused with FSB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
//
// Other non-zero values are cudaError_t codes from the launch.
int fsb_colsum_static(const void* x, long long rows, int H, void* out, cudaStream_t stream);

// The limit above, for callers that load the library dynamically.
int fsb_colsum_static_max_h(void);

// Text for a return code of fsb_colsum_static (static storage, never null).
const char* fsb_colsum_static_strerror(int code);

#ifdef __cplusplus
}
#endif
