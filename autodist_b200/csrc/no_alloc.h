// Column sums of a bf16 matrix for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which has no device code at all); it exists for users of
// this library who reach the kernels from a place where a cudaMalloc is not possible: inside a host callback or
// another library's stream-ordered region, in a process whose memory pool is owned by someone else and must not
// grow, or in a hard real-time loop where an allocation's latency (and its implicit device synchronisation) is not
// acceptable. The ordinary entry point (`keyed_colsum` in elementwise.cu, reached through the Python bindings) asks
// the caller for a scratch tensor; this one brings its own.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest matrix width this entry point accepts. The library keeps 16 * ADB200_NOALLOC_MAX_COLS floats (2 MiB) of
// scratch in a file-scope __device__ array, so every GPU that loads the library holds that much until exit.
#define ADB200_NOALLOC_MAX_COLS 32768

// out[c] = sum over r of x[r * cols + c]   (x: bf16 [rows, cols] row-major on the current device, out: fp32 [cols]).
//
// * Allocates nothing: no cudaMalloc / cudaFree / allocating library call, on any call.
// * cols must be a multiple of 8 and at most ADB200_NOALLOC_MAX_COLS, rows >= 1; x must be 16-byte aligned.
//   Anything else is refused with a non-zero return code and a message (adb200_noalloc_last_error()).
// * The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress) with
//   that device current. Make that first call before any stream capture begins.
// * Every call on a device shares the one scratch array, which keeps whatever the previous call left in it. The
//   kernels overwrite every word they later read, so nothing needs clearing between calls; but two calls whose
//   kernels overlap on the GPU (different streams, no ordering between them) race on the scratch and give wrong sums.
//   Calls on one stream are safe.
// Returns 0 on success, otherwise a cudaError_t value or one of the ADB200_NOALLOC_* codes below.
int adb200_colsum_bf16_noalloc(const void* x_bf16, float* out, int rows, int cols, cudaStream_t stream);

// Human-readable reason of the last refusal on this host thread ("" if the last call succeeded).
const char* adb200_noalloc_last_error(void);

#define ADB200_NOALLOC_BAD_SHAPE 10001
#define ADB200_NOALLOC_TOO_WIDE 10002
#define ADB200_NOALLOC_BAD_POINTER 10003

#ifdef __cplusplus
}
#endif
