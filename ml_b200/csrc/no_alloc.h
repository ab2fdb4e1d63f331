// Allocation-free entry point of the RMSNorm backward kernel.
//
// This entry point has no counterpart in the reference trainer; it exists for callers of this library that are not
// in a position to allocate device memory at all:
//   * host code that has handed the whole device to its own arena or pool and forbids any other cudaMalloc,
//   * latency-critical loops, where cudaMalloc / cudaFree would synchronise the device and stall every stream,
//   * plug-ins and callbacks that run where the CUDA allocation calls (and torch's caching allocator) are off limits.
// The regular entry point, mlb_rmsnorm_bwd, needs a scratch buffer and a few zeroed counters from its caller.  This
// variant takes only inputs and outputs: its scratch is a fixed array that lives inside the library image on every GPU
// that loads the library (about 2.5 MB per GPU, held until the process exits).
//
// Limits and rules
//   * C (row width) must be at most MLB_NOALLOC_RMS_MAX_C, and C * 4 bytes of shared memory must fit the default 48 KB;
//     anything larger is refused with MLB_NOALLOC_ERR_TOO_LARGE and a message (mlb_rmsnorm_bwd_noalloc_error()).
//   * The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress) with that
//     device current.  Make that first call outside of any stream capture.  Host threads that make their first calls
//     on one device at the same moment may each run that look-up; they all obtain and store the same address (a plain
//     pointer-sized write of an identical value), so the set-up needs no lock and the order does not matter.
//   * All calls on a device share the one scratch array, and the array keeps whatever the previous call left in it.
//     The entry point clears the counters that have to start at zero on the caller's stream before each launch.
//     Two calls that overlap on the GPU (different streams, no ordering between them) race on the scratch.
//   * Nothing in this path calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLB_NOALLOC_RMS_MAX_C 2048
#define MLB_NOALLOC_ERR_TOO_LARGE (-10)
#define MLB_NOALLOC_ERR_SETUP (-11)

// dx[rows,C] (bf16) = add + rstd*w*dy - x*rstd^3/C * sum_c(dy*w*x);  dw[C] (fp32) += sum over rows of dy*x*rstd.
// dy, x, add (optional, may be NULL): bf16 [rows,C]; w: bf16 [C]; rstd: fp32 [rows].  All pointers are device memory.
// Returns 0, a negative MLB_NOALLOC_ERR_* code, or a positive cudaError_t.
int mlb_rmsnorm_bwd_noalloc(void* dx, float* dw, const void* dy, const void* x, const void* w, const float* rstd,
                            const void* add, long rows, int C, cudaStream_t stream);

// Text of the last refusal on this thread's most recent failing call ("" if none).
const char* mlb_rmsnorm_bwd_noalloc_error(void);

#ifdef __cplusplus
}
#endif
