// Allocation-free entry point of the library (plain C ABI).
//
// This entry point has no counterpart in the reference: the reference is pure Python on top of PyTorch and
// never exposes a C symbol, let alone one with a fixed memory footprint.
//
// Who needs it. Most of this library obtains its temporary buffers from the PyTorch caching allocator, which
// in turn calls cudaMalloc when its pools run dry. Some hosts cannot tolerate that: a process that has handed
// the whole device memory to another runtime (an inference server or a second framework with its own arena),
// a plain C/C++ program that links this library without PyTorch and has no allocator to lend, or a
// latency-critical loop in which a device allocation -- a driver call that may synchronise the device and may
// fail once memory is fragmented -- is not acceptable in the middle of the run. Such callers own every buffer
// they pass in and need the guarantee that the library takes nothing more from the device heap.
//
// What it is. pt_rmsnorm_bwd_noalloc computes exactly what pt_rmsnorm_bwd computes (the RMSNorm backward:
// dx, plus the weight gradient dw reduced over all rows), but the per-CTA partial sums of dw, which the
// regular entry point takes as a caller-provided scratch buffer, live in a file-scope __device__ array that is
// part of the library image. Inputs and outputs are still the caller's.
//
// Limits and rules:
//   * H must be a multiple of 8 and at most PT_NOALLOC_MAX_H; T must be positive. Larger problems are rejected
//     with PT_NOALLOC_ERR_TOO_LARGE before anything is launched (pt_noalloc_strerror gives the text).
//   * The scratch array holds PT_NOALLOC_MAX_ROWS x PT_NOALLOC_MAX_H floats (2 MiB). Every device that loads
//     the library carries it from load until the process exits, whether or not this entry point is used.
//   * The first call on each device resolves the array's device address (cudaGetSymbolAddress with that
//     device current) and caches it; make that first call outside of any stream capture. No call -- first or
//     later -- allocates or frees device memory. The address cache is a plain per-device table written without a lock:
//     two host threads making the FIRST call on the same device at the same moment both resolve the same address, which
//     is harmless, but do not rely on that first call being cheap; make it once, from one thread, during set-up.
//   * All calls on a device share the one array and it keeps whatever the previous call left in it. The
//     kernels overwrite every element they later read, so nothing needs clearing, but two calls whose
//     kernels overlap on the GPU (different streams, no ordering) race on it: order them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PT_NOALLOC_MAX_H 4096
#define PT_NOALLOC_MAX_ROWS 128

#define PT_NOALLOC_OK 0
#define PT_NOALLOC_ERR_BAD_SHAPE (-20)   /* H not a multiple of 8, or T <= 0 */
#define PT_NOALLOC_ERR_TOO_LARGE (-21)   /* H > PT_NOALLOC_MAX_H */
#define PT_NOALLOC_ERR_SYMBOL (-22)      /* the scratch array's device address could not be resolved */
#define PT_NOALLOC_ERR_LAUNCH (-23)      /* a kernel launch failed */

// dy, x, dres (may be NULL), dx: bf16 [T, H] row-major; w: bf16 [H]; rstd: fp32 [T]; dw: fp32 [H] (overwritten).
// Returns PT_NOALLOC_OK or one of the error codes above. Work is enqueued on `stream`.
int pt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                           void* dx, float* dw, int T, int H, cudaStream_t stream);

// Human-readable text for a return code of pt_rmsnorm_bwd_noalloc.
const char* pt_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
