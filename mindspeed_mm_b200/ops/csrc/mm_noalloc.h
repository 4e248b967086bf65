// Allocation-free entry point of the ops library.  (This has no counterpart in the reference
// framework; it exists for hosts that embed the kernels directly.)
//
// Who needs it: code that runs where device allocation is off limits -- a region being recorded for later
// replay, a real-time or interrupt-style callback, a plug-in inside a host application that owns the
// memory pool and hands out no more, or a caller whose allocator would synchronise the device and stall
// the pipeline it is part of.  Such callers can pass their inputs and outputs but cannot provide (or ask
// the library to obtain) the fp32 partial-sum workspace that the RMSNorm backward kernel needs.
//
// mm_rmsnorm_bwd_noalloc computes exactly what mm_rmsnorm_bwd computes,
//     dx = rstd * (dy*w - x*rstd * mean(dy*w * x*rstd)),   dw = sum_rows dy * x*rstd,
// but keeps the [CTAs x H] fp32 partials of dw in a fixed array that lives in the library image
// (`static __device__`, 256-byte aligned) instead of in memory supplied by the caller.
//
// Limits and rules
//   * H must be a multiple of 8 and at most MM_NOALLOC_MAX_H (4096).  The grid is capped at
//     MM_NOALLOC_MAX_CTAS (296 = 2 per SM), so the array holds 296 * 4096 floats = 4.6 MiB.  Every GPU
//     that loads the library keeps that much reserved until the process exits.
//   * Larger H, H not a multiple of 8, or T < 1 is refused with MM_NOALLOC_E_SIZE; nothing is launched.
//   * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that
//     device current) and caches it; later calls on that device only launch.  Make that first call
//     outside of any stream capture.  No call allocates or frees device or pinned memory.
//   * All calls on a device share the one array.  Nothing in it needs to start at zero (every call
//     overwrites the part it reads back), but two calls whose kernels may overlap on the GPU -- different
//     streams without an ordering between them -- race on it.  Serialise them on one stream or with events.
//   * x, w, dy: bf16; rstd: fp32 [T] as written by mm_rmsnorm_fwd; dx: bf16 [T, H]; dw: bf16 [H];
//     all device pointers, 16-byte aligned, rows dense.
#pragma once
#include <cuda_runtime.h>

#define MM_NOALLOC_MAX_H 4096
#define MM_NOALLOC_MAX_CTAS 296
#define MM_NOALLOC_E_SIZE (-20)    /* shape outside the limits above */
#define MM_NOALLOC_E_SYMBOL (-21)  /* the device address of the workspace could not be resolved */

#ifdef __cplusplus
extern "C" {
#endif
// Returns 0 on success, MM_NOALLOC_E_* on refusal, or a positive cudaError_t from the launch.
int mm_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw, int T,
                           int H, cudaStream_t stream);
// Human-readable text for the codes above.
const char* mm_noalloc_strerror(int code);
#ifdef __cplusplus
}
#endif
