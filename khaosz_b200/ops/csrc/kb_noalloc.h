// Allocation-free entry point of the khaosz_b200 kernel library.
//
// This entry point has no counterpart in the reference framework.  It exists for callers
// that are not allowed to allocate device memory at the point where they need the kernel:
// code running inside a memory-pool or arena owner that forbids re-entrant allocation,
// real-time / serving loops that must not take the allocator lock, and hosts that
// pre-reserve all device memory at start-up so that a later cudaMalloc would simply fail.
// Such callers can still pass their own input and output buffers, but they have nowhere to
// get the kernel's scratch buffer from.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Limits of kb_rmsnorm_bwd_static: the scratch lives in a fixed 4 MiB array inside the
// library's device image (KB_STATIC_RMS_MAX_PARTIALS x KB_STATIC_RMS_MAX_DIM floats), which
// every GPU that loads the library holds until the process exits.
#define KB_STATIC_RMS_MAX_DIM 4096
#define KB_STATIC_RMS_MAX_PARTIALS 256

// RMSNorm backward, same mathematics and argument meaning as kb_rmsnorm_bwd, minus the
// caller-provided scratch:
//   dx[rows, dim]  = d rmsnorm(x) (+ dres_in)        bf16
//   dw[dim]        = sum over rows of dy * x * rstd   fp32, overwritten
// dy, x, dres_in (optional), dx: bf16 [rows, dim]; w: bf16 [dim]; rstd: fp32 [rows].
//
// Returns KB_STATUS_OK, KB_STATUS_BAD_ARG (dim not a multiple of 8, misaligned pointer),
// KB_STATUS_TOO_LARGE when dim > KB_STATIC_RMS_MAX_DIM (kb_rmsnorm_bwd_static_error() then
// holds a readable message), or KB_STATUS_CUDA_ERROR.
//
// * No cudaMalloc / cudaFree / allocating library call is made, on any call.
// * The first call on each device resolves the device address of the scratch array (with
//   that device current).  Make that first call outside of any stream capture.
// * All calls on a device share the one scratch array and it keeps the last call's
//   contents.  Nothing in it has to start at zero: every launch overwrites the rows it later
//   reads.  Two calls that overlap on the GPU (different streams) race on it; serialise them.
int kb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                          const void* dres_in, void* dx, float* dw, int rows, int dim,
                          void* stream);

// Message describing the last failure of kb_rmsnorm_bwd_static on the calling thread.
const char* kb_rmsnorm_bwd_static_error(void);

#ifdef __cplusplus
}
#endif
