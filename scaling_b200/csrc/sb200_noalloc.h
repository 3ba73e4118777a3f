// Allocation-free entry point of libsb200 (no counterpart in the reference framework, which has no native code).
//
// Some hosts of this library must not enter the CUDA allocator on their hot path: a serving process that handed
// the whole device to its own arena at start-up has nothing left for cudaMalloc to return, a real-time loop cannot
// afford the device-wide synchronisation cudaMalloc / cudaFree imply, and a plain C caller has no tensor library
// to borrow a workspace from.  For them the backward pass of RMSNorm / LayerNorm - which needs a workspace for
// the per-CTA partial sums of the weight and bias gradients - is offered in a form that owns its workspace.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in workspace: two arrays of SB200_NOALLOC_MAX_PARTIAL_ROWS x SB200_NOALLOC_MAX_H floats
// (2 x 4 MiB).  The arrays are part of the library image on every device that loads it and stay resident until
// the process exits.
#define SB200_NOALLOC_MAX_PARTIAL_ROWS 128
#define SB200_NOALLOC_MAX_H 8192

// Same computation and argument meaning as sb200_norm_bwd, minus the caller-provided dw_partial / db_partial
// workspaces and the partial_rows count:
//   dx[M, H], dw[H] (and db[H] for LayerNorm with bias) from dy[M, H], x[M, H], w[H], mean[M] (LayerNorm), rstd[M].
//   rms != 0 selects RMSNorm; accumulate != 0 adds into dw / db; dtype is SB_DT_* of dy, x, w, dx, dw, db.
//   dy, x, w, dx, dw and db must be 16-byte aligned (the kernels move 16 bytes per access); with a row length that
//   is a multiple of the vector width this makes every row aligned as well.
// Returns 0 on success, SB_ERR_TOO_LARGE (103) if H exceeds SB200_NOALLOC_MAX_H, SB_ERR_BAD_ARG (102) if H is not
// a multiple of the 16-byte vector width, a required pointer is null or one of the pointers above is not 16-byte
// aligned (nothing is launched in these cases), or the CUDA error code of a failed runtime call.
//
// Contract:
//  * The function never calls cudaMalloc, cudaFree or any other allocating routine.
//  * The first call on each device looks up the device address of the workspace (cudaGetSymbolAddress) with that
//    device current; make this first call before any stream capture begins on that device, on any host thread (a
//    capture in progress on another thread is disturbed by the look-up just the same).
//  * All calls on a device share the one workspace.  Its contents after a call are unspecified; every call
//    overwrites the rows it later reads, so nothing needs clearing in between.  Two calls whose kernels may run
//    at the same time on one device (different streams without ordering) race on the workspace and must be
//    ordered by the caller.
int sb200_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                           void* dx, void* dw, void* db, int M, int H, int rms, int accumulate, int dtype,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
