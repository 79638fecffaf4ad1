// Entry points that never allocate: their scratch lives in a fixed device array that is part of
// the library image.  This file has no counterpart in the reference project; it exists for hosts
// that use libareno_kernels.so directly.
//
// Who needs this.  The ordinary entry points take their scratch from the caller, and the Python
// wrappers get it from PyTorch's caching allocator.  Some callers have no allocator to ask, or may
// not ask it at the point of the call:
//   * a C or C++ host that links this library without PyTorch: its only sources are cudaMalloc
//     and cudaFree, which serialise against all work on the device and can fail outright when a
//     trainer has already filled the card;
//   * code that runs inside an allocator callback or an out-of-memory handler, where asking the
//     allocator again would re-enter it;
//   * a latency-critical loop that must not wait on an allocator lock held by another thread.
// For them the call below needs nothing but its arguments.
#pragma once
#include <cuda_runtime.h>

extern "C" {

// Largest hidden size the fixed scratch can serve, and the scratch size in bytes.
// The array holds ARENO_RMSNORM_BWD_STATIC_BLOCKS x ARENO_RMSNORM_BWD_STATIC_MAX_H floats
// (148 x 8192 x 4 B = 4,849,664 B per device that loads the library).
#define ARENO_RMSNORM_BWD_STATIC_BLOCKS 148
#define ARENO_RMSNORM_BWD_STATIC_MAX_H 8192

// Error codes of this file (all negative; positive values are cudaError_t numbers).
#define ARENO_NOALLOC_ERR_H_TOO_LARGE (-10)   // H exceeds ARENO_RMSNORM_BWD_STATIC_MAX_H
#define ARENO_NOALLOC_ERR_SYMBOL (-11)        // the scratch symbol could not be resolved on this device
#define ARENO_NOALLOC_ERR_DEVICE (-12)        // device ordinal outside the per-device table (>= 64)

// RMSNorm backward, same mathematics and arguments as areno_rmsnorm_bwd minus `dw_partial`:
//   g = dy * (w + w_offset);  dx = inv_rms * (g - h * inv_rms^2 * mean(g * h)) (+ dres_in)
//   dw[c] (+)= sum_rows dy[r, c] * h[r, c] * inv_rms[r]
// dy, h, dres_in (optional), dx: bf16 [rows, H]; w: bf16 or fp32 [H] (wf32 selects); inv_rms: fp32
// [rows]; dw: fp32 [H].  H must be a multiple of 8 and at most ARENO_RMSNORM_BWD_STATIC_MAX_H;
// a larger H is refused with ARENO_NOALLOC_ERR_H_TOO_LARGE before anything is launched.
//
// What the caller must know:
//   * Set-up happens inside the first call on each device: with that device current, the call
//     looks up the device address of the scratch array once and keeps it.  Make that first call
//     during start-up, outside any stream capture; later calls only launch kernels.  A call
//     with rows = 0 does the set-up and launches nothing, which makes a cheap start-up call.
//   * `stream` must belong to the device that is current when the call is made.
//   * Every call on a device uses the same scratch and leaves its partial sums there.  Nothing in
//     it has to be zero beforehand: a call overwrites every element it later reads.  Two calls
//     that may run at the same time on one device (different streams, or different host threads
//     without ordering) would write the same rows and corrupt each other's dw; order them.
//   * The partial sums are folded over at most 148 rows of the scratch, against up to 296 in
//     areno_rmsnorm_bwd, so dw can differ from that entry point in the last fp32 bits; dx is
//     bit-identical.
int areno_rmsnorm_bwd_static(const void* dy, const void* h, const void* w, int wf32, float w_offset,
                             const float* inv_rms, const void* dres_in, void* dx, float* dw, int dw_accumulate,
                             long long rows, int H, cudaStream_t stream);

// Static, human-readable text for a return value of the function above (never NULL, never freed).
const char* areno_no_alloc_strerror(int code);

}  // extern "C"
