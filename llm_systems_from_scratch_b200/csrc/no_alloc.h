// Entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference project; it exists for users of this library whose
// calling context forbids cudaMalloc: a plug-in running inside another framework's memory plan, a
// real-time loop that may not touch the allocator, or a host that has already handed all device memory
// to a pool it does not control.  The ordinary RMSNorm backward (b200_rmsnorm_bwd) needs a scratch
// buffer for per-block weight-gradient partials that its caller allocates.  The variant below keeps
// that scratch in a fixed array inside the library image instead, so the caller passes inputs and
// outputs only.
//
// Limits and rules
//   * d must be a multiple of 8 and at most B200_NOALLOC_MAX_D; larger widths are refused with
//     B200_ERR_NOALLOC_TOO_LARGE (nothing is launched).  rows is unlimited.
//   * The array (B200_NOALLOC_MAX_PARTS x B200_NOALLOC_MAX_D floats, about 4.6 MiB) is part of the
//     library: every GPU that loads the library holds it until the process exits.
//   * The first call on each device looks up the array's device address (with that device current)
//     and caches it.  Make that first call before starting any stream capture on the device.
//   * All calls share the one array.  Its old contents never matter (every partial that is read
//     has been written by the same call), but two calls that run at the same time on one GPU, for
//     example on different streams, race on it.  Serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called on any path.
#pragma once
#include <cuda_runtime.h>

#define B200_NOALLOC_MAX_D 8192
#define B200_NOALLOC_MAX_PARTS 148
#define B200_ERR_NOALLOC_TOO_LARGE (-12)
#define B200_ERR_NOALLOC_SETUP (-13)

#ifdef __cplusplus
extern "C" {
#endif

// dx = [dres +] d(RMSNorm)/dx ; dw (=|+=) d(RMSNorm)/dw.  All pointers are device pointers:
// dy, x, dres (may be null), dx: bf16 (rows, d);  w: bf16 (d);  rstd: fp32 (rows);  dw: fp32 (d).
// With rows == 0 the call still defines dw (zero, or unchanged when accumulating).
// Returns 0 on success, -10 for null / misaligned / unsupported arguments, B200_ERR_NOALLOC_TOO_LARGE when
// d exceeds B200_NOALLOC_MAX_D, B200_ERR_NOALLOC_SETUP when the scratch address cannot be resolved.
int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                             void* dx, float* dw, int rows, int d, int accumulate_dw, cudaStream_t stream);

// The largest width the entry point above accepts.
int b200_rmsnorm_bwd_noalloc_max_d(void);

#ifdef __cplusplus
}
#endif
