// RMSNorm backward that performs no memory allocation of any kind.
//
// This entry point has no counterpart in the reference project; it exists for callers that must
// not allocate while they run: native (C / C++ / ctypes) code that reaches this symbol directly
// and has no business inside torch's caching allocator; a callback that runs while some other
// component holds the allocator's lock; and a latency-critical loop that cannot afford the
// implicit device synchronisation that cudaMalloc / cudaFree bring. The symbol is exported from
// the framework's extension library (`halite_b200/_C.so`), which itself links against torch: the
// process must be able to load torch's libraries, but this function never calls into them. The regular entry point
// (`rmsnorm_bwd` of the Python extension) asks torch for its outputs and for a scratch tensor
// on every call; this one gets inputs and outputs from the caller and keeps its scratch in a
// fixed array inside the library's device image.
//
// Semantics (identical to the regular entry point):
//   g    = dy * (w + w_offset),  xhat = h * rstd[row]
//   dx   = rstd * (g - xhat * mean(g * xhat)) (+ dres when dres != NULL)        bf16 [rows, dim]
//   dw   = sum over rows of dy * xhat                                           fp32 [dim]
//
// Limits: dim is a multiple of 8 and at most HB_RMSNORM_BWD_FIXED_MAX_DIM (8192). The scratch
// is HB_RMSNORM_BWD_FIXED_SLICES (64) x HB_RMSNORM_BWD_FIXED_MAX_DIM floats = 2 MiB per device,
// whatever the call's size. `rows` is between 0 and 2^31 - 1 (the kernels index rows with 32-bit
// integers); rows == 0 only clears dw. A size outside these limits is rejected with
// HB_FIXED_ERR_SIZE and a message on stderr; nothing is launched.
//
// Set-up: the first call on each device looks up the scratch array's device address (one
// `cudaGetSymbolAddress` with that device current) and caches it. That first call therefore
// does more than launch kernels: make it before any stream capture begins on that device.
//
// Sharing: every call on a device uses the same array. Nothing in it has to start at zero: each
// call overwrites every word it later reads. Two calls that overlap in time on one device
// (different streams, or different host threads without stream ordering between them) race on
// the array and produce wrong dw; serialise them on one stream or with events.
//
// Returns 0 on success, a positive cudaError_t value when a CUDA call failed, or one of the
// negative codes below.
#pragma once

#include <stdint.h>

#define HB_RMSNORM_BWD_FIXED_MAX_DIM 8192
#define HB_RMSNORM_BWD_FIXED_SLICES 64

#define HB_FIXED_ERR_SIZE (-1)      // dim <= 0, not a multiple of 8 or > max; rows < 0 or > 2^31 - 1
#define HB_FIXED_ERR_POINTER (-2)   // a required pointer is NULL or not 16-byte aligned

#ifdef __cplusplus
extern "C" {
#endif

// dy, h, dres (optional, may be NULL), dx: bf16 [rows, dim] contiguous; w: bf16 [dim];
// rstd: fp32 [rows]; dw: fp32 [dim]. All device pointers on the current device. `stream` is a
// cudaStream_t passed as an integer-sized handle (0 = the default stream).
int hb_rmsnorm_bwd_fixed_scratch(const void* dy, const void* h, const void* w, const float* rstd,
                                 const void* dres, void* dx, float* dw, int64_t rows, int64_t dim,
                                 float w_offset, void* stream);

#ifdef __cplusplus
}
#endif
