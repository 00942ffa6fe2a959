// Gradient-norm / clip-coefficient entry point that performs no memory allocation of any kind.
//
// This entry point has no counterpart in the reference framework; it exists for hosts of this library that must not
// allocate while they compute the norm:
//   * a plain C or C++ program that links this library without torch (the streaming server runtime, a C test driver).
//     It has no caching allocator, and a raw cudaMalloc / cudaFree pair around every step synchronises the whole device;
//   * a training job running close to the HBM limit, where an allocation inside the optimizer step can fail after the
//     gradients have already been reduced, which loses the step.
// sb_grad_norm_clip (elementwise.cu) takes its block-partials buffer from the caller; this variant keeps the partials in
// a fixed array in the library's own device data segment instead.
//
// Contract
//   * Scratch: one file-scope device array of SB_GRAD_NORM_STATIC_MAX_PARTS floats (8 KB) per device, shared by every
//     call on that device.  `nparts` is the number of block partial sums (= thread blocks of the first kernel); 0 selects
//     the default of 8 per SM.  nparts > SB_GRAD_NORM_STATIC_MAX_PARTS is rejected with SB_GRAD_NORM_STATIC_E_TOO_LARGE
//     and a message on stderr; nothing is launched.
//   * Nothing in the scratch array has to start at zero: every block overwrites its own slot and the finishing kernel
//     reads exactly the first `nparts` slots.  `scalars` belongs to the caller: [0] = norm and [1] = coefficient are
//     overwritten, [2] is a sticky non-finite flag that is only ever set to 1, so the caller clears it when it wants a
//     fresh reading (same convention as sb_grad_norm_clip).
//   * Two calls that overlap in time on one device (different streams, or different host threads on different streams)
//     race on the scratch array and give undefined norms.  Calls issued to one stream are ordered and safe.
//   * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that device current)
//     and caches it.  That set-up can load the module and is not stream-ordered work: make the first call on a device
//     before any stream capture is begun on it.  Later calls only launch the two kernels.
//   * No cudaMalloc / cudaFree / cudaMallocAsync, no torch or other allocating library routine is called, on any path.
#pragma once
#include "common.cuh"

#define SB_GRAD_NORM_STATIC_MAX_PARTS 2048
#define SB_GRAD_NORM_STATIC_E_TOO_LARGE (-2)
#define SB_GRAD_NORM_STATIC_E_BAD_ARG (-1)

// g: fp32 gradients [n] on the current device; scalars: 3 device floats (norm, clip coefficient, non-finite flag).
// Returns 0, one of the negative codes above, or a positive cudaError_t (set-up or launch failure).
SB_API int sb_grad_norm_clip_static(const float* g, long long n, float* scalars, float max_norm, float grad_scale, int nparts,
                                    cudaStream_t stream);

// The compiled-in capacity (SB_GRAD_NORM_STATIC_MAX_PARTS), for callers that bind by symbol only.
SB_API int sb_grad_norm_static_max_parts();
