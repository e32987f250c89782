// Entry point for callers that must not allocate device memory.  It has no counterpart in the
// reference (the reference has no native code at all); it exists for embedders of this library.
// This header is C++ (it includes common.cuh, which needs cuda_runtime.h); the exported symbol itself has C linkage and
// can be bound from any language through the shared library.
#pragma once
#include "common.cuh"

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of CTAs (= partial sums) the built-in scratch array holds.
#define MGW_STATIC_MAX_PARTIALS 1024

// Global L2 norm of all gradients of `group` and the matching clip coefficient, like
// mgw_group_sumsq() followed by mgw_clip_coef(), but without a caller-provided `partials` buffer:
// the per-CTA partial sums go to a fixed array that lives inside the library image.
//
//   out2[0] = sqrt(sum of squares),  out2[1] = min(1, max_norm / (out2[0] + 1e-6))     (device memory)
//
// Who needs this: code that is not allowed to call cudaMalloc (or any allocating routine) at the point
// where it wants the norm -- a host application that gave this library a fixed amount of memory and owns
// every other byte of the device, or a latency-critical section in which an allocation could stall
// the device.  The call itself allocates nothing, frees nothing and calls no library that might.
//
// Rules
//  * n_ctas must be in [1, MGW_STATIC_MAX_PARTIALS]; larger values are rejected with MGW_ERR_TOO_LARGE
//    and an explanatory mgw_last_error() text (the existing entry points accept any size because the
//    caller sizes their buffer).
//  * The scratch array (4 KB) is part of the library image: every GPU that loads the library keeps its own
//    copy until the process exits.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current).  Make that first call outside of any stream capture.
//  * All calls on one device share the array.  Nothing in it has to start at zero -- each launch overwrites
//    exactly the n_ctas slots it then reads -- but two calls whose kernels overlap on the GPU (different
//    streams, no ordering between them) race on it.  Keep calls on one stream or order them with events.
int mgw_grad_clip_coef_static(const MgwGroup* group, float max_norm, float* out2, int n_ctas, void* stream);

#ifdef __cplusplus
}
#endif
