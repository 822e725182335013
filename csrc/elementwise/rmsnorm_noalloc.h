// RMSNorm backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for hosts of this library that
// must not call cudaMalloc (or anything that may call it) on their hot path: code running inside a region that
// is being captured into a CUDA graph, real-time or serving loops that pre-plan all memory and forbid the
// implicit device synchronisation an allocation can cause, and embedders whose memory pool is owned by another
// runtime.  The ordinary entry point (`mt::rmsnorm_bwd` + `mt::rmsnorm_bwd_reduce`) needs a scratch matrix of
// per-block weight-gradient partial sums that its caller allocates; here that scratch is a fixed array inside
// the library's device image.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch: 64 partial rows of at most 8192 floats (2 MiB, resident on every GPU that loads
// the library until the process exits).
#define MT_RMSNORM_NOALLOC_MAX_DIM 8192
#define MT_RMSNORM_NOALLOC_PARTIALS 64

// dx = d(rmsnorm)/dx applied to dy (+ dres if non-null), dw (+)= sum over rows of dy * xhat.
//   x, dy, dres, dx : bf16 [rows, dim] contiguous;  w, dw : fp32 [dim];  rstd : fp32 [rows] from the forward.
// With rows == 0 the sum is empty: dw is set to zero (left unchanged when accumulate_dw is non-zero), dx is untouched.
// Returns 0 on success.  On failure returns a non-zero code and, if `err` is non-null, writes a message of at
// most `err_len` bytes (dim > MT_RMSNORM_NOALLOC_MAX_DIM, dim not a multiple of 8, null pointers, CUDA errors).
//
// No device memory is allocated or freed, by this call or by anything it calls.  The first call on a given
// device looks up the scratch array's device address (cudaGetSymbolAddress) and caches it; make that first call
// outside any stream capture.  All calls on a device share the one scratch array: two calls whose kernels may
// overlap on the GPU (different streams without an ordering between them) race on it and must be serialised by
// the caller.  Every partial row is rewritten in full by each call, so nothing carries over between calls.
// The scratch is looked up for the device that is current when the call is made, so `stream` must belong to that
// device (make the device current first; a stream of another device would run the kernels with the wrong array).
// Calls from several host threads are safe with respect to the address cache (an atomic slot per device, every
// writer storing the same value); the scratch itself is still shared, so the rule about overlapping kernels holds
// across threads too.
int mt_rmsnorm_bwd_noalloc(const void* x, const float* w, const float* rstd, const void* dy, const void* dres,
                           void* dx, float* dw, int64_t rows, int dim, int accumulate_dw, cudaStream_t stream,
                           char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
