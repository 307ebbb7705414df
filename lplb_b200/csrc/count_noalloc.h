// Token histogram for callers that must not allocate.
//
// This entry point has no counterpart in the reference: there, every call of the counting
// stage allocates its result through the framework's allocator
// (reference csrc/plugin.cpp:586-587).
//
// Who needs it.  Two kinds of callers cannot let a library call cudaMalloc (or a caching
// allocator that may fall through to it) on their behalf:
//   * a serving process that hands all of the device's free memory to its own pool at
//     start-up: any later allocation by a library simply fails;
//   * a latency-critical step loop: cudaMalloc and cudaFree synchronise the whole device,
//     so one hidden allocation stalls every stream the process is running.
// For them the histogram's scratch (one row of counts per CTA plus a ticket) lives in a
// fixed array inside the library image instead of in allocated memory.
//
// Limits (the array is sized for them and every GPU that loads the library holds it
// until the process exits): at most LPLB_NOALLOC_MAX_CTAS CTAs and
// LPLB_NOALLOC_MAX_EXPERTS logical experts, 655,616 bytes in total.  Larger requests are
// refused with an error, nothing is launched.
//
// Contract.
//   * `idx` (device, int64 or int32, n_tokens entries in [-1, n_logical); other values are
//     skipped) and `counts_out` (device, int32[n_logical]) belong to the caller.  The call
//     allocates and frees nothing, on the host or on the device.
//   * The current device must be the one that owns the pointers.  The first call on a
//     device looks up the array's device address once (cudaGetSymbolAddress); make that
//     first call before any stream capture begins on that device.
//   * That first call is also a warm-up in a second sense: CUDA loads a library's device
//     image on first use, and loading is what places the array and the kernel's code in
//     device memory.  A process that gives all remaining device memory to its own pool must
//     therefore make one call per device *before* it takes that memory; every later call
//     leaves the amount of free device memory unchanged.
//   * All calls on a device share the one array.  Each call re-zeroes the part that has to
//     start at zero, so leftovers of earlier calls are harmless, but two calls that overlap
//     on the GPU (different streams, no ordering between them) race on it: order them.
//   * The work is enqueued on `stream` (a cudaStream_t passed as void*; null is the
//     default stream).  Nothing is synchronised.
//   * Returns 0 on success.  A negative value is a refused argument, a positive value is
//     the cudaError_t of a failed runtime call.  When `err` is non-null a message of at most
//     `err_len` bytes (terminated) is written on failure.
#pragma once

#include <stddef.h>

#define LPLB_NOALLOC_MAX_CTAS 160
#define LPLB_NOALLOC_MAX_EXPERTS 1024

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int lplb_count_tokens_noalloc(const void* idx, int idx_is64,
                                                                     long long n_tokens, int n_logical, int n_cta,
                                                                     int* counts_out, void* stream, char* err,
                                                                     size_t err_len);

#ifdef __cplusplus
}
#endif
