// Shared device/host helpers for the planner kernels (sm_100a).
//
// Everything that can wait on another CTA or another GPU goes through
// `bounded_wait_ge`, which gives up after a time budget and reports through the
// status block instead of spinning forever (the reference spins without a limit,
// reference lplb/resources/csrc-tmpl/minilp.cu:132 and :150-152).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lplb {

// ---- status block -----------------------------------------------------------------
// One int32[kStatusWords] array per engine, written by kernels, read lazily by the host.
enum StatusWord : int {
  kStErr = 0,        // first error code seen (0 = none), sticky until the host clears it
  kStPhase = 1,      // phase that raised it
  kStDetail = 2,     // e.g. bit mask of peers that never arrived, or the offending index
  kStCalls = 3,      // number of planner launches that finished
  kStLpIters = 4,    // iterations used by the slowest group in the last launch
  kStLpFail = 5,     // groups that did not converge, cumulative
  kStTimeouts = 6,   // waits that ran out, cumulative
  kStBadIdx = 7,     // out-of-range expert indices seen, cumulative
  kStGapPpb = 8,     // largest relative duality gap among the groups of the last launch, in 1e-9 units
  kStBoundsIndex = 9,   // bounds-checking build: the first index that was out of range ...
  kStBoundsLimit = 10,  // ... the size it was checked against (kStDetail holds the source line) ...
  kStBoundsCount = 11,  // ... and how many accesses were skipped, cumulative
  kStatusWords = 16
};

enum ErrCode : int {
  kOk = 0,
  kErrGridTimeout = 1,   // a CTA of the same launch never arrived
  kErrPeerTimeout = 2,   // a peer GPU never published its counts
  kErrLpTimeout = 3,     // the solving CTA never released the result
  kErrBadIndex = 4,      // expert index outside [-1, E)
  kErrLpNotConverged = 5,
  kErrBounds = 6         // bounds-checking build only: an index left its array; the access was skipped
};

enum Phase : int { kPhCount = 1, kPhExchange = 2, kPhSolve = 3, kPhRedirect = 4 };

__device__ __forceinline__ void raise_status(int* status, int code, int phase, int detail) {
  if (atomicCAS(&status[kStErr], 0, code) == 0) {
    status[kStPhase] = phase;
    status[kStDetail] = detail;
  }
}

// ---- bounds-checking build -----------------------------------------------------------
// With -DLPLB_BOUNDS_CHECK every data-dependent shared- or global-memory index of the planner
// and MoE support kernels goes through LPLB_CHECKED: an index outside [0, n) is recorded in the
// status block (first one: code, phase, source line, index, limit) and the access is skipped;
// nothing traps.  This stands in for a memory checker on machines where none can be run; the
// reference's only guard is a device assert on the expert index
// (reference lplb/resources/csrc-tmpl/minilp.cu:429-430).  Without the macro the check
// compiles to `true`.
#ifdef LPLB_BOUNDS_CHECK
__device__ __forceinline__ bool index_in_range(long long i, long long n, int* status, int phase, int line) {
  if (i >= 0 && i < n) return true;
  if (status != nullptr) {
    if (atomicCAS(&status[kStErr], 0, kErrBounds) == 0) {
      status[kStPhase] = phase;
      status[kStDetail] = line;
      status[kStBoundsIndex] = (int)i;
      status[kStBoundsLimit] = (int)n;
    }
    atomicAdd(&status[kStBoundsCount], 1);
  }
  return false;
}
#define LPLB_CHECKED(i, n, status, phase) ::lplb::index_in_range((long long)(i), (long long)(n), (status), (phase), __LINE__)
#else
#define LPLB_CHECKED(i, n, status, phase) true
#endif

// ---- memory-order helpers ------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait until *flag has reached `target` (wrap-safe compare).  Returns false when
// `budget_ns` ran out first.  SYS selects system scope (flags written by a peer GPU).
template <bool SYS>
__device__ __forceinline__ bool bounded_wait_ge(const uint32_t* flag, uint32_t target, uint64_t budget_ns) {
  uint32_t v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
  if ((int32_t)(v - target) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t backoff = 20;
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
      if ((int32_t)(v - target) >= 0) return true;
      __nanosleep(backoff);
    }
    if (backoff < 160) backoff <<= 1;
    if (global_timer_ns() - t0 > budget_ns) return false;
  }
}

// ---- token slicing --------------------------------------------------------------------
// CTA `p` of `n_cta` handles tokens [slice_begin(p), slice_begin(p+1)).  Slices are
// multiples of `align` so vector loads stay aligned.  The counting and redirect kernels
// must agree on this function (the reference has the same coupling,
// reference lplb/resources/csrc-tmpl/minilp.cu:404-408).
__host__ __device__ __forceinline__ long long slice_begin(long long n, int p, int n_cta, int align) {
  long long per = (n + n_cta - 1) / n_cta;
  per = (per + align - 1) / align * align;
  long long b = per * (long long)p;
  return b < n ? b : n;
}

}  // namespace lplb
