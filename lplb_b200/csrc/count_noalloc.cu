// Allocation-free token histogram: see count_noalloc.h for who needs it and the contract.
#include "count_noalloc.h"

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kHeaderBytes = 256;  // ticket, padded so that the rows stay 256-byte aligned
constexpr size_t kScratchBytes =
    kHeaderBytes + sizeof(int) * (size_t)LPLB_NOALLOC_MAX_CTAS * LPLB_NOALLOC_MAX_EXPERTS;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a stand-in for the symbol, never a
// device address: the address is fetched once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

// Same scheme as count_kernel in planner_kernels.cuh, with the per-CTA rows in the fixed
// scratch instead of in an output tensor: every CTA counts its slice into shared memory and
// parks the row; the CTA that takes the last ticket adds the rows up into `counts_out`.
template <typename IdxT>
__global__ void __launch_bounds__(kThreads) count_noalloc_kernel(const IdxT* __restrict__ idx, long long n, int e,
                                                                 unsigned char* scratch, int* __restrict__ counts_out) {
  extern __shared__ int hist[];
  __shared__ bool last;
  unsigned* ticket = reinterpret_cast<unsigned*>(scratch);
  int* rows = reinterpret_cast<int*>(scratch + kHeaderBytes);
  const int p = blockIdx.x, n_cta = gridDim.x;
  for (int i = threadIdx.x; i < e; i += kThreads) hist[i] = 0;
  __syncthreads();
  const long long begin = lplb::slice_begin(n, p, n_cta, kThreads), end = lplb::slice_begin(n, p + 1, n_cta, kThreads);
  for (long long i = begin + threadIdx.x; i < end; i += kThreads) {
    const long long v = (long long)idx[i];
    if (v >= 0 && v < e) atomicAdd(&hist[v], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < e; i += kThreads) rows[(size_t)p * e + i] = hist[i];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1u) == (unsigned)n_cta - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  for (int i = threadIdx.x; i < e; i += kThreads) {
    int total = 0;
    for (int r = 0; r < n_cta; ++r) total += __ldcg(&rows[(size_t)r * e + i]);
    counts_out[i] = total;
  }
}

std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {};  // device address of g_scratch, per device ordinal

int fail(int code, char* err, size_t err_len, const char* what, const char* detail) {
  if (err && err_len) snprintf(err, err_len, "lplb_count_tokens_noalloc: %s%s%s", what, detail ? ": " : "", detail ? detail : "");
  return code;
}

}  // namespace

extern "C" int lplb_count_tokens_noalloc(const void* idx, int idx_is64, long long n_tokens, int n_logical, int n_cta,
                                         int* counts_out, void* stream, char* err, size_t err_len) {
  if (!counts_out || (!idx && n_tokens > 0)) return fail(-1, err, err_len, "null pointer argument", nullptr);
  if (n_tokens < 0) return fail(-2, err, err_len, "negative token count", nullptr);
  if (n_logical < 1 || n_logical > LPLB_NOALLOC_MAX_EXPERTS)
    return fail(-3, err, err_len, "n_logical outside 1..1024 (LPLB_NOALLOC_MAX_EXPERTS): the fixed scratch cannot hold it", nullptr);
  if (n_cta < 1 || n_cta > LPLB_NOALLOC_MAX_CTAS)
    return fail(-4, err, err_len, "n_cta outside 1..160 (LPLB_NOALLOC_MAX_CTAS): the fixed scratch cannot hold it", nullptr);

  int dev = -1;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return fail((int)rc, err, err_len, "cudaGetDevice failed", cudaGetErrorString(rc));
  if (dev < 0 || dev >= kMaxDevices) return fail(-5, err, err_len, "device ordinal above 63", nullptr);

  unsigned char* scratch = nullptr;
  {
    // Set-up, once per device, with that device current: the array's address on this device.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
      void* addr = nullptr;
      rc = cudaGetSymbolAddress(&addr, g_scratch);
      if (rc != cudaSuccess) return fail((int)rc, err, err_len, "cudaGetSymbolAddress failed", cudaGetErrorString(rc));
      g_scratch_addr[dev] = static_cast<unsigned char*>(addr);
    }
    scratch = g_scratch_addr[dev];
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The ticket has to start at zero whatever an earlier (possibly failed) call left behind.
  // The rows need no clearing: every CTA overwrites its whole row before the ticket is taken.
  rc = cudaMemsetAsync(scratch, 0, kHeaderBytes, s);
  if (rc != cudaSuccess) return fail((int)rc, err, err_len, "cudaMemsetAsync failed", cudaGetErrorString(rc));
  const size_t smem = sizeof(int) * (size_t)n_logical;
  // cudaLaunchKernel returns the outcome of this launch itself, so an earlier, unrelated error
  // that the calling thread has not collected yet is neither reported as ours nor cleared.
  void* args[] = {const_cast<void**>(&idx), &n_tokens, &n_logical, &scratch, &counts_out};
  const void* kernel = idx_is64 ? reinterpret_cast<const void*>(&count_noalloc_kernel<int64_t>)
                                : reinterpret_cast<const void*>(&count_noalloc_kernel<int32_t>);
  rc = cudaLaunchKernel(kernel, dim3(n_cta), dim3(kThreads), args, smem, s);
  if (rc != cudaSuccess) return fail((int)rc, err, err_len, "kernel launch failed", cudaGetErrorString(rc));
  return 0;
}
