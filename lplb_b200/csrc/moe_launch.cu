// Launchers of the benchmark MoE layer kernels and the TMA descriptor builder.
#include "moe_api.h"

#include <cudaTypedefs.h>

#include "moe_support.cuh"
#include "planner_api.h"

namespace lplb {
namespace moe {

size_t gemm_smem_bytes() { return kGemmSmem; }

namespace {

// The driver entry point is fetched at run time so that the library has no link-time
// dependency on libcuda (it is imported on GPU-less build hosts too).
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

bool shape_ok(const LayerShape& sh) {
  return sh.n_ranks >= 1 && sh.n_ranks <= kMaxRanks && sh.my_rank >= 0 && sh.my_rank < sh.n_ranks &&
         sh.n_local >= 1 && sh.n_local <= kMaxLocalExperts && sh.hidden % kBN == 0 && sh.hidden % kBK == 0 &&
         (2 * sh.inter) % kBN == 0 && sh.inter % kBK == 0 && sh.topk >= 1 && sh.topk <= kCombineMaxTopk &&
         (long long)sh.max_tokens * sh.topk < (1 << 20) && sh.capacity > 0 && sh.capacity < (1 << 24);
}

}  // namespace

int make_tensor_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  auto fn = encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols * 2) % 16 || box_rows == 0 || box_rows > 256) return -2;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                         elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : (int)rc;
}

cudaError_t launch_plan(const LayerShape& sh, const LayerBuffers& b, int n_cta, uint32_t epoch,
                        unsigned long long timeout_ns, int fused, cudaStream_t stream) {
  if (!shape_ok(sh) || n_cta < 1) return cudaErrorInvalidValue;
  const int P = sh.n_ranks * sh.n_local;
  PlanArgs a{};
  for (int r = 0; r < sh.n_ranks; ++r) a.cnt_words[r] = b.cnt_words[r];
  a.local_counts = b.by_cta + (size_t)(n_cta - 1) * P;  // last prefix row = totals
  a.plan = b.plan;
  a.status = b.status;
  a.n_ranks = sh.n_ranks;
  a.my_rank = sh.my_rank;
  a.n_local = sh.n_local;
  a.capacity = sh.capacity;
  a.fused = fused;
  a.epoch = epoch;
  a.timeout_ns = timeout_ns;
  plan_kernel<<<1, kSupportThreads, sizeof(int) * 2 * P, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_dispatch(const LayerShape& sh, const LayerBuffers& b, const void* x, const void* phys_idx,
                            int idx_is64, int n_tokens, int n_cta, uint32_t epoch, cudaStream_t stream) {
  if (!shape_ok(sh) || n_cta < 1 || n_tokens < 0 || n_tokens > sh.max_tokens) return cudaErrorInvalidValue;
  const int P = sh.n_ranks * sh.n_local;
  DispatchArgs a{};
  for (int r = 0; r < sh.n_ranks; ++r) {
    a.recv_x[r] = static_cast<__nv_bfloat16*>(b.recv_x[r]);
    a.recv_meta[r] = b.recv_meta[r];
    a.flags[r] = b.flags[r];
  }
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.idx = phys_idx;
  a.dst_row_start = b.plan + 2 * sh.n_local;
  a.by_cta = b.by_cta;
  a.pair_slot = b.pair_slot;
  a.status = b.status;
  a.ticket = b.tickets + 0;
  a.n_pairs = (long long)n_tokens * sh.topk;
  a.idx_is64 = idx_is64;
  a.topk = sh.topk;
  a.hidden = sh.hidden;
  a.n_local = sh.n_local;
  a.n_ranks = sh.n_ranks;
  a.my_rank = sh.my_rank;
  a.capacity = sh.capacity;
  a.epoch = epoch;
  const size_t smem = sizeof(int) * (3 * (size_t)P + kDispatchChunk);
  dispatch_kernel<<<n_cta, kSupportThreads, smem, stream>>>(a);
  return cudaGetLastError();
}

namespace {
int* plan_tail(const LayerShape& sh, const LayerBuffers& b) {
  const int P = sh.n_ranks * sh.n_local;
  return b.plan + 2 * sh.n_local + P + sh.n_ranks * P;
}
}  // namespace

cudaError_t launch_schedule(const LayerShape& sh, const LayerBuffers& b, const void* phys_idx, int idx_is64,
                            int n_tokens, int n_cta, cudaStream_t stream) {
  if (!shape_ok(sh) || n_cta < 1 || n_tokens < 0 || n_tokens > sh.max_tokens) return cudaErrorInvalidValue;
  const int P = sh.n_ranks * sh.n_local;
  int* tail = plan_tail(sh, b);
  ScheduleArgs a{};
  a.idx = phys_idx;
  a.by_cta = b.by_cta;
  a.dst_row_start = b.plan + 2 * sh.n_local;
  a.order_base = tail + 8;
  a.send_base = tail + 8 + P;
  a.pair_slot = b.pair_slot;
  a.send_pair = b.send_pair;
  a.send_target = b.send_target;
  a.status = b.status;
  a.n_pairs = (long long)n_tokens * sh.topk;
  a.idx_is64 = idx_is64;
  a.n_local = sh.n_local;
  a.n_ranks = sh.n_ranks;
  a.capacity = sh.capacity;
  schedule_kernel<<<n_cta, kSupportThreads, sizeof(int) * P, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_dispatch_gemm(const LayerShape& sh, const LayerBuffers& b, const CUtensorMap& tmap_a,
                                 const CUtensorMap& tmap_b, const void* x, uint32_t epoch,
                                 unsigned long long timeout_ns, int n_cta, int send_ctas, cudaStream_t stream) {
  if (!shape_ok(sh) || n_cta < 1 || send_ctas < 0 || send_ctas >= n_cta) return cudaErrorInvalidValue;
  const int P = sh.n_ranks * sh.n_local;
  int* tail = plan_tail(sh, b);
  GemmArgs a{};
  a.send_ctas = send_ctas;
  a.rows = b.plan;
  a.row_start = b.plan + sh.n_local;
  a.n_experts = sh.n_local;
  a.n_ranks = sh.n_ranks;
  a.my_rank = sh.my_rank;
  a.epoch = epoch;
  a.status = b.status;
  a.timeout_ns = timeout_ns;
  a.n_tiles_n = 2 * sh.inter / kBN;
  a.k_blocks = sh.hidden / kBK;
  a.n_per_expert = 2 * sh.inter;
  a.act = static_cast<__nv_bfloat16*>(b.act);
  a.act_ld = sh.inter;
  a.wait_flags = nullptr;
  a.ticket = b.tickets + 1;
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.send_pair = b.send_pair;
  a.send_target = b.send_target;
  a.pair_slot = b.pair_slot;
  a.n_send = tail + 2;
  a.arrive_target = tail + 8 + 2 * P;
  for (int r = 0; r < sh.n_ranks; ++r) {
    a.recv_x[r] = static_cast<__nv_bfloat16*>(b.recv_x[r]);
    a.recv_meta[r] = b.recv_meta[r];
    a.arrived[r] = b.arrived[r];
  }
  a.topk = sh.topk;
  a.hidden = sh.hidden;
  a.debug = b.debug;
  auto kernel = grouped_gemm_kernel<kSwiGLU, true>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem);
  if (err != cudaSuccess) return err;
  kernel<<<n_cta, kFusedThreads, kGemmSmem, stream>>>(tmap_a, tmap_b, a);
  return cudaGetLastError();
}

cudaError_t launch_gemm(const LayerShape& sh, const LayerBuffers& b, const CUtensorMap& tmap_a,
                        const CUtensorMap& tmap_b, int which, uint32_t epoch, unsigned long long timeout_ns,
                        int n_cta, cudaStream_t stream) {
  if (!shape_ok(sh) || n_cta < 1 || (which != 0 && which != 1)) return cudaErrorInvalidValue;
  GemmArgs a{};
  a.rows = b.plan;
  a.row_start = b.plan + sh.n_local;
  a.n_experts = sh.n_local;
  a.n_ranks = sh.n_ranks;
  a.my_rank = sh.my_rank;
  a.epoch = epoch;
  a.status = b.status;
  a.timeout_ns = timeout_ns;
  cudaError_t err;
  if (which == 0) {
    a.n_tiles_n = 2 * sh.inter / kBN;
    a.k_blocks = sh.hidden / kBK;
    a.n_per_expert = 2 * sh.inter;
    a.act = static_cast<__nv_bfloat16*>(b.act);
    a.act_ld = sh.inter;
    a.wait_flags = b.flags[sh.my_rank];  // dispatch done, one word per source rank
    a.ticket = b.tickets + 1;
    auto kernel = grouped_gemm_kernel<kSwiGLU, false>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem);
    if (err != cudaSuccess) return err;
    kernel<<<n_cta, kGemmThreads, kGemmSmem, stream>>>(tmap_a, tmap_b, a);
  } else {
    a.n_tiles_n = sh.hidden / kBN;
    a.k_blocks = sh.inter / kBK;
    a.n_per_expert = sh.hidden;
    a.meta = b.recv_meta[sh.my_rank];
    for (int r = 0; r < sh.n_ranks; ++r) {
      a.comb[r] = static_cast<__nv_bfloat16*>(b.comb[r]);
      a.done_flags[r] = b.flags[r] + sh.n_ranks;  // combine done
    }
    a.out_ld = sh.hidden;
    a.wait_flags = nullptr;
    a.ticket = b.tickets + 2;
    auto kernel = grouped_gemm_kernel<kScatter, false>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem);
    if (err != cudaSuccess) return err;
    kernel<<<n_cta, kGemmThreads, kGemmSmem, stream>>>(tmap_a, tmap_b, a);
  }
  return cudaGetLastError();
}

cudaError_t launch_combine(const LayerShape& sh, const LayerBuffers& b, const float* weights, void* out, int n_tokens,
                           uint32_t epoch, unsigned long long timeout_ns, int n_cta, cudaStream_t stream) {
  if (!shape_ok(sh) || n_tokens < 0 || n_tokens > sh.max_tokens || n_cta < 1) return cudaErrorInvalidValue;
  CombineArgs a{};
  a.comb = static_cast<const __nv_bfloat16*>(b.comb[sh.my_rank]);
  a.weights = weights;
  a.pair_slot = b.pair_slot;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.wait_flags = b.flags[sh.my_rank] + sh.n_ranks;
  a.status = b.status;
  a.n_tokens = n_tokens;
  a.topk = sh.topk;
  a.hidden = sh.hidden;
  a.n_ranks = sh.n_ranks;
  a.epoch = epoch;
  a.timeout_ns = timeout_ns;
  combine_kernel<<<n_cta, kSupportThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace moe
}  // namespace lplb
