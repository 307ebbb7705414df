// Launchers for the planner kernels: shape dispatch to the ahead-of-time instantiations.
#include "planner_api.h"
#include "planner_kernels.cuh"

namespace lplb {

namespace {

Topo make_topo(const TopoDesc& t) {
  Topo o;
  o.r2o = t.r2o;
  o.o2r = t.o2r;
  o.phy2log = t.phy2log;
  o.log2phy = t.log2phy;
  o.log2edge = t.log2edge;
  o.log2slot = t.log2slot;
  o.n_group = t.n_group;
  o.g = t.g;
  o.d = t.d;
  o.ll = t.ll;
  o.c = t.c;
  o.pl = t.ll + t.c * t.d;
  o.e = t.n_group * t.g * t.ll;
  return o;
}

int padded_group(int g) { return g <= 8 ? 8 : (g <= 16 ? 16 : 32); }
int padded_dup(int d) { return d <= 4 ? d : 8; }

// The counting and redirect kernels work for any topology; the solvers (and with them the
// fused kernel) cover groups of up to kMaxGroupSize ranks and kMaxDup replicas.
bool shape_ok(const TopoDesc& t, bool need_solver = true, int solver = kSolverAuto) {
  const bool tables = t.g >= 1 && t.d >= 1 && t.n_group >= 1 && t.ll >= t.c * t.d &&
                      (long long)t.n_group * t.g * t.ll <= kMaxLogicalExperts;
  return tables && (!need_solver || resolve_solver(t.g, t.d, solver) > 0);
}

// Calls fn.template operator()<GP, D>() for the instantiation that covers (g, d): GP = 8, 16,
// 32 for the warp solver, GP = 0 for the thread-block solver (D is then the padded count).
template <typename Fn>
cudaError_t dispatch_shape(int g, int d, int solver, Fn&& fn) {
  const int kind = resolve_solver(g, d, solver);
  if (kind == kSolverBlock) {
    const int dp = padded_dup(d);
#define LPLB_CASE(D_) \
  if (dp == D_) return fn.template operator()<0, D_>();
    LPLB_CASE(1) LPLB_CASE(2) LPLB_CASE(3) LPLB_CASE(4) LPLB_CASE(8)
#undef LPLB_CASE
    return cudaErrorInvalidValue;
  }
  if (kind != kSolverWarp) return cudaErrorInvalidValue;
  const int gp = padded_group(g);
#define LPLB_CASE(GP_, D_) \
  if (gp == GP_ && d == D_) return fn.template operator()<GP_, D_>();
  LPLB_CASE(8, 1) LPLB_CASE(8, 2) LPLB_CASE(8, 3) LPLB_CASE(8, 4)
  LPLB_CASE(16, 1) LPLB_CASE(16, 2) LPLB_CASE(16, 3) LPLB_CASE(16, 4)
  LPLB_CASE(32, 1) LPLB_CASE(32, 2) LPLB_CASE(32, 3) LPLB_CASE(32, 4)
#undef LPLB_CASE
  return cudaErrorInvalidValue;
}

size_t fused_smem(int e) { return sizeof(int) * 5 * (size_t)e; }
size_t bundle_smem(const Topo& tp) { return sizeof(int) * (size_t)tp.n_group * tp.g * (tp.d + 1); }
// bundle sums followed by the thread-block solver's scratch area
size_t block_smem(int n_ranks, int g, int d) { return bundle_bytes_aligned(n_ranks, d) + block_solver_smem_bytes(g, padded_dup(d)); }

template <typename K>
cudaError_t allow_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  if (bytes > 227 * 1024) return cudaErrorInvalidValue;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

IpmParams make_params(const SolveParams& prm) {
  return IpmParams{prm.max_iters, prm.tol, prm.anchor, prm.anchor_valid, prm.guard, prm.snap_mu};
}

}  // namespace

int resolve_solver(int g, int d, int requested) {
  const bool warp_ok = g >= 1 && d >= 1 && g <= kMaxWarpGroupSize && d <= kMaxWarpDup;
  const bool block_ok = g >= 1 && d >= 1 && g <= kMaxGroupSize && d <= kMaxDup && g <= kBlkMaxGroup;
  if (requested == kSolverWarp) return warp_ok ? kSolverWarp : -1;
  if (requested == kSolverBlock) return block_ok ? kSolverBlock : -1;
  if (warp_ok && g <= 8) return kSolverWarp;
  return block_ok ? kSolverBlock : -1;
}

int anchor_dup(int g, int d, int requested) { return resolve_solver(g, d, requested) == kSolverBlock ? padded_dup(d) : d; }

size_t planner_workspace_bytes(int n_logical) { return workspace_bytes(n_logical); }

cudaError_t launch_count(const void* idx, int idx_is64, long long n, int n_logical, int n_cta, int* by_cta,
                         void* workspace, int* status, cudaStream_t stream) {
  if (n_logical < 1 || n_logical > kMaxLogicalExperts || n_cta < 1) return cudaErrorInvalidValue;
  const size_t smem = sizeof(int) * (size_t)n_logical;
  auto* ws = static_cast<Workspace*>(workspace);
  if (idx_is64)
    count_kernel<int64_t><<<n_cta, kBlock, smem, stream>>>(static_cast<const int64_t*>(idx), n, n_logical, by_cta, ws,
                                                           status);
  else
    count_kernel<int32_t><<<n_cta, kBlock, smem, stream>>>(static_cast<const int32_t*>(idx), n, n_logical, by_cta, ws,
                                                           status);
  return cudaGetLastError();
}

struct SolveLaunch {
  const int* workload;
  Topo tp;
  IpmParams prm;
  float* probs;
  float* normalised;
  Counter avail;
  int* status;
  cudaStream_t stream;
  template <int GP, int D>
  cudaError_t operator()() const {
    if constexpr (GP == 0) {
      const size_t smem = block_smem(tp.n_group * tp.g, tp.g, tp.d);
      cudaError_t err = allow_smem(solve_block_kernel<D>, smem);
      if (err != cudaSuccess) return err;
      solve_block_kernel<D><<<tp.n_group, kBlock, smem, stream>>>(workload, tp, prm, probs, normalised, avail, status);
    } else {
      // As few solving warps per CTA as still fit the groups on one wave of CTAs.
      int dev = 0, sms = 1;
      cudaError_t err = cudaGetDevice(&dev);
      if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (err != cudaSuccess) return err;
      int warps = 1;
      while (warps < kWarps && (tp.n_group + warps * (32 / GP) - 1) / (warps * (32 / GP)) > sms) warps *= 2;
      const int per_cta = warps * (32 / GP);
      const int grid = (tp.n_group + per_cta - 1) / per_cta;
      const size_t smem = bundle_smem(tp);
      if ((err = allow_smem(solve_kernel<GP, D>, smem)) != cudaSuccess) return err;
      solve_kernel<GP, D><<<grid, kBlock, smem, stream>>>(workload, tp, prm, probs, normalised, avail, status, warps);
    }
    return cudaGetLastError();
  }
};

cudaError_t launch_solve(const int* workload, const TopoDesc& topo, SolveParams prm, float* probs, float* normalised,
                         void* avail, int avail_is64, int* status, cudaStream_t stream) {
  if (!shape_ok(topo, true, prm.solver)) return cudaErrorInvalidValue;
  SolveLaunch l{workload, make_topo(topo), make_params(prm), probs, normalised, Counter{avail, avail_is64}, status,
                stream};
  return dispatch_shape(topo.g, topo.d, prm.solver, l);
}

cudaError_t launch_redirect(const void* idx, int idx_is64, long long n, const float* probs, const int* by_cta,
                            const TopoDesc& topo, int n_cta, void* out, cudaStream_t stream) {
  if (!shape_ok(topo, false) || n_cta < 1) return cudaErrorInvalidValue;
  const Topo tp = make_topo(topo);
  const size_t smem = fused_smem(tp.e);
  cudaError_t err;
  if (idx_is64) {
    if ((err = allow_smem(redirect_kernel<int64_t>, smem)) != cudaSuccess) return err;
    redirect_kernel<int64_t><<<n_cta, kBlock, smem, stream>>>(static_cast<const int64_t*>(idx), n, probs, by_cta, tp,
                                                              static_cast<int64_t*>(out));
  } else {
    if ((err = allow_smem(redirect_kernel<int32_t>, smem)) != cudaSuccess) return err;
    redirect_kernel<int32_t><<<n_cta, kBlock, smem, stream>>>(static_cast<const int32_t*>(idx), n, probs, by_cta, tp,
                                                              static_cast<int32_t*>(out));
  }
  return cudaGetLastError();
}

cudaError_t launch_exchange(const int* in, int n_logical, const ExchangeDesc& exd, void* workspace, int* out,
                            int* status, cudaStream_t stream) {
  if (n_logical < 1 || n_logical > kMaxLogicalExperts || exd.n_ranks < 2 || exd.n_ranks > kMaxRanks)
    return cudaErrorInvalidValue;
  Exchange ex{exd.recv, exd.n_ranks, exd.my_rank, exd.node_size, exd.timeout_ns};
  const size_t smem = sizeof(int) * (size_t)n_logical;
  cudaError_t err = allow_smem(exchange_kernel, smem);
  if (err != cudaSuccess) return err;
  exchange_kernel<<<1, kBlock, smem, stream>>>(in, n_logical, ex, static_cast<Workspace*>(workspace), out, status);
  return cudaGetLastError();
}

template <typename IdxT>
struct FusedLaunch {
  const IdxT* idx;
  long long n;
  Topo tp;
  Exchange ex;
  IpmParams prm;
  Workspace* ws;
  float* probs;
  Counter avail;
  int* status;
  IdxT* out;
  int n_cta;
  unsigned long long grid_timeout_ns;
  unsigned long long* trace;
  int cooperative;
  cudaStream_t stream;
  template <int GP, int D>
  cudaError_t operator()() {
    auto kernel = fused_run_kernel<GP, D, IdxT>;
    const size_t smem = fused_smem(tp.e) + (GP == 0 ? block_smem(tp.n_group * tp.g, tp.g, tp.d) : bundle_smem(tp));
    cudaError_t err = allow_smem(kernel, smem);
    if (err != cudaSuccess) return err;
    void* args[] = {&idx, &n, &tp, &ex, &prm, &ws, &probs, &avail, &status, &out, &grid_timeout_ns, &trace};
    if (cooperative)
      return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(n_cta), dim3(kBlock), args, smem,
                                         stream);
    return cudaLaunchKernel(reinterpret_cast<void*>(kernel), dim3(n_cta), dim3(kBlock), args, smem, stream);
  }
};

cudaError_t launch_fused(const void* idx, int idx_is64, long long n, const TopoDesc& topo, const ExchangeDesc& exd,
                         SolveParams prm, void* workspace, float* probs, void* avail, int avail_is64, int* status,
                         void* out, int n_cta, unsigned long long grid_timeout_ns, unsigned long long* trace,
                         int cooperative, cudaStream_t stream) {
  if (!shape_ok(topo, true, prm.solver) || n_cta < 2 || exd.n_ranks > kMaxRanks) return cudaErrorInvalidValue;
  Exchange ex{exd.recv, exd.n_ranks, exd.my_rank, exd.node_size, exd.timeout_ns};
  if (idx_is64) {
    FusedLaunch<int64_t> l{static_cast<const int64_t*>(idx), n, make_topo(topo), ex, make_params(prm),
                           static_cast<Workspace*>(workspace), probs, Counter{avail, avail_is64}, status,
                           static_cast<int64_t*>(out), n_cta, grid_timeout_ns, trace, cooperative, stream};
    return dispatch_shape(topo.g, topo.d, prm.solver, l);
  }
  FusedLaunch<int32_t> l{static_cast<const int32_t*>(idx), n, make_topo(topo), ex, make_params(prm),
                         static_cast<Workspace*>(workspace), probs, Counter{avail, avail_is64}, status,
                         static_cast<int32_t*>(out), n_cta, grid_timeout_ns, trace, cooperative, stream};
  return dispatch_shape(topo.g, topo.d, prm.solver, l);
}

struct OccupancyQuery {
  size_t smem;
  int is64;
  int* result;
  template <int GP, int D>
  cudaError_t operator()() const {
    int per_sm = 0, dev = 0, sms = 0;
    cudaError_t err;
    if (is64) {
      if ((err = allow_smem(fused_run_kernel<GP, D, int64_t>, smem)) != cudaSuccess) return err;
      err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_run_kernel<GP, D, int64_t>, kBlock, smem);
    } else {
      if ((err = allow_smem(fused_run_kernel<GP, D, int32_t>, smem)) != cudaSuccess) return err;
      err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_run_kernel<GP, D, int32_t>, kBlock, smem);
    }
    if (err != cudaSuccess) return err;
    if ((err = cudaGetDevice(&dev)) != cudaSuccess) return err;
    if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return err;
    *result = per_sm * sms;
    return cudaSuccess;
  }
};

int max_fused_ctas(const TopoDesc& topo, int solver, int idx_is64) {
  int result = 0;
  if (!shape_ok(topo, true, solver)) return 0;
  const Topo tp = make_topo(topo);
  const bool block = resolve_solver(topo.g, topo.d, solver) == kSolverBlock;
  OccupancyQuery q{fused_smem(tp.e) + (block ? block_smem(tp.n_group * tp.g, tp.g, tp.d) : bundle_smem(tp)), idx_is64,
                   &result};
  if (dispatch_shape(topo.g, topo.d, solver, q) != cudaSuccess) return 0;
  return result;
}

}  // namespace lplb
