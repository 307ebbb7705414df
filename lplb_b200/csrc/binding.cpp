// Python binding of the native planner runtime.
//
// `PlannerEngine` owns everything that lives on the GPU for one planner: the static
// topology/placement tables, the per-engine workspace and status block, and (when a
// process group is attached) the peer-memory exchange buffers.  It plays the role of the
// reference's `CompiledSolver` (reference csrc/plugin.cpp:122-147, :663-679) without a
// run-time compiler.  The exchange bootstrap mirrors what the reference's `init_comm`
// does for its intra-node tier (reference csrc/plugin.cpp:395-448): allocate with
// cudaMalloc, export a CUDA-IPC handle, let Python all-gather the handles through
// torch.distributed, open the peers' handles and upload a pointer table.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "planner_api.h"

namespace py = pybind11;

#define LPLB_CHECK(cond, msg)                                   \
  do {                                                          \
    if (!(cond)) {                                              \
      std::ostringstream oss_;                                  \
      oss_ << "lplb_b200: " << msg << " (" #cond ")";           \
      throw std::runtime_error(oss_.str());                     \
    }                                                           \
  } while (0)

#define LPLB_CUDA(expr)                                                                 \
  do {                                                                                  \
    cudaError_t err_ = (expr);                                                          \
    if (err_ != cudaSuccess) {                                                          \
      std::ostringstream oss_;                                                          \
      oss_ << "lplb_b200: " #expr " failed: " << cudaGetErrorName(err_) << ": "        \
           << cudaGetErrorString(err_);                                                 \
      throw std::runtime_error(oss_.str());                                             \
    }                                                                                   \
  } while (0)

namespace {

struct IpcBlock {
  // One cudaMalloc'd region: uint64 recv[2][n_ranks][E], every word (epoch << 32) | count.
  void* base = nullptr;
  size_t bytes = 0;
};

class PlannerEngine {
 public:
  PlannerEngine(int n_group, int g, int d, int ll, int c, int device)
      : n_group_(n_group), g_(g), d_(d), ll_(ll), c_(c), device_(device) {
    // Groups beyond the device solvers' sizes can still be counted and redirected here; their LP
    // is solved by the caller (see Planner.solve_probs).
    LPLB_CHECK(g >= 1 && d >= 1, "group size and replicas per rank must be positive");
    LPLB_CHECK(ll >= c * d, "local logical experts < replicated experts");
    e_ = n_group * g * ll;
    LPLB_CHECK(e_ <= lplb::kMaxLogicalExperts, "too many logical experts: " << e_);
    c10::cuda::CUDAGuard guard(device_);
    auto opts = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device_);
    const size_t ws_bytes = lplb::planner_workspace_bytes(e_);
    workspace_ = torch::zeros({(int64_t)((ws_bytes + 3) / 4)}, opts);
    status_ = torch::zeros({16}, opts);
    probs_ = torch::zeros({n_group, g, d}, opts.dtype(torch::kFloat32));
  }

  ~PlannerEngine() {
    try {
      close_exchange();
    } catch (...) {
    }
  }

  void set_topology(const torch::Tensor& r2o, const torch::Tensor& o2r) {
    LPLB_CHECK(r2o.dim() == 2 && r2o.size(0) == g_ && r2o.size(1) == d_, "r2o must be [G, D]");
    LPLB_CHECK(o2r.sizes() == r2o.sizes(), "o2r must match r2o");
    r2o_ = to_dev_i32(r2o);
    o2r_ = to_dev_i32(o2r);
  }

  void set_mapping(const torch::Tensor& phy2log, const torch::Tensor& log2phy, const torch::Tensor& log2edge) {
    const int64_t pl = ll_ + c_ * d_;
    LPLB_CHECK(phy2log.numel() == (int64_t)n_group_ * g_ * pl, "phy2log has the wrong size");
    LPLB_CHECK(log2phy.dim() == 2 && log2phy.size(0) == e_ && log2phy.size(1) == 2, "log2phy must be [E, 2]");
    LPLB_CHECK(log2edge.numel() == e_, "log2edge must be [E]");
    // The tables keep their device addresses for the engine's lifetime (a captured CUDA graph
    // of a launch stays valid across re-placements); new contents are copied in, ordered on
    // the current stream after the launches already enqueued.
    store_i32(phy2log_, phy2log);
    store_i32(log2phy_, log2phy);
    store_i32(log2edge_, log2edge);
    // log2slot[e] = rank * (D + 1) + bundle: where expert e's count goes in the LP's per-rank
    // sums (bundle d of the rank for its replicated experts, slot D for the others).
    {
      c10::cuda::CUDAGuard guard(device_);
      auto i64 = torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, device_);
      const int64_t ranks = (int64_t)n_group_ * g_;
      auto own = phy2log_.view({ranks, pl}).slice(1, 0, ll_).to(torch::kInt64).reshape({-1});
      auto sl = torch::arange(ll_, i64);
      auto code = torch::where(sl < (int64_t)c_ * d_, sl.remainder(d_), torch::full_like(sl, d_));
      auto slot = (torch::arange(ranks, i64).unsqueeze(1) * (d_ + 1) + code.unsqueeze(0)).reshape({-1});
      auto table = torch::zeros({e_}, i64);
      LPLB_CHECK(own.numel() == e_, "phy2log does not hold every logical expert once");
      table.scatter_(0, own.clamp(0, e_ - 1), slot);
      store_i32(log2slot_, table);
    }
    invalidate_warm_start();  // a new placement is a new LP
  }

  // Warm starts: keep a centred iterate per group on the device and start the next solve from
  // it while it still fits the data (see IpmParams in lp_solver.cuh).
  void set_warm_start(bool on, double guard, double snap_mu) {
    c10::cuda::CUDAGuard dev_guard(device_);
    if (on) {
      LPLB_CHECK(guard > 0 && snap_mu > 0, "guard and snap_mu must be positive");
      const int dp = lplb::anchor_dup(g_, d_, prm_.solver);
      if (!anchor_.defined() || anchor_.size(2) != 4 * dp + 3) {
        auto f64 = torch::TensorOptions().dtype(torch::kFloat64).device(torch::kCUDA, device_);
        anchor_ = torch::zeros({n_group_, g_, 4 * dp + 3}, f64);
        anchor_valid_ = torch::zeros({n_group_}, status_.options());
      }
      warm_ = true;
      prm_.anchor = anchor_.data_ptr<double>();
      prm_.anchor_valid = anchor_valid_.data_ptr<int>();
      prm_.guard = guard;
      prm_.snap_mu = snap_mu;
    } else {
      prm_.anchor = nullptr;
      prm_.anchor_valid = nullptr;
      warm_ = false;
    }
  }

  // Which device solver runs the LPs: "auto" (warp solver up to 8 ranks, thread-block solver
  // above), "warp" or "block".  The warm-start state is laid out per solver, so it is dropped.
  void set_solver(const std::string& kind) {
    int k = kind == "auto" ? lplb::kSolverAuto : kind == "warp" ? lplb::kSolverWarp : kind == "block" ? lplb::kSolverBlock : -1;
    LPLB_CHECK(k >= 0, "solver must be auto, warp or block, got " << kind);
    LPLB_CHECK(lplb::resolve_solver(g_, d_, k) > 0, "the " << kind << " solver does not cover " << g_ << " ranks x " << d_ << " replicas");
    prm_.solver = k;
    max_cta64_ = max_cta32_ = -1;
    if (warm_) set_warm_start(true, prm_.guard, prm_.snap_mu);
    invalidate_warm_start();
  }
  // [n_group] int32: 1 where a saved iterate exists (empty tensor when warm starts are off).
  torch::Tensor warm_start_valid() const {
    return anchor_valid_.defined() ? anchor_valid_ : torch::zeros({0}, status_.options());
  }
  std::string solver() const {
    const int k = lplb::resolve_solver(g_, d_, prm_.solver);
    return k == lplb::kSolverWarp ? "warp" : k == lplb::kSolverBlock ? "block" : "none";
  }
  // Forget the saved iterates (next solve of every group starts cold).  Stream-ordered.
  void invalidate_warm_start() {
    if (anchor_valid_.defined()) anchor_valid_.zero_();
  }

  void set_params(int max_iters, double tol, double peer_timeout_us, double grid_timeout_us) {
    LPLB_CHECK(max_iters >= 1 && max_iters <= 1000, "max_iters out of range");
    LPLB_CHECK(tol > 0, "tol must be positive");
    prm_.max_iters = max_iters;
    prm_.tol = tol;
    peer_timeout_ns_ = (unsigned long long)(peer_timeout_us * 1e3);
    grid_timeout_ns_ = (unsigned long long)(grid_timeout_us * 1e3);
  }

  // ---- stand-alone stages ---------------------------------------------------------
  std::tuple<torch::Tensor, torch::Tensor> count_idx(const torch::Tensor& idx, int n_cta) {
    check_idx(idx);
    LPLB_CHECK(n_cta >= 1, "n_sms must be positive");
    c10::cuda::CUDAGuard guard(device_);
    auto by_cta = torch::empty({n_cta, e_}, status_.options());
    LPLB_CUDA(lplb::launch_count(idx.data_ptr(), idx.scalar_type() == torch::kInt64, idx.numel(), e_, n_cta,
                                 by_cta.data_ptr<int>(), workspace_.data_ptr(), status_.data_ptr<int>(), stream()));
    return {by_cta[n_cta - 1], by_cta};
  }

  std::tuple<torch::Tensor, torch::Tensor> solve(const torch::Tensor& workload, torch::Tensor avail) {
    require_mapping();
    LPLB_CHECK(workload.is_cuda() && workload.scalar_type() == torch::kInt32 && workload.is_contiguous(),
               "workload must be a contiguous int32 CUDA tensor");
    LPLB_CHECK(workload.numel() == e_, "workload must have " << e_ << " entries, got " << workload.numel());
    LPLB_CHECK(has_native_solver(), "no device solver for this group size; use the tensor-op solver");
    check_avail(avail);
    c10::cuda::CUDAGuard guard(device_);
    auto probs = torch::empty({n_group_, g_, d_}, probs_.options());
    auto normalised = torch::empty({n_group_, g_, ll_}, probs_.options());
    LPLB_CUDA(lplb::launch_solve(workload.data_ptr<int>(), topo(), prm_, probs.data_ptr<float>(),
                                 normalised.data_ptr<float>(), avail.data_ptr(),
                                 avail.scalar_type() == torch::kInt64, status_.data_ptr<int>(), stream()));
    return {probs, normalised};
  }

  torch::Tensor map_idx(const torch::Tensor& idx, const torch::Tensor& probs, const torch::Tensor& by_cta, int n_cta) {
    require_mapping();
    check_idx(idx);
    LPLB_CHECK(probs.is_cuda() && probs.scalar_type() == torch::kFloat32 && probs.is_contiguous() &&
                   probs.numel() == (int64_t)n_group_ * g_ * d_,
               "o_weight must be a contiguous float32 CUDA tensor with NG*G*D entries");
    LPLB_CHECK(by_cta.is_cuda() && by_cta.scalar_type() == torch::kInt32 && by_cta.is_contiguous() &&
                   by_cta.dim() == 2 && by_cta.size(0) == n_cta && by_cta.size(1) == e_,
               "local_workload_by_sm must be the [n_sms, E] int32 tensor returned by count_workload with the same n_sms");
    c10::cuda::CUDAGuard guard(device_);
    auto out = torch::empty_like(idx);
    LPLB_CUDA(lplb::launch_redirect(idx.data_ptr(), idx.scalar_type() == torch::kInt64, idx.numel(),
                                    probs.data_ptr<float>(), by_cta.data_ptr<int>(), topo(), n_cta, out.data_ptr(),
                                    stream()));
    return out;
  }

  // Sum a caller-provided int32[E] statistics vector over the peers (NVLink push exchange).
  torch::Tensor all_reduce_counts(const torch::Tensor& workload) {
    LPLB_CHECK(exchange_open_, "exchange buffers are not open; call open_exchange first");
    LPLB_CHECK(workload.is_cuda() && workload.scalar_type() == torch::kInt32 && workload.is_contiguous() &&
                   workload.numel() == e_,
               "workload must be a contiguous int32 CUDA tensor with " << e_ << " entries");
    c10::cuda::CUDAGuard guard(device_);
    auto out = torch::empty_like(workload);
    LPLB_CUDA(lplb::launch_exchange(workload.data_ptr<int>(), e_, exchange_desc(), workspace_.data_ptr(),
                                    out.data_ptr<int>(), status_.data_ptr<int>(), stream()));
    return out;
  }

  // ---- single launch ------------------------------------------------------------------
  // `idx` may also be a pinned host tensor: the kernel then reads it over PCIe itself and,
  // if `out` is a pinned host tensor too, writes the result straight back, which replaces two
  // copy-engine transfers and their launch latencies.  `out` must match `idx` in shape/dtype.
  torch::Tensor run_fused(const torch::Tensor& idx, torch::Tensor avail, int n_cta, bool use_exchange,
                          c10::optional<torch::Tensor> out_opt) {
    require_mapping();
    const bool host_idx = !idx.is_cuda();
    if (host_idx) {
      LPLB_CHECK(idx.is_pinned(), "host indices must be in pinned memory");
      LPLB_CHECK(idx.scalar_type() == torch::kInt64 || idx.scalar_type() == torch::kInt32, "indices must be int64 or int32");
      LPLB_CHECK(idx.is_contiguous(), "indices must be contiguous");
    } else {
      check_idx(idx);
    }
    check_avail(avail);
    c10::cuda::CUDAGuard guard(device_);
    const int is64 = idx.scalar_type() == torch::kInt64;
    LPLB_CHECK(has_native_solver(), "the fused kernel needs a group of at most " << lplb::kMaxGroupSize
                                        << " ranks with at most " << lplb::kMaxDup << " replicas each");
    LPLB_CHECK(!use_exchange || n_ranks_ <= 32, "the in-kernel exchange covers at most 32 ranks");
    int& limit = is64 ? max_cta64_ : max_cta32_;
    if (limit < 0) limit = lplb::max_fused_ctas(topo(), prm_.solver, is64);
    LPLB_CHECK(limit >= 2, "fused kernel cannot be resident on this device");
    // one CTA solves, the others count and redirect: a request for a single CTA still gets one worker
    if (n_cta < 2) n_cta = 2;
    if (n_cta > limit) n_cta = limit;
    torch::Tensor out;
    if (out_opt.has_value()) {
      out = *out_opt;
      LPLB_CHECK(out.sizes() == idx.sizes() && out.scalar_type() == idx.scalar_type() && out.is_contiguous(),
                 "out must match idx in shape and dtype and be contiguous");
      LPLB_CHECK((out.is_cuda() && out.get_device() == device_) || (!out.is_cuda() && out.is_pinned()),
                 "out must live on this device or in pinned host memory");
    } else {
      LPLB_CHECK(!host_idx, "pass a pinned `out` tensor together with pinned host indices");
      out = torch::empty_like(idx);
    }
    lplb::ExchangeDesc ex{nullptr, 1, 0, 0, peer_timeout_ns_};
    if (use_exchange) {
      LPLB_CHECK(exchange_open_, "exchange buffers are not open; call open_exchange first");
      ex = exchange_desc();
    }
    LPLB_CUDA(lplb::launch_fused(idx.data_ptr(), is64, idx.numel(), topo(), ex, prm_, workspace_.data_ptr(),
                                 probs_.data_ptr<float>(), avail.data_ptr(), avail.scalar_type() == torch::kInt64,
                                 status_.data_ptr<int>(), out.data_ptr(), n_cta, grid_timeout_ns_,
                                 trace_.defined() ? reinterpret_cast<unsigned long long*>(trace_.data_ptr()) : nullptr,
                                 cooperative_ ? 1 : 0, stream()));
    return out;
  }

  // ---- exchange bootstrap ---------------------------------------------------------------
  // Step 1 (every rank): allocate and return the IPC handle as bytes.
  py::bytes alloc_exchange(int n_ranks, int my_rank) {
    LPLB_CHECK(!block_.base, "exchange buffers already allocated");
    LPLB_CHECK(n_ranks >= 2 && n_ranks <= 32 && my_rank >= 0 && my_rank < n_ranks, "bad rank layout");
    c10::cuda::CUDAGuard guard(device_);
    n_ranks_ = n_ranks;
    my_rank_ = my_rank;
    block_.bytes = lplb::exchange_buffer_bytes(n_ranks, e_);
    LPLB_CUDA(cudaMalloc(&block_.base, block_.bytes));
    LPLB_CUDA(cudaMemset(block_.base, 0, block_.bytes));
    LPLB_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t handle;
    LPLB_CUDA(cudaIpcGetMemHandle(&handle, block_.base));
    return py::bytes(reinterpret_cast<const char*>(&handle), sizeof(handle));
  }

  // Step 2 (every rank, after the handles were all-gathered): map the peers.
  void open_exchange(const std::vector<std::string>& handles) {
    LPLB_CHECK(block_.base, "call alloc_exchange first");
    LPLB_CHECK((int)handles.size() == n_ranks_, "need one handle per rank");
    c10::cuda::CUDAGuard guard(device_);
    std::vector<int64_t> recv(n_ranks_);
    peers_.assign(n_ranks_, nullptr);
    for (int r = 0; r < n_ranks_; ++r) {
      void* base = block_.base;
      if (r != my_rank_) {
        LPLB_CHECK(handles[r].size() == sizeof(cudaIpcMemHandle_t), "malformed IPC handle from rank " << r);
        cudaIpcMemHandle_t handle;
        memcpy(&handle, handles[r].data(), sizeof(handle));
        LPLB_CUDA(cudaIpcOpenMemHandle(&base, handle, cudaIpcMemLazyEnablePeerAccess));
        peers_[r] = base;
      }
      recv[r] = reinterpret_cast<int64_t>(base);
    }
    auto opts = torch::TensorOptions().dtype(torch::kInt64);
    recv_table_ = torch::from_blob(recv.data(), {n_ranks_}, opts).clone().to(torch::Device(torch::kCUDA, device_));
    exchange_open_ = true;
  }

  // Single-process stand-in for the peer mapping, for tests on one GPU: every "peer"
  // pointer aliases this rank's own block.  Slots and flags of the other ranks are only
  // ever written by `debug_fill_slot`, so a test decides which peers "arrived".
  void open_exchange_loopback(int n_ranks, int my_rank) {
    LPLB_CHECK(!block_.base, "exchange buffers already allocated");
    LPLB_CHECK(n_ranks >= 2 && n_ranks <= 32 && my_rank >= 0 && my_rank < n_ranks, "bad rank layout");
    c10::cuda::CUDAGuard guard(device_);
    n_ranks_ = n_ranks;
    my_rank_ = my_rank;
    block_.bytes = lplb::exchange_buffer_bytes(n_ranks, e_);
    LPLB_CUDA(cudaMalloc(&block_.base, block_.bytes));
    LPLB_CUDA(cudaMemset(block_.base, 0, block_.bytes));
    std::vector<int64_t> recv(n_ranks_, reinterpret_cast<int64_t>(block_.base));
    auto opts = torch::TensorOptions().dtype(torch::kInt64);
    recv_table_ = torch::from_blob(recv.data(), {n_ranks_}, opts).clone().to(torch::Device(torch::kCUDA, device_));
    peers_.clear();
    exchange_open_ = true;
  }

  // Test hook: make it look as if `rank` had published `counts` for launch number `epoch`
  // (the launch after `completed_launches()` has epoch completed + 1).
  void debug_fill_slot(int rank, const torch::Tensor& counts, int64_t epoch, int level) {
    LPLB_CHECK(block_.base && rank >= 0 && rank < n_ranks_, "no exchange block or bad rank");
    LPLB_CHECK(counts.numel() == e_, "counts must have E entries");
    c10::cuda::CUDAGuard guard(device_);
    auto words = (counts.to(torch::kCPU, torch::kInt64).contiguous() & 0xffffffffLL) + (epoch << 32);
    LPLB_CUDA(cudaDeviceSynchronize());
    LPLB_CHECK(level == 0 || level == 1, "level is 0 or 1");
    auto* slot = static_cast<unsigned long long*>(block_.base) + (((size_t)(epoch & 1) * 2 + level) * n_ranks_ + rank) * e_;
    LPLB_CUDA(cudaMemcpy(slot, words.data_ptr<int64_t>(), sizeof(int64_t) * e_, cudaMemcpyHostToDevice));
  }

  // Launches (fused or stand-alone exchange) completed so far on this engine; synchronises.
  int64_t completed_launches() {
    c10::cuda::CUDAGuard guard(device_);
    return (int64_t)(uint32_t)workspace_[0].item<int>();
  }

  // Collective by convention: every rank calls it between steps, with no launch in flight,
  // after a barrier.  Zeroes this rank's epochs, flags and receive buffers.
  void reset_exchange() {
    c10::cuda::CUDAGuard guard(device_);
    LPLB_CUDA(cudaDeviceSynchronize());
    workspace_.zero_();
    invalidate_warm_start();
    if (block_.base) LPLB_CUDA(cudaMemset(block_.base, 0, block_.bytes));
    LPLB_CUDA(cudaDeviceSynchronize());
  }

  void close_exchange() {
    if (!block_.base) return;
    c10::cuda::CUDAGuard guard(device_);
    cudaDeviceSynchronize();
    for (void* p : peers_)
      if (p) cudaIpcCloseMemHandle(p);
    peers_.clear();
    cudaFree(block_.base);
    block_.base = nullptr;
    exchange_open_ = false;
  }

  // Two-level schedule of the exchange: ranks form nodes of `node_size` consecutive ranks
  // (must divide the rank count); 0 restores the one-level all-to-all.
  void set_exchange_nodes(int node_size) {
    LPLB_CHECK(node_size >= 0 && (node_size == 0 || (n_ranks_ % node_size == 0)), "node_size must divide the rank count");
    node_size_ = node_size;
  }

  // Cooperative launch (default) makes the driver guarantee that all CTAs of the fused kernel
  // are co-resident; an ordinary launch is cheaper but leaves that to the caller.
  void set_cooperative(bool on) { cooperative_ = on; }

  // Phase stamps of the fused kernel (see fused_run_kernel): off by default.
  void enable_trace(bool on) {
    c10::cuda::CUDAGuard guard(device_);
    if (on && !trace_.defined())
      trace_ = torch::zeros({16}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, device_));
    if (!on) trace_ = torch::Tensor();
  }
  torch::Tensor trace() const { return trace_; }

  bool exchange_open() const { return exchange_open_; }
  torch::Tensor status() const { return status_; }
  torch::Tensor last_probs() const { return probs_; }
  torch::Tensor workspace() const { return workspace_; }
  int n_logical() const { return e_; }
  bool has_native_solver() const { return lplb::resolve_solver(g_, d_, prm_.solver) > 0; }
  int max_fused_ctas(bool is64) {
    require_mapping();
    c10::cuda::CUDAGuard guard(device_);
    return lplb::max_fused_ctas(topo(), prm_.solver, is64);
  }

 private:
  cudaStream_t stream() const { return c10::cuda::getCurrentCUDAStream(device_).stream(); }

  torch::Tensor to_dev_i32(const torch::Tensor& t) const {
    return t.to(torch::Device(torch::kCUDA, device_), torch::kInt32).contiguous().clone();
  }
  void store_i32(torch::Tensor& dst, const torch::Tensor& src) const {
    if (!dst.defined()) {
      dst = to_dev_i32(src);
      return;
    }
    c10::cuda::CUDAGuard guard(device_);
    dst.copy_(src.reshape(dst.sizes()));
  }

  lplb::ExchangeDesc exchange_desc() const {
    return lplb::ExchangeDesc{reinterpret_cast<unsigned long long* const*>(recv_table_.data_ptr()), n_ranks_,
                              my_rank_, node_size_, peer_timeout_ns_};
  }

  void require_mapping() const {
    LPLB_CHECK(r2o_.defined() && phy2log_.defined(), "topology and mapping must be set before launching");
  }

  void check_idx(const torch::Tensor& idx) const {
    LPLB_CHECK(idx.is_cuda() && idx.get_device() == device_, "indices must live on cuda:" << device_);
    LPLB_CHECK(idx.scalar_type() == torch::kInt64 || idx.scalar_type() == torch::kInt32, "indices must be int64 or int32");
    LPLB_CHECK(idx.is_contiguous(), "indices must be contiguous");
  }

  void check_avail(const torch::Tensor& avail) const {
    LPLB_CHECK(avail.is_cuda() && avail.numel() == 1 &&
                   (avail.scalar_type() == torch::kInt32 || avail.scalar_type() == torch::kInt64),
               "avail_counter must be a one-element int32 or int64 CUDA tensor");
  }

  lplb::TopoDesc topo() const {
    return lplb::TopoDesc{r2o_.data_ptr<int>(),     o2r_.data_ptr<int>(),      phy2log_.data_ptr<int>(),
                          log2phy_.data_ptr<int>(), log2edge_.data_ptr<int>(), log2slot_.data_ptr<int>(),
                          n_group_, g_, d_, ll_, c_};
  }

  int n_group_, g_, d_, ll_, c_, e_, device_;
  lplb::SolveParams prm_{24, 1e-4};
  unsigned long long peer_timeout_ns_ = 1000000000ull, grid_timeout_ns_ = 1000000000ull;
  torch::Tensor r2o_, o2r_, phy2log_, log2phy_, log2edge_, log2slot_;
  bool warm_ = false;
  torch::Tensor workspace_, status_, probs_, trace_, anchor_, anchor_valid_;
  int max_cta64_ = -1, max_cta32_ = -1;
  // exchange
  IpcBlock block_;
  std::vector<void*> peers_;
  torch::Tensor recv_table_;
  int n_ranks_ = 1, my_rank_ = 0, node_size_ = 0;
  bool exchange_open_ = false;
  bool cooperative_ = true;
};

}  // namespace

void bind_moe(py::module_& m);  // moe_binding.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "lplb_b200 native runtime (sm_100a)";
  py::class_<PlannerEngine>(m, "PlannerEngine")
      .def(py::init<int, int, int, int, int, int>(), py::arg("n_group"), py::arg("group_size"),
           py::arg("dup_per_rank"), py::arg("n_local_logical"), py::arg("n_combined"), py::arg("device"))
      .def("set_topology", &PlannerEngine::set_topology)
      .def("set_mapping", &PlannerEngine::set_mapping)
      .def("set_params", &PlannerEngine::set_params)
      .def("set_warm_start", &PlannerEngine::set_warm_start)
      .def("set_solver", &PlannerEngine::set_solver)
      .def("solver", &PlannerEngine::solver)
      .def("warm_start_valid", &PlannerEngine::warm_start_valid)
      .def("invalidate_warm_start", &PlannerEngine::invalidate_warm_start)
      .def("count_idx", &PlannerEngine::count_idx)
      .def("solve", &PlannerEngine::solve)
      .def("map_idx", &PlannerEngine::map_idx)
      .def("run_fused", &PlannerEngine::run_fused, py::arg("idx"), py::arg("avail"), py::arg("n_cta"),
           py::arg("use_exchange"), py::arg("out") = py::none())
      .def("all_reduce_counts", &PlannerEngine::all_reduce_counts)
      .def("alloc_exchange", &PlannerEngine::alloc_exchange)
      .def("open_exchange", &PlannerEngine::open_exchange)
      .def("open_exchange_loopback", &PlannerEngine::open_exchange_loopback)
      .def("debug_fill_slot", &PlannerEngine::debug_fill_slot, py::arg("rank"), py::arg("counts"), py::arg("epoch"),
           py::arg("level") = 0)
      .def("completed_launches", &PlannerEngine::completed_launches)
      .def("reset_exchange", &PlannerEngine::reset_exchange)
      .def("close_exchange", &PlannerEngine::close_exchange)
      .def("exchange_open", &PlannerEngine::exchange_open)
      .def("set_cooperative", &PlannerEngine::set_cooperative)
      .def("set_exchange_nodes", &PlannerEngine::set_exchange_nodes)
      .def("enable_trace", &PlannerEngine::enable_trace)
      .def("trace", &PlannerEngine::trace)
      .def("status", &PlannerEngine::status)
      .def("last_probs", &PlannerEngine::last_probs)
      .def("workspace", &PlannerEngine::workspace)
      .def("n_logical", &PlannerEngine::n_logical)
      .def("has_native_solver", &PlannerEngine::has_native_solver)
      .def("max_fused_ctas", &PlannerEngine::max_fused_ctas);
  bind_moe(m);
  m.attr("MAX_GROUP_SIZE") = lplb::kMaxGroupSize;
  m.attr("MAX_DUP") = lplb::kMaxDup;
  m.attr("MAX_LOGICAL_EXPERTS") = lplb::kMaxLogicalExperts;
}
