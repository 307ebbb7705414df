// Python binding of the benchmark MoE layer engine: buffers, peer mapping, weights and the
// forward pass (count -> plan -> dispatch -> GEMM1+SwiGLU -> GEMM2+combine -> reduce).
// The reference has no MoE layer; this exists for the end-to-end measurement that consumes
// the planner's redirected indices.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <cstring>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "moe_api.h"
#include "planner_api.h"

namespace py = pybind11;

#define MOE_CHECK(cond, msg)                                  \
  do {                                                        \
    if (!(cond)) {                                            \
      std::ostringstream oss_;                                \
      oss_ << "lplb_b200.moe: " << msg << " (" #cond ")";     \
      throw std::runtime_error(oss_.str());                   \
    }                                                         \
  } while (0)

#define MOE_CUDA(expr)                                                                          \
  do {                                                                                          \
    cudaError_t err_ = (expr);                                                                  \
    if (err_ != cudaSuccess) {                                                                  \
      std::ostringstream oss_;                                                                  \
      oss_ << "lplb_b200.moe: " #expr " failed: " << cudaGetErrorName(err_) << ": "            \
           << cudaGetErrorString(err_);                                                         \
      throw std::runtime_error(oss_.str());                                                     \
    }                                                                                           \
  } while (0)

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

class MoeEngine {
 public:
  MoeEngine(int hidden, int inter, int n_local, int n_ranks, int my_rank, int topk, int max_tokens, int capacity,
            int device)
      : device_(device) {
    sh_.hidden = hidden;
    sh_.inter = inter;
    sh_.n_local = n_local;
    sh_.n_ranks = n_ranks;
    sh_.my_rank = my_rank;
    sh_.topk = topk;
    sh_.max_tokens = max_tokens;
    sh_.capacity = capacity;
    MOE_CHECK(n_ranks >= 1 && n_ranks <= lplb::moe::kApiMaxRanks, "1..8 ranks supported");
    MOE_CHECK(hidden % 256 == 0 && inter % 128 == 0, "hidden must be a multiple of 256, inter of 128");
    MOE_CHECK((long long)max_tokens * topk < (1 << 20), "tokens * topk must stay below 2^20");
    MOE_CHECK(capacity % 128 == 0 && capacity < (1 << 24), "capacity must be a multiple of 128 below 2^24");
    p_ = n_ranks * n_local;
    off_recv_x_ = 0;
    off_meta_ = align_up(off_recv_x_ + (size_t)capacity * hidden * 2, 256);
    off_comb_ = align_up(off_meta_ + (size_t)capacity * 4, 256);
    off_cnt_ = align_up(off_comb_ + (size_t)max_tokens * topk * hidden * 2, 256);
    off_flags_ = align_up(off_cnt_ + sizeof(unsigned long long) * 2 * (size_t)n_ranks * p_, 256);
    off_arrived_ = align_up(off_flags_ + sizeof(uint32_t) * 2 * n_ranks, 256);
    block_bytes_ = align_up(off_arrived_ + sizeof(uint32_t) * n_local, 256);
  }

  ~MoeEngine() {
    try {
      close();
    } catch (...) {
    }
  }

  size_t peer_block_bytes() const { return block_bytes_; }

  // Allocate this rank's peer-visible block and the local buffers; returns the IPC handle.
  py::bytes alloc() {
    MOE_CHECK(!block_, "already allocated");
    c10::cuda::CUDAGuard guard(device_);
    MOE_CUDA(cudaMalloc(&block_, block_bytes_));
    MOE_CUDA(cudaMemset(block_, 0, block_bytes_));
    auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device_);
    act_ = torch::empty({sh_.capacity, sh_.inter}, i32.dtype(torch::kBFloat16));
    plan_ = torch::zeros({lplb::moe::plan_words(sh_.n_ranks, sh_.n_local)}, i32);
    workspace_ = torch::zeros({(int64_t)((lplb::planner_workspace_bytes(p_) + 3) / 4)}, i32);
    tickets_ = torch::zeros({4}, i32);
    pair_slot_ = torch::full({(int64_t)sh_.max_tokens * sh_.topk}, -1, i32);
    send_pair_ = torch::zeros({(int64_t)sh_.max_tokens * sh_.topk}, i32);
    send_target_ = torch::full({(int64_t)sh_.max_tokens * sh_.topk}, -1, i32);
    status_ = torch::zeros({32}, i32);  // see kMoeStatusWords in moe_support.cuh
    MOE_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t handle;
    MOE_CUDA(cudaIpcGetMemHandle(&handle, block_));
    return py::bytes(reinterpret_cast<const char*>(&handle), sizeof(handle));
  }

  // Map the peers' blocks (handles in rank order; this rank's own entry is ignored).
  void open(const std::vector<std::string>& handles) {
    MOE_CHECK(block_, "call alloc first");
    MOE_CHECK((int)handles.size() == sh_.n_ranks, "need one handle per rank");
    c10::cuda::CUDAGuard guard(device_);
    bases_.assign(sh_.n_ranks, nullptr);
    for (int r = 0; r < sh_.n_ranks; ++r) {
      if (r == sh_.my_rank) {
        bases_[r] = static_cast<char*>(block_);
        continue;
      }
      MOE_CHECK(handles[r].size() == sizeof(cudaIpcMemHandle_t), "malformed IPC handle from rank " << r);
      cudaIpcMemHandle_t handle;
      std::memcpy(&handle, handles[r].data(), sizeof(handle));
      void* base = nullptr;
      MOE_CUDA(cudaIpcOpenMemHandle(&base, handle, cudaIpcMemLazyEnablePeerAccess));
      bases_[r] = static_cast<char*>(base);
      opened_.push_back(base);
    }
    fill_buffers();
  }

  void close() {
    if (!block_) return;
    c10::cuda::CUDAGuard guard(device_);
    cudaDeviceSynchronize();
    for (void* p : opened_) cudaIpcCloseMemHandle(p);
    opened_.clear();
    cudaFree(block_);
    block_ = nullptr;
    ready_ = false;
  }

  // w13: [n_local, 2*inter, hidden] bf16, rows of every 256-row tile ordered 128 gate rows
  // then the 128 matching up rows.  w2: [n_local, hidden, inter] bf16.
  void set_weights(const torch::Tensor& w13, const torch::Tensor& w2) {
    MOE_CHECK(ready_, "open the peer blocks first");
    auto ok = [&](const torch::Tensor& t) {
      return t.is_cuda() && t.get_device() == device_ && t.scalar_type() == torch::kBFloat16 && t.is_contiguous();
    };
    MOE_CHECK(ok(w13) && w13.dim() == 3 && w13.size(0) == sh_.n_local && w13.size(1) == 2 * sh_.inter &&
                  w13.size(2) == sh_.hidden,
              "w13 must be contiguous bf16 [n_local, 2*inter, hidden] on this device");
    MOE_CHECK(ok(w2) && w2.dim() == 3 && w2.size(0) == sh_.n_local && w2.size(1) == sh_.hidden &&
                  w2.size(2) == sh_.inter,
              "w2 must be contiguous bf16 [n_local, hidden, inter] on this device");
    w13_ = w13;
    w2_ = w2;
    c10::cuda::CUDAGuard guard(device_);
    int rc = lplb::moe::make_tensor_map(&tm_x_, buf_.recv_x[sh_.my_rank], sh_.capacity, sh_.hidden, 128);
    MOE_CHECK(rc == 0, "tensor map for the receive buffer failed with code " << rc);
    rc = lplb::moe::make_tensor_map(&tm_w13_, w13.data_ptr(), (uint64_t)sh_.n_local * 2 * sh_.inter, sh_.hidden, 256);
    MOE_CHECK(rc == 0, "tensor map for w13 failed with code " << rc);
    rc = lplb::moe::make_tensor_map(&tm_act_, act_.data_ptr(), sh_.capacity, sh_.inter, 128);
    MOE_CHECK(rc == 0, "tensor map for the activation buffer failed with code " << rc);
    rc = lplb::moe::make_tensor_map(&tm_w2_, w2.data_ptr(), (uint64_t)sh_.n_local * sh_.hidden, sh_.inter, 256);
    MOE_CHECK(rc == 0, "tensor map for w2 failed with code " << rc);
    have_weights_ = true;
  }

  // One forward pass.  x: [T, hidden] bf16, phys_idx: [T, topk] int64/int32 physical expert
  // ids (-1 = dropped), weights: [T, topk] float32.  `upto` stops after a stage for tests:
  // 1 plan, 2 dispatch, 3 first GEMM, 4 second GEMM, 5 (default) everything.
  torch::Tensor forward(const torch::Tensor& x, const torch::Tensor& phys_idx, const torch::Tensor& weights,
                        int n_cta, int upto, bool fuse_dispatch) {
    MOE_CHECK(ready_ && have_weights_, "engine is not ready: open peers and set weights first");
    MOE_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 2 &&
                  x.size(1) == sh_.hidden && x.size(0) <= sh_.max_tokens,
              "x must be contiguous bf16 [tokens <= max_tokens, hidden]");
    const int n_tokens = (int)x.size(0);
    MOE_CHECK(phys_idx.is_cuda() && phys_idx.is_contiguous() && phys_idx.numel() == (int64_t)n_tokens * sh_.topk &&
                  (phys_idx.scalar_type() == torch::kInt64 || phys_idx.scalar_type() == torch::kInt32),
              "phys_idx must be contiguous int64/int32 [tokens, topk]");
    MOE_CHECK(weights.is_cuda() && weights.is_contiguous() && weights.scalar_type() == torch::kFloat32 &&
                  weights.numel() == phys_idx.numel(),
              "weights must be contiguous float32 [tokens, topk]");
    MOE_CHECK(n_cta >= 1, "n_cta must be positive");
    c10::cuda::CUDAGuard guard(device_);
    cudaStream_t s = c10::cuda::getCurrentCUDAStream(device_).stream();
    const int is64 = phys_idx.scalar_type() == torch::kInt64;
    ++epoch_;
    if (!by_cta_.defined() || by_cta_.size(0) != n_cta)
      by_cta_ = torch::empty({n_cta, p_}, status_.options());
    buf_.by_cta = by_cta_.data_ptr<int>();
    auto out = torch::empty({n_tokens, sh_.hidden}, x.options());
    MOE_CUDA(lplb::launch_count(phys_idx.data_ptr(), is64, phys_idx.numel(), p_, n_cta, buf_.by_cta,
                                workspace_.data_ptr(), status_.data_ptr<int>() + 8, s));
    // The fused path cannot stop between dispatch and the first GEMM: stage 2 then means both.
    const bool fused = fuse_dispatch && upto >= 3;
    MOE_CUDA(lplb::moe::launch_plan(sh_, buf_, n_cta, epoch_, timeout_ns_, fused ? 1 : 0, s));
    if (upto <= 1) return out;
    if (fused) {
      MOE_CUDA(lplb::moe::launch_schedule(sh_, buf_, phys_idx.data_ptr(), is64, n_tokens, n_cta, s));
      MOE_CUDA(lplb::moe::launch_dispatch_gemm(sh_, buf_, tm_x_, tm_w13_, x.data_ptr(), epoch_, timeout_ns_,
                                               gemm_ctas(), send_ctas_, s));
    } else {
      MOE_CUDA(lplb::moe::launch_dispatch(sh_, buf_, x.data_ptr(), phys_idx.data_ptr(), is64, n_tokens, n_cta,
                                          epoch_, s));
      if (upto <= 2) return out;
      MOE_CUDA(lplb::moe::launch_gemm(sh_, buf_, tm_x_, tm_w13_, 0, epoch_, timeout_ns_, gemm_ctas(), s));
    }
    if (upto <= 3) return out;
    MOE_CUDA(lplb::moe::launch_gemm(sh_, buf_, tm_act_, tm_w2_, 1, epoch_, timeout_ns_, gemm_ctas(), s));
    if (upto <= 4) return out;
    MOE_CUDA(lplb::moe::launch_combine(sh_, buf_, weights.data_ptr<float>(), out.data_ptr(), n_tokens, epoch_,
                                       timeout_ns_, 4 * sm_count(), s));
    return out;
  }

  void set_timeout_us(double us) { timeout_ns_ = (unsigned long long)(us * 1e3); }
  // Fused dispatch: 0 = four sender warps beside the tile roles in every CTA; n > 0 = n CTAs
  // (of one per SM) only send rows and the rest only run tiles.
  void set_send_ctas(int n) {
    MOE_CHECK(n >= 0 && n < gemm_ctas(), "send_ctas must be in [0, number of GEMM CTAs)");
    send_ctas_ = n;
  }
  torch::Tensor status() const { return status_; }
  torch::Tensor plan() const { return plan_; }
  torch::Tensor act() const { return act_; }
  torch::Tensor pair_slot() const { return pair_slot_; }
  // Timing of the fused dispatch+GEMM kernel, [n_sm, 4] ns per CTA: start, senders done,
  // time the TMA producer spent waiting for rows, end.  Zeroed on enable.
  torch::Tensor enable_debug(bool on) {
    c10::cuda::CUDAGuard guard(device_);
    if (on) {
      debug_ = torch::zeros({sm_count(), 4}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, device_));
      buf_.debug = reinterpret_cast<unsigned long long*>(debug_.data_ptr());
    } else {
      debug_ = torch::Tensor();
      buf_.debug = nullptr;
    }
    return debug_;
  }
  int64_t epoch() const { return epoch_; }

  // Back to the state after open(): launch number 0, all epoch-tagged words, flags, arrival
  // counters and the status block of this rank cleared.  For use after a timeout, when the
  // ranks no longer agree on how many rows or flags were delivered.  Every rank must call it
  // with none of the layer's kernels in flight anywhere, and no rank may launch again before
  // all have returned (the Python layer puts a barrier on either side).
  void reset() {
    MOE_CHECK(ready_, "engine is not open");
    c10::cuda::CUDAGuard guard(device_);
    MOE_CUDA(cudaDeviceSynchronize());
    MOE_CUDA(cudaMemset(static_cast<char*>(block_) + off_cnt_, 0, block_bytes_ - off_cnt_));
    plan_.zero_();
    tickets_.zero_();
    status_.zero_();
    workspace_.zero_();
    epoch_ = 0;
    MOE_CUDA(cudaDeviceSynchronize());
  }

  // Views of this rank's peer-visible buffers (for tests).
  torch::Tensor recv_x() const {
    auto opts = torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA, device_);
    return torch::from_blob(buf_.recv_x[sh_.my_rank], {sh_.capacity, sh_.hidden}, opts);
  }
  torch::Tensor recv_meta() const {
    auto opts = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device_);
    return torch::from_blob(buf_.recv_meta[sh_.my_rank], {sh_.capacity}, opts);
  }
  torch::Tensor comb() const {
    auto opts = torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA, device_);
    return torch::from_blob(buf_.comb[sh_.my_rank], {(int64_t)sh_.max_tokens * sh_.topk, sh_.hidden}, opts);
  }

 private:
  int sm_count() {
    if (sms_ == 0) cudaDeviceGetAttribute(&sms_, cudaDevAttrMultiProcessorCount, device_);
    return sms_;
  }
  int gemm_ctas() { return sm_count(); }

  void fill_buffers() {
    for (int r = 0; r < sh_.n_ranks; ++r) {
      char* base = bases_[r];
      buf_.recv_x[r] = base + off_recv_x_;
      buf_.recv_meta[r] = reinterpret_cast<int*>(base + off_meta_);
      buf_.comb[r] = base + off_comb_;
      buf_.cnt_words[r] = reinterpret_cast<unsigned long long*>(base + off_cnt_);
      buf_.flags[r] = reinterpret_cast<uint32_t*>(base + off_flags_);
      buf_.arrived[r] = reinterpret_cast<uint32_t*>(base + off_arrived_);
    }
    buf_.act = act_.data_ptr();
    buf_.plan = plan_.data_ptr<int>();
    buf_.by_cta = nullptr;
    buf_.debug = nullptr;
    buf_.pair_slot = pair_slot_.data_ptr<int>();
    buf_.send_pair = send_pair_.data_ptr<int>();
    buf_.send_target = send_target_.data_ptr<int>();
    buf_.planner_workspace = workspace_.data_ptr();
    buf_.tickets = reinterpret_cast<unsigned*>(tickets_.data_ptr<int>());
    buf_.status = status_.data_ptr<int>();
    ready_ = true;
  }

  lplb::moe::LayerShape sh_{};
  lplb::moe::LayerBuffers buf_{};
  int device_, p_ = 0, sms_ = 0;
  size_t off_recv_x_ = 0, off_meta_ = 0, off_comb_ = 0, off_cnt_ = 0, off_flags_ = 0, off_arrived_ = 0, block_bytes_ = 0;
  void* block_ = nullptr;
  std::vector<char*> bases_;
  std::vector<void*> opened_;
  torch::Tensor act_, plan_, workspace_, tickets_, status_, by_cta_, pair_slot_, send_pair_, send_target_, debug_, w13_, w2_;
  CUtensorMap tm_x_{}, tm_w13_{}, tm_act_{}, tm_w2_{};
  bool ready_ = false, have_weights_ = false;
  uint32_t epoch_ = 0;
  unsigned long long timeout_ns_ = 2000000000ull;
  int send_ctas_ = 0;
};

}  // namespace

void bind_moe(py::module_& m) {
  py::class_<MoeEngine>(m, "MoeEngine")
      .def(py::init<int, int, int, int, int, int, int, int, int>(), py::arg("hidden"), py::arg("inter"),
           py::arg("n_local"), py::arg("n_ranks"), py::arg("my_rank"), py::arg("topk"), py::arg("max_tokens"),
           py::arg("capacity"), py::arg("device"))
      .def("peer_block_bytes", &MoeEngine::peer_block_bytes)
      .def("alloc", &MoeEngine::alloc)
      .def("open", &MoeEngine::open)
      .def("close", &MoeEngine::close)
      .def("set_weights", &MoeEngine::set_weights)
      .def("forward", &MoeEngine::forward, py::arg("x"), py::arg("phys_idx"), py::arg("weights"), py::arg("n_cta"),
           py::arg("upto") = 5, py::arg("fuse_dispatch") = false)
      .def("set_timeout_us", &MoeEngine::set_timeout_us)
      .def("set_send_ctas", &MoeEngine::set_send_ctas)
      .def("reset", &MoeEngine::reset)
      .def("status", &MoeEngine::status)
      .def("plan", &MoeEngine::plan)
      .def("act", &MoeEngine::act)
      .def("pair_slot", &MoeEngine::pair_slot)
      .def("enable_debug", &MoeEngine::enable_debug)
      .def("epoch", &MoeEngine::epoch)
      .def("recv_x", &MoeEngine::recv_x)
      .def("recv_meta", &MoeEngine::recv_meta)
      .def("comb", &MoeEngine::comb);
}
