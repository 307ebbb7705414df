// Lock-step warp and thread-block emulation for running the LP solvers on a CPU.
//
// When LPLB_HOST_SIM is defined, lp_solver.cuh and lp_block_solver.cuh compile as plain
// C++: the CUDA function qualifiers vanish and the intrinsics they use (__shfl_sync,
// __shfl_xor_sync, __all_sync, __syncwarp, __syncthreads, a named barrier) are served by
// host threads that meet at a barrier on every intrinsic.  A warp is 32 threads; a block
// (run_block) is a set of warps that also share a block-wide and a named barrier, with
// "shared memory" being an ordinary buffer that the caller passes in.  This works because
// the solvers are written so that all threads that take part in an intrinsic issue the
// same sequence of them.  The CPU test-suite uses it to check the exact device arithmetic
// against the float64 oracle without a GPU: a shuffle or barrier behind a thread-dependent
// condition shows up as a deadlock here, before any GPU run.  It has no counterpart in the
// reference.
#pragma once
#ifdef LPLB_HOST_SIM

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#define __device__
#define __host__
#define __forceinline__ inline
#define __noinline__
#define __global__

namespace lplb_sim {

class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    std::unique_lock<std::mutex> lk(m_);
    const uint64_t gen = gen_;
    if (++count_ == n_) {
      count_ = 0;
      ++gen_;
      cv_.notify_all();
    } else {
      cv_.wait(lk, [&] { return gen_ != gen; });
    }
  }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  int n_, count_ = 0;
  uint64_t gen_ = 0;
};

struct Warp {
  Barrier barrier{32};
  uint64_t slot[32];
  int pred[32];
};

// Barriers of a thread block: all threads, and the first `named_count` threads.
struct Block {
  explicit Block(int n_threads) : all(n_threads) {}
  Barrier all;
  std::mutex m;
  std::unique_ptr<Barrier> named;
  int named_count = 0;
  Barrier& named_barrier(int count) {
    std::lock_guard<std::mutex> lk(m);
    if (!named || named_count != count) {
      named = std::make_unique<Barrier>(count);
      named_count = count;
    }
    return *named;
  }
};

inline thread_local Warp* g_warp = nullptr;
inline thread_local int g_lane = 0;
inline thread_local Block* g_block = nullptr;

template <typename T>
inline T exchange(T v, int src_lane) {
  static_assert(sizeof(T) <= 8, "shuffle payload");
  uint64_t raw = 0;
  std::memcpy(&raw, &v, sizeof(T));
  g_warp->slot[g_lane] = raw;
  g_warp->barrier.wait();
  raw = g_warp->slot[src_lane & 31];
  g_warp->barrier.wait();
  T out;
  std::memcpy(&out, &raw, sizeof(T));
  return out;
}

// Run fn(lane) on 32 lock-stepped lanes.
inline void run_warp(const std::function<void(int)>& fn) {
  Warp warp;
  std::vector<std::thread> lanes;
  for (int l = 0; l < 32; ++l)
    lanes.emplace_back([&, l] {
      g_warp = &warp;
      g_lane = l;
      fn(l);
    });
  for (auto& t : lanes) t.join();
}

// Run fn(tid) on n_threads (a multiple of 32) lock-stepped threads forming one thread block.
inline void run_block(int n_threads, const std::function<void(int)>& fn) {
  const int n_warps = n_threads / 32;
  std::vector<std::unique_ptr<Warp>> warps;
  for (int w = 0; w < n_warps; ++w) warps.push_back(std::make_unique<Warp>());
  Block block(n_threads);
  std::vector<std::thread> threads;
  for (int t = 0; t < n_threads; ++t)
    threads.emplace_back([&, t] {
      g_warp = warps[t / 32].get();
      g_lane = t % 32;
      g_block = &block;
      fn(t);
    });
  for (auto& t : threads) t.join();
}

}  // namespace lplb_sim

inline void __syncwarp() { lplb_sim::g_warp->barrier.wait(); }
inline void __syncthreads() { lplb_sim::g_block->all.wait(); }
// Barrier among the first `count` threads of the block (bar.sync 1, count on the device).
inline void lplb_sim_named_barrier(int count) { lplb_sim::g_block->named_barrier(count).wait(); }

template <typename T>
inline T __shfl_sync(unsigned, T v, int src, int width = 32) {
  const int base = lplb_sim::g_lane / width * width;
  return lplb_sim::exchange(v, base + (src % width + width) % width);
}
template <typename T>
inline T __shfl_xor_sync(unsigned, T v, int mask, int width = 32) {
  const int base = lplb_sim::g_lane / width * width;
  const int src = (lplb_sim::g_lane - base) ^ mask;
  return lplb_sim::exchange(v, src < width ? base + src : lplb_sim::g_lane);
}
inline int __all_sync(unsigned, int pred) {
  lplb_sim::g_warp->pred[lplb_sim::g_lane] = pred;
  lplb_sim::g_warp->barrier.wait();
  int all = 1;
  for (int l = 0; l < 32; ++l) all &= lplb_sim::g_warp->pred[l] != 0;
  lplb_sim::g_warp->barrier.wait();
  return all;
}
inline int __any_sync(unsigned, int pred) {
  lplb_sim::g_warp->pred[lplb_sim::g_lane] = pred;
  lplb_sim::g_warp->barrier.wait();
  int any = 0;
  for (int l = 0; l < 32; ++l) any |= lplb_sim::g_warp->pred[l] != 0;
  lplb_sim::g_warp->barrier.wait();
  return any;
}
inline double rsqrt(double x) { return 1.0 / std::sqrt(x); }
inline float __fdividef(float a, float b) { return a / b; }

#endif  // LPLB_HOST_SIM
