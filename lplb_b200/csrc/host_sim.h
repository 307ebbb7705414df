// Lock-step warp emulation for running the warp-level LP solver on a CPU.
//
// When LPLB_HOST_SIM is defined, lp_solver.cuh compiles as plain C++: the CUDA function
// qualifiers vanish and the warp intrinsics it uses (__shfl_sync, __shfl_xor_sync,
// __all_sync) are served by 32 host threads that meet at a barrier on every intrinsic.
// This works because the solver is written so that all 32 lanes issue the same sequence
// of intrinsics.  The CPU test-suite uses it to check the exact device arithmetic against
// the float64 oracle without a GPU.  It has no counterpart in the reference.
#pragma once
#ifdef LPLB_HOST_SIM

#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
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

inline thread_local Warp* g_warp = nullptr;
inline thread_local int g_lane = 0;

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

}  // namespace lplb_sim

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
inline double rsqrt(double x) { return 1.0 / std::sqrt(x); }
inline float __fdividef(float a, float b) { return a / b; }

#endif  // LPLB_HOST_SIM
