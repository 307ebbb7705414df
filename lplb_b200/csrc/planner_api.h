// Host-side launch interface of the planner kernels.  Plain C++ with raw device pointers
// and a stream so that the CUDA translation units do not need the torch headers; the
// pybind layer (binding.cpp) owns tensors, shapes and allocation.
//
// Counterpart of the launchers in the reference's csrc/plugin.cpp:491-660.  There is no
// run-time compiler here: every (group size, replicas per rank) shape is instantiated
// ahead of time for sm_100a, which removes the NVRTC/nvJitLink/disk-cache machinery of
// reference csrc/plugin.cpp:149-352.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lplb {

struct TopoDesc {
  const int* r2o;
  const int* o2r;
  const int* phy2log;
  const int* log2phy;
  const int* log2edge;
  const int* log2slot;  // [E] rank * (d + 1) + bundle of the expert (d = the rank's non-replicated ones)
  int n_group, g, d, ll, c;
};

struct ExchangeDesc {
  unsigned long long* const* recv;  // device array of n_ranks pointers (nullptr when n_ranks == 1);
                                    // each points at that rank's uint64[2][2][n_ranks][E] receive buffer
  int n_ranks;
  int my_rank;
  int node_size;                    // two-level schedule over nodes of this many ranks; 0 = one level
  unsigned long long timeout_ns;
};

struct SolveParams {
  int max_iters;
  double tol;
  double* anchor = nullptr;      // warm-start state [n_group][G][4 * DP + 3] (DP = anchor_dup(d)), or null
  int* anchor_valid = nullptr;   // [n_group]
  double guard = 0.05;
  double snap_mu = 1e-3;
  int solver = 0;                // kSolverAuto / kSolverWarp / kSolverBlock
};

// Two device solvers.  The warp solver keeps a group of up to 32 ranks (up to 4 replicas per
// rank) in one warp's registers; the thread-block solver takes any group of up to
// kMaxGroupSize ranks with up to kMaxDup replicas per rank, its matrix in shared memory.
// kSolverAuto picks the warp solver for groups of up to 8 ranks and the block solver above.
enum SolverKind : int { kSolverAuto = 0, kSolverWarp = 1, kSolverBlock = 2 };
constexpr int kMaxWarpGroupSize = 32;
constexpr int kMaxWarpDup = 4;
constexpr int kMaxGroupSize = 128;
constexpr int kMaxDup = 8;
constexpr int kMaxLogicalExperts = 8192;

// The solver that `requested` resolves to for this shape, or -1 when no device solver fits.
int resolve_solver(int g, int d, int requested);
// Replica slots per rank in the warm-start state for this shape and solver.
int anchor_dup(int g, int d, int requested);

size_t planner_workspace_bytes(int n_logical);
inline size_t exchange_buffer_bytes(int n_ranks, int n_logical) { return sizeof(unsigned long long) * 4 * (size_t)n_ranks * n_logical; }

// idx_is64: 1 for int64 indices, 0 for int32.  All functions return a cudaError_t from the
// launch (cudaSuccess when enqueued); cudaErrorInvalidValue for unsupported shapes.
cudaError_t launch_count(const void* idx, int idx_is64, long long n, int n_logical, int n_cta, int* by_cta,
                         void* workspace, int* status, cudaStream_t stream);

cudaError_t launch_solve(const int* workload, const TopoDesc& topo, SolveParams prm, float* probs, float* normalised,
                         void* avail, int avail_is64, int* status, cudaStream_t stream);

cudaError_t launch_redirect(const void* idx, int idx_is64, long long n, const float* probs, const int* by_cta,
                            const TopoDesc& topo, int n_cta, void* out, cudaStream_t stream);

// Sum int32[E] counts over the peers of `ex` (in-kernel push over NVLink peer memory).
cudaError_t launch_exchange(const int* in, int n_logical, const ExchangeDesc& ex, void* workspace, int* out,
                            int* status, cudaStream_t stream);

// Single-launch count + exchange + solve + redirect.  n_cta >= 2: CTA 0 exchanges and solves,
// the other n_cta - 1 CTAs count and redirect.  Cooperative launch: n_cta must not exceed
// max_fused_ctas().  `trace` (may be null) receives 8 globaltimer stamps, see the kernel.
// cooperative = 0 uses an ordinary launch: no co-residency guarantee from the driver, so the
// caller must know the GPU has room for n_cta CTAs (the in-kernel waits stay bounded).
cudaError_t launch_fused(const void* idx, int idx_is64, long long n, const TopoDesc& topo, const ExchangeDesc& ex,
                         SolveParams prm, void* workspace, float* probs, void* avail, int avail_is64, int* status,
                         void* out, int n_cta, unsigned long long grid_timeout_ns, unsigned long long* trace,
                         int cooperative, cudaStream_t stream);

// Co-resident CTA limit of the fused kernel for this topology on the current device (0 when the
// shape has no device solver or its tables do not fit shared memory).
int max_fused_ctas(const TopoDesc& topo, int solver, int idx_is64);

}  // namespace lplb
