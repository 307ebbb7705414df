// CPU build of the warp-level and thread-block LP solvers (see host_sim.h): C entry points
// for ctypes.  Compiled with -DLPLB_HOST_SIM by the CPU tests; not part of the GPU extension.
#define LPLB_HOST_SIM 1
#include "lp_block_solver.cuh"
#include "lp_solver.cuh"

namespace {

template <int GP, int D>
void solve_batch(int g, const int* r2o, const int* o2r, int nb, const double* w, const double* fixed, int max_iters,
                 double tol, double* f_out, int* iters, int* converged, double* anchor, int* anchor_valid,
                 double guard, double snap_mu) {
  constexpr int kSeg = 32 / GP;
  for (int b0 = 0; b0 < nb; b0 += kSeg) {
    lplb_sim::run_warp([&](int lane) {
      const int seg = lane / GP, li = lane % GP, b = b0 + seg;
      const bool live = b < nb && li < g;
      double wl[D], f[D], fx = 0.0;
      int src[D], dst[D];
      for (int d = 0; d < D; ++d) {
        wl[d] = 0.0;
        src[d] = dst[d] = li;
      }
      if (live) {
        fx = fixed[(size_t)b * g + li];
        for (int d = 0; d < D; ++d) {
          wl[d] = w[((size_t)b * g + li) * D + d];
          src[d] = r2o[li * D + d];
          dst[d] = o2r[li * D + d];
        }
      }
      lplb::IpmParams prm{max_iters, tol, anchor, anchor_valid, guard, snap_mu};
      double* slot = live && anchor ? anchor + ((size_t)b * g + li) * (4 * D + 3) : nullptr;
      int* flag = live && anchor ? anchor_valid + b : nullptr;
      const lplb::IpmOutcome res = lplb::ipm_solve_segment<GP, D>(li, wl, fx, src, dst, prm, f, slot, flag);
      if (live) {
        for (int d = 0; d < D; ++d) f_out[((size_t)b * g + li) * D + d] = f[d];
        if (li == 0) {
          iters[b] = res.iters;
          converged[b] = res.converged ? 1 : 0;
        }
      }
    });
  }
}

// The thread-block solver, one emulated CTA of kBlkThreads threads per instance.  DP >= d is the
// instantiated replica count; slots d..DP-1 are padded with self edges of weight zero, which is
// how the GPU launcher runs replica counts without an instantiation of their own.
template <int DP>
void solve_batch_block(int g, int d, const int* r2o, const int* o2r, int nb, const double* w, const double* fixed,
                       int max_iters, double tol, double* f_out, int* iters, int* converged, double* anchor,
                       int* anchor_valid, double guard, double snap_mu) {
  std::vector<double> scratch(lplb::blk_layout(g, DP).total);
  for (int b = 0; b < nb; ++b) {
    lplb_sim::run_block(lplb::kBlkThreads, [&](int tid) {
      const bool live = tid < g;
      double wl[DP], f[DP], fx = 0.0;
      int src[DP], dst[DP];
      for (int k = 0; k < DP; ++k) {
        wl[k] = 0.0;
        src[k] = dst[k] = tid;
      }
      if (live) {
        fx = fixed[(size_t)b * g + tid];
        for (int k = 0; k < d; ++k) {
          wl[k] = w[((size_t)b * g + tid) * d + k];
          src[k] = r2o[tid * d + k];
          dst[k] = o2r[tid * d + k];
        }
      }
      lplb::IpmParams prm{max_iters, tol, anchor, anchor_valid, guard, snap_mu};
      double* slot = live && anchor ? anchor + ((size_t)b * g + tid) * (4 * DP + 3) : nullptr;
      int* flag = live && anchor ? anchor_valid + b : nullptr;
      const lplb::IpmOutcome res =
          lplb::ipm_solve_block<DP>(tid, g, wl, fx, src, dst, prm, f, slot, flag, scratch.data());
      if (live) {
        for (int k = 0; k < d; ++k) f_out[((size_t)b * g + tid) * d + k] = f[k];
        if (tid == 0) {
          iters[b] = res.iters;
          converged[b] = res.converged ? 1 : 0;
        }
      }
    });
  }
}

}  // namespace

// Thread-block solver for any group size up to kBlkMaxGroup and up to 8 replicas per rank.
// anchor [nb][g][4*DP+3] with DP = d for d <= 4, else 8; null for cold solves only.
extern "C" int lplb_sim_solve_block(int g, int d, const int* r2o, const int* o2r, int nb, const double* w,
                                    const double* fixed, int max_iters, double tol, double* f_out, int* iters,
                                    int* converged, double* anchor, int* anchor_valid, double guard, double snap_mu) {
  if (g < 1 || g > lplb::kBlkMaxGroup || d < 1 || d > 8) return 1;
#define LPLB_CASE(DP_)                                                                                          \
  if ((d <= 4 ? d : 8) == DP_) {                                                                                \
    solve_batch_block<DP_>(g, d, r2o, o2r, nb, w, fixed, max_iters, tol, f_out, iters, converged, anchor,       \
                           anchor_valid, guard, snap_mu);                                                       \
    return 0;                                                                                                   \
  }
  LPLB_CASE(1) LPLB_CASE(2) LPLB_CASE(3) LPLB_CASE(4) LPLB_CASE(8)
#undef LPLB_CASE
  return 1;
}

// anchor [nb][g][4*d+3] and anchor_valid [nb] may be null (cold solves only).
extern "C" int lplb_sim_solve_warm(int g, int d, const int* r2o, const int* o2r, int nb, const double* w,
                                   const double* fixed, int max_iters, double tol, double* f_out, int* iters,
                                   int* converged, double* anchor, int* anchor_valid, double guard, double snap_mu) {
  const int gp = g <= 8 ? 8 : (g <= 16 ? 16 : 32);
#define LPLB_CASE(GP_, D_)                                                                             \
  if (gp == GP_ && d == D_) {                                                                          \
    solve_batch<GP_, D_>(g, r2o, o2r, nb, w, fixed, max_iters, tol, f_out, iters, converged, anchor,   \
                         anchor_valid, guard, snap_mu);                                                  \
    return 0;                                                                                          \
  }
  LPLB_CASE(8, 1) LPLB_CASE(8, 2) LPLB_CASE(8, 4) LPLB_CASE(16, 2) LPLB_CASE(32, 2) LPLB_CASE(32, 1)
#undef LPLB_CASE
  return 1;
}

extern "C" int lplb_sim_solve(int g, int d, const int* r2o, const int* o2r, int nb, const double* w,
                              const double* fixed, int max_iters, double tol, double* f_out, int* iters,
                              int* converged) {
  return lplb_sim_solve_warm(g, d, r2o, o2r, nb, w, fixed, max_iters, tol, f_out, iters, converged, nullptr, nullptr,
                             0.05, 1e-3);
}
