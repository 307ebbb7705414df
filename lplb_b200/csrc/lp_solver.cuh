// Warp-level interior-point solver for the per-group balancing LP (sm_100a).
//
//   min t  s.t.  base_i + sum_k M[i,k] f_k <= t,  0 <= f <= 1
//
// One LP group of G <= GP ranks is solved by GP consecutive lanes of a warp; a warp
// therefore carries 32/GP independent groups at once.  Lane i is rank i and owns the D
// edges (i, d): the replicated bundles whose origin is rank i.  All cross-rank traffic
// is warp shuffles with segment width GP, nothing goes through shared memory and there
// is no block barrier inside the iteration.
//
// The method is a Mehrotra predictor-corrector primal-dual iteration in float64 on the
// compact form.  The normal matrix N = M diag(theta) M^T + diag(s/y) is a weighted
// graph Laplacian of the topology plus a positive diagonal, GP x GP, factored as L D L^T
// (no square roots).  For GP = 16 and 32 lane i keeps row i in registers and the
// factorisation updates both triangles, so that after step j lane j already holds column j
// of L and both substitutions run with statically indexed registers.  For GP = 8 the 36
// entries are all-gathered and every lane factors and solves the whole system itself.
//
// It replaces the reference's primal affine-scaling loop on the (G+GD) x (2GD+G+2)
// equality form with cuBLASDx/cuSolverDx block calls
// (reference lplb/resources/csrc-tmpl/minilp.cu:28-59 and :323-401): a 24x24 system
// shrinks to 8x8 for the Cube, 96x96 to 32x32 for the 8x4 torus, the start point is
// feasible without a big-M column, and the loop stops on a duality-gap test instead of
// after a fixed five steps.
#pragma once

#ifdef LPLB_HOST_SIM
#include "host_sim.h"
#else
#include <cuda_runtime.h>
#endif
#include <math.h>

namespace lplb {

struct IpmParams {
  int max_iters;   // hard cap on iterations
  double tol;      // relative duality gap and feasibility target
  // Warm start (optional).  `anchor` holds, per group and rank, a well-centred iterate
  // (complementarity about `snap_mu`) saved by the last cold solve: f, v, z, q per bundle, then
  // s, y, t.  A solve starts from it when the new data leave it nearly primal feasible (largest
  // row residual <= `guard`, in units of the mean rank load), which is the case while
  // consecutive batches come from the same distribution; otherwise it starts cold and
  // replaces the anchor.  Null = always cold.
  double* anchor = nullptr;  // [n_group][G][4 * D + 3]
  int* anchor_valid = nullptr;  // [n_group]
  double guard = 0.05;
  double snap_mu = 1e-3;
  // Rehearsal (optional): a solve on made-up data whose only purpose is to pull the solver's
  // code into the instruction caches before the real statistics are there.  It leaves at the
  // next check after `*stop` (a word in shared memory that another warp sets) becomes
  // non-zero.  Null for every real solve.
  const volatile int* stop = nullptr;
};

struct IpmOutcome {
  int iters;
  bool converged;
  bool finite;
  double gap;
};

// Mask of the first n lanes of a warp.
__host__ __device__ constexpr unsigned first_lanes(int n) { return n >= 32 ? 0xffffffffu : (1u << (n & 31)) - 1u; }

// `lanes` in all of these: the lanes that execute the call (whole segments).
template <int GP>
__device__ __forceinline__ double seg_shfl(unsigned lanes, double v, int src) {
  return __shfl_sync(lanes, v, src, GP);
}
template <int GP>
__device__ __forceinline__ double seg_sum(unsigned lanes, double v) {
#pragma unroll
  for (int o = GP / 2; o > 0; o >>= 1) v += __shfl_xor_sync(lanes, v, o, GP);
  return v;
}
template <int GP>
__device__ __forceinline__ double seg_max(unsigned lanes, double v) {
#pragma unroll
  for (int o = GP / 2; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(lanes, v, o, GP));
  return v;
}
template <int GP>
__device__ __forceinline__ float seg_minf(unsigned lanes, float v) {
#pragma unroll
  for (int o = GP / 2; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(lanes, v, o, GP));
  return v;
}

// Largest step in [0, +inf) that keeps val + a*dval >= 0, as a float (the 0.995 safety
// fraction applied by the caller dwarfs the rounding of this ratio).
__device__ __forceinline__ float ratio_to_bound(double val, double dval) {
  return dval < 0.0 ? __fdividef((float)val, -(float)dval) : 3.0e38f;
}

// 1/x for a positive, finite double: the hardware's ~2^-23 approximation refined by two
// Newton steps (error squared each time), five dependent instructions instead of the
// forty-odd of an IEEE division.  Relative error is a few ulp, far below the solver's needs.
__device__ __forceinline__ double fast_rcp(double x) {
#ifdef LPLB_HOST_SIM
  return 1.0 / x;
#else
  double r;
  asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(x));
  r = fma(r, fma(-x, r, 1.0), r);
  r = fma(r, fma(-x, r, 1.0), r);
  return r;
#endif
}

// ---- distributed factorisation (any GP): lane i keeps row i ---------------------------------
// N = L D L^T with unit lower L.  Both triangles of the trailing matrix are kept current, so
// after step j lane j can read column j of L out of its own row by symmetry.  On return, on
// lane i: row[j<i] = L[i][j], row[i] = 1/D[i], row[j>i] = L[j][i].  A pivot
// that rounding drove non-positive or non-finite is replaced by a huge one, which zeroes that
// unknown in the solves instead of spreading NaNs.  Updates are masked multiplies, not
// branches, and the loop body is two shuffles, one FMA and one multiply per entry: the
// unrolled code of an iteration is close to the instruction cache's size at GP = 32, where
// the measured time moves by +-25 % with the code's size and layout.
template <int GP>
__device__ __forceinline__ void ldl_factor_rows(unsigned lanes, double (&row)[GP], int li) {
#pragma unroll
  for (int j = 0; j < GP; ++j) {
    double piv = seg_shfl<GP>(lanes, row[j], j);
    if (!(piv > 1e-300) || !(piv < 1e300)) piv = 1e300;
    const double dinv = fast_rcp(piv);
    const double lij = li > j ? row[j] * dinv : 0.0;  // L[i][j] on lanes below the pivot, else 0
    // Lane j's own trailing entries are untouched by the update (its lij is 0); scaling them
    // by 1/D[j] leaves L[k][j] there for the backward sweep.  Every other lane scales by 1.
    const double scale = li == j ? dinv : 1.0;
#pragma unroll
    for (int k = j + 1; k < GP; ++k) {
      const double u = seg_shfl<GP>(lanes, row[k], j);  // unscaled N[j][k] = N[k][j]
      row[k] = fma(-lij, u, row[k]) * scale;
    }
    row[j] = li > j ? lij : (li == j ? dinv : row[j]);
  }
}

// Solve L D L^T x = g for NRHS (1 or 2) right-hand sides held one element per lane.
template <int GP, int NRHS>
__device__ __forceinline__ void ldl_solve_rows(unsigned lanes, const double (&row)[GP], int li, double& g0, double& g1) {
#pragma unroll
  for (int j = 0; j < GP; ++j) {
    const double l = li > j ? row[j] : 0.0;
    g0 = fma(-l, seg_shfl<GP>(lanes, g0, j), g0);
    if constexpr (NRHS == 2) g1 = fma(-l, seg_shfl<GP>(lanes, g1, j), g1);
  }
  {
    double dinv = row[0];
#pragma unroll
    for (int j = 1; j < GP; ++j) dinv = li == j ? row[j] : dinv;
    g0 *= dinv;
    if constexpr (NRHS == 2) g1 *= dinv;
  }
#pragma unroll
  for (int j = GP - 1; j >= 0; --j) {
    const double l = li < j ? row[j] : 0.0;
    g0 = fma(-l, seg_shfl<GP>(lanes, g0, j), g0);
    if constexpr (NRHS == 2) g1 = fma(-l, seg_shfl<GP>(lanes, g1, j), g1);
  }
}

// ---- replicated factorisation (GP == 8): every lane factors the whole 8x8 matrix -----------
// The 36 entries of the lower triangle are all-gathered with shuffles, after which the
// factorisation and the substitutions are straight-line FMA code with static register
// indices: no shuffle latency on the dependent chain, no predication.
struct Ldl8 {
  double a[36];    // lower triangle, row-major packed: (i, k) at i*(i+1)/2 + k; L below, unused on the diagonal
  double dinv[8];  // 1/D
  __device__ __forceinline__ static constexpr int at(int i, int k) { return i * (i + 1) / 2 + k; }
};

__device__ __forceinline__ void ldl8_factor(unsigned lanes, const double (&row)[8], Ldl8& m) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int k = 0; k <= i; ++k) m.a[Ldl8::at(i, k)] = seg_shfl<8>(lanes, row[k], i);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    double piv = m.a[Ldl8::at(j, j)];
    if (!(piv > 1e-300) || !(piv < 1e300)) piv = 1e300;
    m.dinv[j] = fast_rcp(piv);
#pragma unroll
    for (int i = j + 1; i < 8; ++i) {
      const double lij = m.a[Ldl8::at(i, j)] * m.dinv[j];
#pragma unroll
      for (int k = j + 1; k <= i; ++k) m.a[Ldl8::at(i, k)] = fma(-lij, m.a[Ldl8::at(k, j)], m.a[Ldl8::at(i, k)]);
    }
#pragma unroll
    for (int i = j + 1; i < 8; ++i) m.a[Ldl8::at(i, j)] *= m.dinv[j];
  }
}

__device__ __forceinline__ double ldl8_solve(unsigned lanes, const Ldl8& m, int li, double g) {
  double b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) b[k] = seg_shfl<8>(lanes, g, k);
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = j + 1; i < 8; ++i) b[i] = fma(-m.a[Ldl8::at(i, j)], b[j], b[i]);
#pragma unroll
  for (int j = 0; j < 8; ++j) b[j] *= m.dinv[j];
#pragma unroll
  for (int j = 7; j >= 0; --j)
#pragma unroll
    for (int i = 0; i < j; ++i) b[i] = fma(-m.a[Ldl8::at(j, i)], b[j], b[i]);
  double x = b[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) x = li == k ? b[k] : x;
  return x;
}

// The lanes in `lanes` (whole segments of GP lanes) call this together, no others.  `li` is the
// lane's index inside its segment.
// Always inlined into its caller: left to the compiler, the decision changed from build to build
// with unrelated edits elsewhere in the translation unit, and a solve ran 2 to 4 us slower
// whenever the function ended up out of line.
//   w[d]      load of own bundle d (any non-negative unit)
//   fixed     load of the lane's non-replicated experts (same unit)
//   src[d]    segment lane whose bundle d this rank holds a replica of  (r2o[i][d])
//   dst[d]    segment lane that holds the replica of own bundle d       (o2r[i][d])
// Padding lanes (rank >= G) pass w = 0, fixed = 0, src = dst = li.
// Returns the shares f[d] of own bundles kept on the origin, clamped to [0, 1].
// `anchor` / `anchor_valid`: this lane's slot of the warm-start state and its group's flag
// (both null when warm starts are off or the lane is padding).
template <int GP, int D>
__device__ __forceinline__ IpmOutcome ipm_solve_segment(int li, const double (&w_in)[D], double fixed, const int (&src_in)[D],
                                                        const int (&dst_in)[D], const IpmParams prm,
                                                        double (&f_out)[D], double* anchor = nullptr,
                                                        int* anchor_valid = nullptr, const unsigned lanes = 0xffffffffu) {
  constexpr double kEta = 0.995;
  constexpr int kComp = GP + 2 * GP * D;
  constexpr double kInvComp = 1.0 / kComp;
  // Private copies: when this function is not inlined the caller's arrays live in local memory,
  // and every use in the loop would be a load that has to be repeated after each store.
  int src[D], dst[D];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    src[d] = src_in[d];
    dst[d] = dst_in[d];
  }

  // The saved iterate is read first, valid or not (the slot is always allocated): its loads and
  // the load of the flag are in flight while the scaling and the cold start point are computed.
  double fa[D], va[D], za[D], qa[D], sa = 1.0, ya = 1.0 / GP, ta = 0.0;
  const bool slot = anchor != nullptr && anchor_valid != nullptr;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    fa[d] = slot ? anchor[d] : 0.5;
    va[d] = slot ? anchor[D + d] : 0.5;
    za[d] = slot ? anchor[2 * D + d] : 1.0;
    qa[d] = slot ? anchor[3 * D + d] : 1.0;
  }
  if (slot) {
    sa = anchor[4 * D];
    ya = anchor[4 * D + 1];
    ta = anchor[4 * D + 2];
  }
  const bool have = slot && *anchor_valid != 0;

  // ---- scale so that the mean rank load is 1 ---------------------------------------
  double mine = fixed;
#pragma unroll
  for (int d = 0; d < D; ++d) mine += w_in[d];
  const double total = seg_sum<GP>(lanes, mine);
  IpmOutcome out{0, true, true, 0.0};
  // A segment with no load at all (also: a segment past the last group) must still walk
  // through every shuffle below with the rest of the warp, so it is not returned early:
  // it starts out `done`, computes on harmless zeros and reports f = 1 at the end.
  const bool empty = !(total > 0.0);
  const double inv_scale = empty ? 0.0 : (double)GP * fast_rcp(total);
  double w[D], base = fixed * inv_scale;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    w[d] = w_in[d] * inv_scale;
    base += seg_shfl<GP>(lanes, w[d], src[d]);
  }
  // A self edge (origin == holder; also every padding lane) moves no load: its column
  // of M is zero.  Its load is already part of `base`, so drop the weight.
#pragma unroll
  for (int d = 0; d < D; ++d)
    if (dst[d] == li) w[d] = 0.0;

  auto m_times = [&](const double(&x)[D]) -> double {  // (M x)_i
    double acc = 0.0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      const double wx = w[d] * x[d];
      acc += wx - seg_shfl<GP>(lanes, wx, src[d]);
    }
    return acc;
  };

  // ---- warm start from the anchor, if it still fits the data -----------------------------
  // The decision is taken per segment; lanes without a slot (padding) follow their segment.
  if (!have) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
      fa[d] = va[d] = 0.5;
      za[d] = qa[d] = 1.0;
    }
    sa = 1.0;
    ya = 1.0 / GP;
    ta = 0.0;
  }
  const double mfa = m_times(fa);  // shuffles inside: every lane takes part, with or without a slot
  const double rp = have ? fabs(ta - base - mfa - sa) : 0.0;
  // every reduction below is executed by all calling lanes, whatever their segment decides
  const bool seg_has = seg_max<GP>(lanes, have ? 1.0 : 0.0) > 0.0;
  const double rp_max = seg_max<GP>(lanes, rp);
  const double t_anchor = seg_max<GP>(lanes, have ? ta : -1e300);
  const bool fits = seg_has && !empty && rp_max <= prm.guard;
  const bool cold = !fits;

  // ---- start point -------------------------------------------------------------------------
  // The feasible cold start costs four reductions; it is skipped when every calling lane takes
  // its start from the anchor (the usual case from the second batch on).
  double f[D], v[D], z[D], q[D], t = t_anchor, s = sa, y = ya;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    f[d] = fa[d];
    v[d] = va[d];
    z[d] = za[d];
    q[d] = qa[d];
  }
  if (!__all_sync(lanes, fits && have)) {
    double cf[D];
#pragma unroll
    for (int d = 0; d < D; ++d) cf[d] = 0.5;
    const double load = base + m_times(cf);
    const double lmax = seg_max<GP>(lanes, load), lmin = -seg_max<GP>(lanes, -load);
    const double ct = lmax + 0.5 * (lmax - lmin) + 0.05;
    const double cs = ct - load;
    const double mu0 = seg_sum<GP>(lanes, cs * (1.0 / GP)) / GP;
    if (!(fits && have)) {  // this lane starts cold (its segment does, or it is a padding lane)
#pragma unroll
      for (int d = 0; d < D; ++d) {
        f[d] = v[d] = 0.5;
        z[d] = q[d] = 2.0 * mu0;
      }
      s = cs;
      y = 1.0 / GP;
    }
    if (!fits) t = ct;
  }
  bool saved = false;

  bool done = empty;
  int iters = 0;
  double gap = 1e300, gap_scale = 1.0;

  // one shared-memory read for the whole warp, so every lane takes the same way out
  auto told_to_stop = [&]() -> bool { return prm.stop != nullptr && __any_sync(lanes, *prm.stop != 0); };
  bool halted = false;

  for (int it = 0; it <= prm.max_iters; ++it) {
    if (told_to_stop()) break;
    // ---- residuals, gap, stopping test ---------------------------------------------
    const double mf = m_times(f);
    const double r_p = t - base - mf - s;
    double r_u[D], r_d[D];
    double comp = s * y, dual_part = y * base, neg_rd = 0.0, worst_u = 0.0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      r_u[d] = 1.0 - f[d] - v[d];
      r_d[d] = z[d] - q[d] - w[d] * (y - seg_shfl<GP>(lanes, y, dst[d]));
      comp += z[d] * f[d] + q[d] * v[d];
      dual_part -= q[d];
      neg_rd += fmin(r_d[d], 0.0);
      worst_u = fmax(worst_u, fabs(r_u[d]));
    }
    const double mu = seg_sum<GP>(lanes, comp) * kInvComp;  // a division costs some 300 cycles per evaluation
    const double r_t = 1.0 - seg_sum<GP>(lanes, y);
    const double primal = seg_max<GP>(lanes, base + mf);
    const double dual = seg_sum<GP>(lanes, dual_part + neg_rd);
    const double infeas = fmax(seg_max<GP>(lanes, worst_u), fabs(r_t));
    if (!done) {
      gap = primal - dual;  // absolute here, made relative once at the end
      gap_scale = fabs(primal);
      // at mu ~ 1e-13 the iterate is optimal to machine precision: stop instead of dividing by it
      if ((gap <= prm.tol * gap_scale && infeas <= prm.tol) || mu <= 1e-13) done = true;
    }
    // A cold solve leaves its first iterate at or below snap_mu behind as the next anchor.
    if (cold && !saved && !empty && anchor != nullptr && mu <= prm.snap_mu) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        anchor[d] = f[d];
        anchor[D + d] = v[d];
        anchor[2 * D + d] = z[d];
        anchor[3 * D + d] = q[d];
      }
      anchor[4 * D] = s;
      anchor[4 * D + 1] = y;
      anchor[4 * D + 2] = t;
      if (li == 0 && anchor_valid != nullptr) *anchor_valid = 1;
      saved = true;
    }
    // Every segment of the warp has to leave the loop together.
    if (__all_sync(lanes, done) || it == prm.max_iters) break;
    if (!done) ++iters;
    if (told_to_stop()) break;

    // ---- normal matrix row -----------------------------------------------------------
    double inv_f[D], inv_v[D], theta[D], cw[D];
    const double inv_y = fast_rcp(y);
    const double inv_mu = fast_rcp(kComp * mu);
#pragma unroll
    for (int d = 0; d < D; ++d) {
      inv_f[d] = fast_rcp(f[d]);
      inv_v[d] = fast_rcp(v[d]);
      theta[d] = fast_rcp(z[d] * inv_f[d] + q[d] * inv_v[d]);
      cw[d] = theta[d] * w[d] * w[d];
    }
    double row[GP];
    {
      double diag = s * inv_y;
      double held[D];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        held[d] = seg_shfl<GP>(lanes, cw[d], src[d]);
        diag += cw[d] + held[d];
      }
#pragma unroll
      for (int j = 0; j < GP; ++j) {
        double e = (j == li) ? diag : 0.0;
#pragma unroll
        for (int d = 0; d < D; ++d) {
          e -= (dst[d] == j) ? cw[d] : 0.0;
          e -= (src[d] == j) ? held[d] : 0.0;
        }
        row[j] = e;
      }
    }

    if (told_to_stop()) break;
    // ---- factorisation -------------------------------------------------------------------
    Ldl8 dense;
    if constexpr (GP == 8) ldl8_factor(lanes, row, dense);
    else ldl_factor_rows<GP>(lanes, row, li);

    // ---- predictor (pass 0) and corrector (pass 1) share one body ------------------------
    // Pass 0 also solves N b = 1 for the border column that carries sum(dy) = r_t.
    double df[D], dv[D], dz[D], dq[D], ds = 0.0, dy = 0.0, dt = 0.0;
    double border = 1.0, inv_border_sum = 1.0, sm = 0.0;
#pragma unroll
    for (int d = 0; d < D; ++d) df[d] = dv[d] = dz[d] = dq[d] = 0.0;
    float apf = 0.f, adf = 0.f;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      if (told_to_stop()) {
        halted = true;
        break;
      }
      // complementarity targets: -XZe for the predictor, sigma*mu*e - XZe - dXdZe after it
      const double r_sy = sm - s * y - ds * dy;
      double r_zf[D], r_qv[D], rd_t[D];
      double acc = 0.0;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        r_zf[d] = sm - z[d] * f[d] - dz[d] * df[d];
        r_qv[d] = sm - q[d] * v[d] - dq[d] * dv[d];
        rd_t[d] = r_d[d] + r_zf[d] * inv_f[d] - (r_qv[d] - q[d] * r_u[d]) * inv_v[d];
        const double wx = w[d] * theta[d] * rd_t[d];
        acc += wx - seg_shfl<GP>(lanes, wx, src[d]);
      }
      double a = acc - r_p + r_sy * inv_y;
      if constexpr (GP == 8) {
        a = ldl8_solve(lanes, dense, li, a);
        if (pass == 0) border = ldl8_solve(lanes, dense, li, 1.0);
      } else {
        // One instantiation serves both passes (pass 1 carries a dummy second right-hand
        // side): at GP = 32 the unrolled iteration body is near the instruction cache's size
        // and a second copy of the substitution code costs more than the wasted FMAs.
        double b2 = pass == 0 ? 1.0 : 0.0;
        ldl_solve_rows<GP, 2>(lanes, row, li, a, b2);
        if (pass == 0) border = b2;
      }
      if (told_to_stop()) {
        halted = true;
        break;
      }
      if (pass == 0) inv_border_sum = fast_rcp(seg_sum<GP>(lanes, border));
      dt = (seg_sum<GP>(lanes, a) - r_t) * inv_border_sum;
      dy = a - dt * border;
      ds = (r_sy - s * dy) * inv_y;
      float rp = ratio_to_bound(s, ds), rd = ratio_to_bound(y, dy);
#pragma unroll
      for (int d = 0; d < D; ++d) {
        df[d] = theta[d] * (rd_t[d] - w[d] * (dy - seg_shfl<GP>(lanes, dy, dst[d])));
        dv[d] = r_u[d] - df[d];
        dz[d] = (r_zf[d] - z[d] * df[d]) * inv_f[d];
        dq[d] = (r_qv[d] - q[d] * dv[d]) * inv_v[d];
        rp = fminf(rp, fminf(ratio_to_bound(f[d], df[d]), ratio_to_bound(v[d], dv[d])));
        rd = fminf(rd, fminf(ratio_to_bound(z[d], dz[d]), ratio_to_bound(q[d], dq[d])));
      }
      apf = seg_minf<GP>(lanes, rp);
      adf = seg_minf<GP>(lanes, rd);
      if (pass == 0) {  // centring parameter from the affine step
        const double ap = fmin((double)apf, 1.0), ad = fmin((double)adf, 1.0);
        double comp_aff = (s + ap * ds) * (y + ad * dy);
#pragma unroll
        for (int d = 0; d < D; ++d)
          comp_aff += (z[d] + ad * dz[d]) * (f[d] + ap * df[d]) + (q[d] + ad * dq[d]) * (v[d] + ap * dv[d]);
        const double ratio = fmin(fmax(seg_sum<GP>(lanes, comp_aff) * inv_mu, 0.0), 1.0);
        sm = ratio * ratio * ratio * mu;
      }
    }
    if (halted) break;
    const double ap = fmin(kEta * (double)apf, 1.0), ad = fmin(kEta * (double)adf, 1.0);
    if (!done) {
      t += ap * dt;
      s += ap * ds;
      y += ad * dy;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        f[d] += ap * df[d];
        v[d] += ap * dv[d];
        z[d] += ad * dz[d];
        q[d] += ad * dq[d];
      }
    }
  }

  bool finite = true;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    finite = finite && (f[d] == f[d]) && fabs(f[d]) < 1e300;
    f_out[d] = fmin(fmax(f[d], 0.0), 1.0);
  }
  finite = seg_max<GP>(lanes, finite ? 0.0 : 1.0) == 0.0;
  if (!finite) {
#pragma unroll
    for (int d = 0; d < D; ++d) f_out[d] = 0.5;
  }
  if (empty) {  // nothing to balance: keep everything on the origin
#pragma unroll
    for (int d = 0; d < D; ++d) f_out[d] = 1.0;
    gap = 0.0;
  }
  out.iters = iters;
  out.converged = done && finite;
  out.finite = finite;
  out.gap = empty ? 0.0 : gap * fast_rcp(fmax(gap_scale, 1e-300));
  return out;
}

// Out-of-line entry for the 32-rank instantiation.  Inlined into a kernel, the 32-register-pair
// matrix row plus the caller's own state no longer fit the register file and the compiler
// moves the row to local memory, which costs an order of magnitude; as a separate function
// the solver gets the whole register budget to itself.  The smaller instantiations are inlined:
// out of line they measured about 2 us slower per solve.
template <int GP, int D>
__device__ __noinline__ IpmOutcome ipm_solve_segment_ool(int li, const double (&w_in)[D], double fixed,
                                                         const int (&src)[D], const int (&dst)[D],
                                                         const IpmParams prm, double (&f_out)[D], double* anchor,
                                                         int* anchor_valid, const unsigned lanes) {
  return ipm_solve_segment<GP, D>(li, w_in, fixed, src, dst, prm, f_out, anchor, anchor_valid, lanes);
}

}  // namespace lplb
