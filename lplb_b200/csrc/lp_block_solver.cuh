// Thread-block interior-point solver for LP groups of any size (sm_100a).
//
// Same LP, same Mehrotra predictor-corrector iteration and same warm-start rule as the warp
// solver in lp_solver.cuh, organised for groups that do not fit one warp's registers: the
// group size G is a run-time value (up to kBlkMaxGroup ranks), the G x G normal matrix lives
// in shared memory and one CTA of kBlkThreads threads solves one group.
//
//   * Thread i < G is rank i and keeps its D edges in registers; values that cross ranks go
//     through small shared-memory vectors followed by a barrier among the "row warps" only
//     (one __syncwarp for G <= 32, a named barrier otherwise).
//   * N = L D L^T is factored in 8 x 8 blocks, right-looking: the diagonal block is factored
//     in registers (straight-line code, as the warp solver does for an 8-rank group), the
//     panel below it is one thread per row, and the trailing update is spread over all
//     threads of the CTA.  Two block barriers per block column.
//   * The factorisation stores, instead of L itself, the products that make the triangular
//     solves short: W_k = L_kk^-1 for every diagonal block and L_ik W_k for every block below
//     it.  A forward or backward substitution is then one barrier and eight multiply-adds per
//     block column, whatever the rank's position, instead of one dependent step per rank.
//
// All loops over G are rolled; nothing is unrolled over the group size, so the code size does
// not grow with G (the warp solver's 32-rank instantiation is bound by its unrolled code).
//
// Replaces what the reference gets from cuBLASDx/cuSolverDx block calls for arbitrary
// GROUP_SIZE (reference lplb/resources/csrc-tmpl/minilp.cu:28-59, :323-367), on the compact
// G x G form instead of the (G + G D)^2 one.
#pragma once

#include "lp_solver.cuh"

namespace lplb {


constexpr int kBlkThreads = 256;
constexpr int kBlkWarps = kBlkThreads / 32;
constexpr int kBlkMaxGroup = 128;  // row threads fill at most half of the CTA's warps
constexpr int kPanelLd = 9;        // leading dimension of the 8-wide panels (odd: no bank conflicts)

// Shared-memory plan of one solve, in doubles from the start of the scratch area.
struct BlkLayout {
  int g, gp, gp32, ld, nb, r_warps;
  int mat, wblk, pl, px, dinv, gv, xv, xch, red, ctrl, total;
};

__host__ __device__ inline BlkLayout blk_layout(int g, int d) {
  BlkLayout l;
  l.g = g;
  l.gp = (g + 7) & ~7;      // matrix order: G rounded up to whole 8 x 8 blocks (padding rows are identity)
  l.gp32 = (g + 31) & ~31;  // threads that run the per-rank code: whole warps
  l.ld = l.gp + 1;          // odd leading dimension: a column walk by consecutive threads is conflict-free
  l.nb = l.gp >> 3;
  l.r_warps = l.gp32 >> 5;
  int o = 0;
  l.mat = o, o += l.gp * l.ld;         // lower triangle of N, then L_ik W_k below the diagonal blocks
  l.wblk = o, o += l.gp * kPanelLd;    // row r: W_k[r % 8][0..8), k = r / 8 (unit diagonal, zeros above)
  l.pl = o, o += l.gp * kPanelLd;      // current panel of L
  l.px = o, o += l.gp * kPanelLd;      // current panel of L D
  l.dinv = o, o += l.gp32;             // 1 / D
  l.gv = o, o += 2 * l.gp32;           // substitution vectors (two right-hand sides)
  l.xv = o, o += 2 * l.gp32;
  l.xch = o, o += (3 * d + 2) * l.gp32;  // per-rank values read by other ranks
  l.red = o, o += 2 * kBlkWarps * 8;   // cross-warp reductions, two alternating copies
  l.ctrl = o, o += 2;                  // int: "another iteration follows"
  l.total = o;
  return l;
}
__host__ __device__ inline size_t block_solver_smem_bytes(int g, int d) { return sizeof(double) * (size_t)blk_layout(g, d).total; }

// Barrier among the row warps.
__device__ __forceinline__ void rows_sync(int r_warps) {
#ifdef LPLB_HOST_SIM
  if (r_warps == 1) __syncwarp();
  else lplb_sim_named_barrier(r_warps * 32);
#else
  if (r_warps == 1) __syncwarp();
  else asm volatile("bar.sync 1, %0;" ::"r"(r_warps * 32) : "memory");
#endif
}

// Reduce K values over all row threads; bit k of MAXMASK selects max instead of sum.  Every row
// thread ends with bitwise identical results (a butterfly adds the same pairs on both sides,
// and the per-warp partials are combined in one order), which keeps decisions uniform.
template <int K, unsigned MAXMASK>
__device__ __forceinline__ void rows_reduce(double (&v)[K], const BlkLayout& l, double* sm, int warp, int lane,
                                            int& phase) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const double other = __shfl_xor_sync(0xffffffffu, v[k], o);
      v[k] = ((MAXMASK >> k) & 1u) ? fmax(v[k], other) : v[k] + other;
    }
  }
  if (l.r_warps > 1) {
    double* red = sm + l.red + phase * (kBlkWarps * 8);
    phase ^= 1;
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < K; ++k) red[warp * 8 + k] = v[k];
    }
    rows_sync(l.r_warps);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      double acc = red[k];
      for (int w = 1; w < l.r_warps; ++w) acc = ((MAXMASK >> k) & 1u) ? fmax(acc, red[w * 8 + k]) : acc + red[w * 8 + k];
      v[k] = acc;
    }
  }
}

// 1/x with one Newton step on the hardware approximation: about 40 correct bits, which is what
// a pivot needs (the iteration recomputes its residuals from the data every time), and a
// shorter dependent chain than fast_rcp on the factorisation's critical path.
__device__ __forceinline__ double pivot_rcp(double x) {
#ifdef LPLB_HOST_SIM
  return 1.0 / x;
#else
  double r;
  asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(x));
  return fma(r, fma(-x, r, 1.0), r);
#endif
}

// Packed lower triangle of an 8 x 8 block: (i, k), k <= i.
__device__ __forceinline__ constexpr int tri8(int i, int k) { return i * (i + 1) / 2 + k; }

// In: `a` = lower triangle of a symmetric positive definite 8 x 8 block.  Out: strictly lower
// part of `a` = unit lower L of a = L D L^T, dinv = 1/D.  Straight-line code with static
// register indices.  A pivot that rounding drove non-positive or non-finite is replaced by a
// huge one, which zeroes that unknown in the solves.
__device__ __forceinline__ void blk8_factor(double (&a)[36], double (&dinv)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    double piv = a[tri8(j, j)];
    if (!(piv > 1e-300) || !(piv < 1e300)) piv = 1e300;
    dinv[j] = pivot_rcp(piv);
#pragma unroll
    for (int i = j + 1; i < 8; ++i) {
      const double lij = a[tri8(i, j)] * dinv[j];
#pragma unroll
      for (int k = j + 1; k <= i; ++k) a[tri8(i, k)] = fma(-lij, a[tri8(k, j)], a[tri8(i, k)]);
    }
#pragma unroll
    for (int i = j + 1; i < 8; ++i) a[tri8(i, j)] *= dinv[j];
  }
}

// Strictly lower part of `w` = inverse of the unit lower L held in the strictly lower part of `a`.
__device__ __forceinline__ void blk8_invert(const double (&a)[36], double (&w)[36]) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int r = c + 1; r < 8; ++r) {
      double s = a[tri8(r, c)];
#pragma unroll
      for (int k = c + 1; k < r; ++k) s = fma(a[tri8(r, k)], w[tri8(k, c)], s);
      w[tri8(r, c)] = -s;
    }
}

// Factor the matrix in shared memory (lower triangle of N in `mat`), all kBlkThreads threads.
// On return: wblk holds W_k = L_kk^-1 per diagonal block, dinv holds 1/D, and below the
// diagonal blocks `mat` holds L_ik W_k.  The diagonal blocks of `mat` are left as they were.
//
// Per block column the dependent chain is: diagonal block (every thread of the panel warps
// factors it for itself, no hand-over), the rows below it (one thread per row: L and L D of the
// row), a barrier, the trailing update by all threads, a barrier.  What the chain does not need
// runs beside it: another warp inverts the diagonal block and stores W_k, and the products
// L_ik W_k that the substitutions use are formed by all threads next to the trailing update.
__device__ __forceinline__ void blk_factor(const int tid, const BlkLayout& l, double* sm) {
  double* mat = sm + l.mat;
  double* wblk = sm + l.wblk;
  double* pl = sm + l.pl;
  double* px = sm + l.px;
  double* dinvs = sm + l.dinv;
  const int warp = tid >> 5, ld = l.ld;
  for (int kb = 0; kb < l.nb; ++kb) {
    const int k0 = kb * 8, r0 = k0 + 8, m = l.gp - r0;  // m rows below this block column
    const int panel_warps = (m + 31) >> 5;               // warps 0 .. panel_warps-1 own the rows below
    const int inv_warp = panel_warps;                    // the next warp inverts the diagonal block
    if (warp <= inv_warp) {
      double a[36], dinv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int k = 0; k <= i; ++k) a[tri8(i, k)] = mat[(k0 + i) * ld + k0 + k];
      blk8_factor(a, dinv);
      if (warp == inv_warp) {  // same values from every lane
        double w[36];
        blk8_invert(a, w);
#pragma unroll
        for (int i = 1; i < 8; ++i)
#pragma unroll
          for (int k = 0; k < i; ++k) wblk[(k0 + i) * kPanelLd + k] = w[tri8(i, k)];
#pragma unroll
        for (int j = 0; j < 8; ++j) dinvs[k0 + j] = dinv[j];
      } else if (tid < m) {
        // row of the panel: x = A_row L_kk^-T = (L D)_row by substitution, L_row = x / D
        const int row = r0 + tid;
        double x[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) x[c] = mat[row * ld + k0 + c];
#pragma unroll
        for (int c = 1; c < 8; ++c)
#pragma unroll
          for (int k = 0; k < c; ++k) x[c] = fma(-x[k], a[tri8(c, k)], x[c]);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          px[row * kPanelLd + c] = x[c];
          pl[row * kPanelLd + c] = x[c] * dinv[c];
        }
      }
    }
    __syncthreads();
    if (m == 0) break;
    // trailing update of the lower triangle: A_ij -= sum_c L_ic (L D)_jc
    const int ti = tid >> 4, tj = tid & 15;
    for (int i = ti; i < m; i += 16) {
      if (tj > i) continue;
      const int row = r0 + i;
      double li[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) li[c] = pl[row * kPanelLd + c];
      for (int j = tj; j <= i; j += 16) {
        const int col = r0 + j;
        double acc = mat[row * ld + col];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc = fma(-li[c], px[col * kPanelLd + c], acc);
        mat[row * ld + col] = acc;
      }
    }
    // what the substitutions read below this diagonal block: (L_ik W_k)[row][c] = sum_j L[row][j] W_k[j][c]
    // (W_k has a unit diagonal and zeros above it, so the full sum needs no case distinction)
    for (int t = tid; t < m * 8; t += kBlkThreads) {
      const int row = r0 + (t >> 3), c = t & 7;
      double acc = 0.0;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fma(pl[row * kPanelLd + j], wblk[(k0 + j) * kPanelLd + c], acc);
      mat[row * ld + k0 + c] = acc;
    }
    __syncthreads();
  }
}

// Solve L D L^T x = g for one (g0) or two (g0, g1) right-hand sides held one element per row
// thread; row threads only.  One barrier per block column and direction.
template <bool TWO>
__device__ __forceinline__ void blk_solve(const int tid, const BlkLayout& l, double* sm, double& g0, double& g1) {
  const double* mat = sm + l.mat;
  const double* wblk = sm + l.wblk;
  const double* dinvs = sm + l.dinv;
  double* gv = sm + l.gv;
  double* xv = sm + l.xv;
  const int ld = l.ld, n32 = l.gp32;
  const bool has_row = tid < l.gp;
  const int myblk = tid >> 3, il = tid & 7;
  // forward: y_k = W_k g_k on the block's rows, g_i -= (L_ik W_k) g_k below it
  for (int kb = 0; kb < l.nb; ++kb) {
    const int k0 = kb * 8;
    if (myblk == kb) {
      gv[tid] = g0;
      if (TWO) gv[n32 + tid] = g1;
    }
    rows_sync(l.r_warps);
    if (has_row && myblk >= kb) {
      const double* coef = myblk == kb ? wblk + tid * kPanelLd : mat + tid * ld + k0;
      double a0 = 0.0, a1 = 0.0, b0 = 0.0, b1 = 0.0;
#pragma unroll
      for (int k = 0; k < 8; k += 2) {
        a0 = fma(coef[k], gv[k0 + k], a0);
        a1 = fma(coef[k + 1], gv[k0 + k + 1], a1);
        if (TWO) {
          b0 = fma(coef[k], gv[n32 + k0 + k], b0);
          b1 = fma(coef[k + 1], gv[n32 + k0 + k + 1], b1);
        }
      }
      if (myblk == kb) {
        g0 = a0 + a1;
        if (TWO) g1 = b0 + b1;
      } else {
        g0 -= a0 + a1;
        if (TWO) g1 -= b0 + b1;
      }
    }
  }
  // diagonal
  const double di = has_row ? dinvs[tid] : 0.0;
  xv[tid] = g0 * di;
  if (TWO) xv[n32 + tid] = g1 * di;
  rows_sync(l.r_warps);
  // backward: x_k = W_k^T y_k - sum over later blocks j of (L_jk W_k)^T x_j
  double a0 = 0.0, b0 = 0.0;
  if (has_row) {
    const int k0 = myblk * 8;
    double a1 = 0.0, b1 = 0.0;
#pragma unroll
    for (int k = 0; k < 8; k += 2) {
      a0 = fma(wblk[(k0 + k) * kPanelLd + il], xv[k0 + k], a0);
      a1 = fma(wblk[(k0 + k + 1) * kPanelLd + il], xv[k0 + k + 1], a1);
      if (TWO) {
        b0 = fma(wblk[(k0 + k) * kPanelLd + il], xv[n32 + k0 + k], b0);
        b1 = fma(wblk[(k0 + k + 1) * kPanelLd + il], xv[n32 + k0 + k + 1], b1);
      }
    }
    a0 += a1;
    b0 += b1;
  }
  for (int jb = l.nb - 1; jb >= 1; --jb) {
    const int j0 = jb * 8;
    if (myblk == jb) {
      gv[tid] = a0;
      if (TWO) gv[n32 + tid] = b0;
    }
    rows_sync(l.r_warps);
    if (has_row && myblk < jb) {
      double s0 = 0.0, s1 = 0.0, u0 = 0.0, u1 = 0.0;
#pragma unroll
      for (int k = 0; k < 8; k += 2) {
        s0 = fma(mat[(j0 + k) * ld + tid], gv[j0 + k], s0);
        s1 = fma(mat[(j0 + k + 1) * ld + tid], gv[j0 + k + 1], s1);
        if (TWO) {
          u0 = fma(mat[(j0 + k) * ld + tid], gv[n32 + j0 + k], u0);
          u1 = fma(mat[(j0 + k + 1) * ld + tid], gv[n32 + j0 + k + 1], u1);
        }
      }
      a0 -= s0 + s1;
      if (TWO) b0 -= u0 + u1;
    }
  }
  g0 = a0;
  if (TWO) g1 = b0;
}

// All kBlkThreads threads of the CTA call this together for one group of g <= kBlkMaxGroup
// ranks.  Thread tid < g is rank tid and passes its data as in ipm_solve_segment; every other
// thread passes w = 0, fixed = 0, src = dst = tid and null anchor pointers.  `sm` is
// block_solver_smem_bytes(g, D) of shared memory.  The outcome is the same on every row
// thread; f_out is meaningful on threads tid < g.
template <int D>
__device__ __forceinline__ IpmOutcome ipm_solve_block(const int tid, const int g, const double (&w_in)[D],
                                                      const double fixed, const int (&src_in)[D],
                                                      const int (&dst_in)[D], const IpmParams prm, double (&f_out)[D],
                                                      double* anchor, int* anchor_valid, double* sm) {
  constexpr double kEta = 0.995;
  // Private copies: when this function is not inlined the caller's arrays live in local memory,
  // and every use in the loop would be a load that has to be repeated after each store.
  int src[D], dst[D];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    src[d] = src_in[d];
    dst[d] = dst_in[d];
  }
  const BlkLayout l = blk_layout(g, D);
  const int warp = tid >> 5, lane = tid & 31;
  const int n32 = l.gp32, rw = l.r_warps;
  const bool is_row = warp < rw;
  const bool live = tid < g;
  // one reciprocal each, computed side by side: a double-precision division costs some 300 cycles
  const double kcomp = (double)(g + 2 * g * D), inv_kcomp = fast_rcp(kcomp), inv_g = fast_rcp((double)g);
  double* mat = sm + l.mat;
  double* wblk = sm + l.wblk;
  int* ctrl = reinterpret_cast<int*>(sm + l.ctrl);
  // per-rank values that other ranks read, one vector per use so that one barrier per use suffices
  double* x_wf = sm + l.xch;                 // D vectors: w f (also the first products of the set-up)
  double* x_y = x_wf + D * n32;              // y
  double* x_cw = x_y + n32;                  // D vectors: theta w^2 (also w during the set-up)
  double* x_rhs = x_cw + D * n32;            // D vectors: products of the two Newton solves (also the anchor's)
  double* x_dy = x_rhs + D * n32;            // dy

  for (int k = tid; k < l.gp * l.ld; k += kBlkThreads) mat[k] = 0.0;
  for (int k = tid; k < l.gp * kPanelLd; k += kBlkThreads) {
    const int r = k / kPanelLd, c = k - r * kPanelLd;
    wblk[k] = c == (r & 7) ? 1.0 : 0.0;
  }
  __syncthreads();

  IpmOutcome out{0, true, true, 0.0};
  if (!is_row) {
    // helper warps take part in the factorisations only
    for (;;) {
      __syncthreads();
      if (!ctrl[0]) break;
      blk_factor(tid, l, sm);
    }
    return out;
  }

  int red_phase = 0;
  // ---- scale so that the mean rank load is 1 ---------------------------------------
  double mine = fixed;
#pragma unroll
  for (int d = 0; d < D; ++d) mine += w_in[d];
  double total;
  {
    double r[1] = {live ? mine : 0.0};
    rows_reduce<1, 0u>(r, l, sm, warp, lane, red_phase);
    total = r[0];
  }
  const bool empty = !(total > 0.0);
  const double inv_scale = empty ? 0.0 : (double)g * fast_rcp(total);
  double w[D], base = fixed * inv_scale;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    w[d] = w_in[d] * inv_scale;
    x_cw[d * n32 + tid] = w[d];
  }
  rows_sync(rw);
#pragma unroll
  for (int d = 0; d < D; ++d) base += x_cw[d * n32 + src[d]];
  // a self edge moves no load: its column of M is zero, its load is already part of `base`
#pragma unroll
  for (int d = 0; d < D; ++d)
    if (dst[d] == tid) w[d] = 0.0;

  auto m_times = [&](const double(&x)[D], double* buf) -> double {  // (M x)_i, one barrier
#pragma unroll
    for (int d = 0; d < D; ++d) buf[d * n32 + tid] = w[d] * x[d];
    rows_sync(rw);
    double acc = 0.0;
#pragma unroll
    for (int d = 0; d < D; ++d) acc += w[d] * x[d] - buf[d * n32 + src[d]];
    return acc;
  };

  // ---- feasible start ------------------------------------------------------------------
  double f[D], v[D], z[D], q[D];
#pragma unroll
  for (int d = 0; d < D; ++d) f[d] = v[d] = 0.5;
  const double load = base + m_times(f, x_wf);
  double t, s, y = inv_g;
  {
    double r[2] = {live ? load : -1e300, live ? -load : -1e300};
    rows_reduce<2, 3u>(r, l, sm, warp, lane, red_phase);
    const double lmax = r[0], lmin = -r[1];
    t = lmax + 0.5 * (lmax - lmin) + 0.05;
    s = live ? t - load : 1.0;
    double r2[1] = {live ? s * y : 0.0};
    rows_reduce<1, 0u>(r2, l, sm, warp, lane, red_phase);
    const double mu0 = r2[0] * inv_g;
#pragma unroll
    for (int d = 0; d < D; ++d) z[d] = q[d] = 2.0 * mu0;
  }

  // ---- warm start from the anchor, if it still fits the data -----------------------------
  bool cold = true;
  {
    // The slot is read whether or not it is valid (it is always allocated), so that its loads
    // and the load of the flag are in flight together instead of one behind the other.
    double fa[D], va[D], za[D], qa[D], sa = 1.0, ya = inv_g, ta = 0.0;
    const bool slot = live && anchor != nullptr && anchor_valid != nullptr;
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
    if (!have) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        fa[d] = va[d] = 0.5;
        za[d] = qa[d] = 1.0;
      }
      sa = 1.0;
      ya = inv_g;
      ta = 0.0;
    }
    const double mfa = m_times(fa, x_rhs);
    double r[3] = {have ? 1.0 : 0.0, have ? fabs(ta - base - mfa - sa) : 0.0, have ? ta : -1e300};
    rows_reduce<3, 7u>(r, l, sm, warp, lane, red_phase);
    const bool fits = r[0] > 0.0 && !empty && r[1] <= prm.guard;
    if (fits && have) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        f[d] = fa[d];
        v[d] = va[d];
        z[d] = za[d];
        q[d] = qa[d];
      }
      s = sa;
      y = ya;
    }
    if (fits) {
      t = r[2];
      cold = false;
    }
  }
  bool saved = false;

  bool done = empty;
  int iters = 0;
  double gap = 1e300, gap_scale = 1.0;

  for (int it = 0;; ++it) {
    // ---- residuals, gap, stopping test ---------------------------------------------
#pragma unroll
    for (int d = 0; d < D; ++d) x_wf[d * n32 + tid] = w[d] * f[d];
    x_y[tid] = y;
    rows_sync(rw);
    double mf = 0.0;
    double r_u[D], r_d[D];
    double comp = s * y, dual_part = y * base, neg_rd = 0.0, worst_u = 0.0;
#pragma unroll
    for (int d = 0; d < D; ++d) {
      mf += w[d] * f[d] - x_wf[d * n32 + src[d]];
      r_u[d] = 1.0 - f[d] - v[d];
      r_d[d] = z[d] - q[d] - w[d] * (y - x_y[dst[d]]);
      comp += z[d] * f[d] + q[d] * v[d];
      dual_part -= q[d];
      neg_rd += fmin(r_d[d], 0.0);
      worst_u = fmax(worst_u, fabs(r_u[d]));
    }
    const double r_p = t - base - mf - s;
    double mu, r_t;
    {
      double r[5] = {live ? comp : 0.0, live ? y : 0.0, live ? dual_part + neg_rd : 0.0,
                     live ? base + mf : -1e300, live ? worst_u : 0.0};
      rows_reduce<5, 24u>(r, l, sm, warp, lane, red_phase);
      mu = r[0] * inv_kcomp;
      r_t = 1.0 - r[1];
      const double dual = r[2], primal = r[3], infeas = fmax(r[4], fabs(r_t));
      if (!done) {
        gap = primal - dual;
        gap_scale = fabs(primal);
        if ((gap <= prm.tol * gap_scale && infeas <= prm.tol) || mu <= 1e-13) done = true;
      }
    }
    // A cold solve leaves its first iterate at or below snap_mu behind as the next anchor.
    if (cold && !saved && !empty && mu <= prm.snap_mu) {
      if (live && anchor != nullptr) {
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
        if (tid == 0 && anchor_valid != nullptr) *anchor_valid = 1;
      }
      saved = true;
    }
    const bool go = !done && it < prm.max_iters;

    // ---- normal matrix, one row per rank --------------------------------------------------
    double inv_f[D], inv_v[D], theta[D];
    double inv_y = 1.0, inv_mu = 1.0;
    if (go) {
      ++iters;
      inv_y = fast_rcp(y);
      inv_mu = fast_rcp(kcomp * mu);
      double cw[D];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        inv_f[d] = fast_rcp(f[d]);
        inv_v[d] = fast_rcp(v[d]);
        theta[d] = fast_rcp(z[d] * inv_f[d] + q[d] * inv_v[d]);
        cw[d] = theta[d] * w[d] * w[d];
        x_cw[d * n32 + tid] = cw[d];
      }
      rows_sync(rw);
      if (tid < l.gp) {
        // Row `tid` of the lower triangle: zeros, then the 2 D off-diagonal terms and the
        // diagonal.  Terms that fall into the same column are merged in registers first, so
        // the row is written with plain stores and no store waits for a load.
        double* mrow = mat + tid * l.ld;
        for (int j = 0; j < tid; ++j) mrow[j] = 0.0;
        double diag = live ? s * inv_y : 1.0;
        if (live) {
          int col[2 * D];
          double val[2 * D];
#pragma unroll
          for (int d = 0; d < D; ++d) {
            const double held = x_cw[d * n32 + src[d]];
            diag += cw[d] + held;
            col[2 * d] = dst[d];
            val[2 * d] = cw[d];
            col[2 * d + 1] = src[d];
            val[2 * d + 1] = held;
          }
#pragma unroll
          for (int a = 0; a < 2 * D; ++a) {
            bool first = true;  // the first term of a column collects the later ones
            double acc = val[a];
#pragma unroll
            for (int b = 0; b < 2 * D; ++b) {
              if (b < a && col[b] == col[a]) first = false;
              if (b > a && col[b] == col[a]) acc += val[b];
            }
            if (first && col[a] < tid) mrow[col[a]] = -acc;
          }
        }
        mrow[tid] = diag;
      }
    }
    if (tid == 0) ctrl[0] = go ? 1 : 0;
    __syncthreads();
    if (!go) break;
    blk_factor(tid, l, sm);

    // ---- predictor (pass 0) and corrector (pass 1) share one body ------------------------
    double df[D], dv[D], dz[D], dq[D], ds = 0.0, dy = 0.0, dt = 0.0;
    double border = 0.0, inv_border_sum = 1.0, sig_mu = 0.0;
#pragma unroll
    for (int d = 0; d < D; ++d) df[d] = dv[d] = dz[d] = dq[d] = 0.0;
    double apf = 0.0, adf = 0.0;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const double r_sy = sig_mu - s * y - ds * dy;
      double r_zf[D], r_qv[D], rd_t[D];
      double acc = 0.0;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        r_zf[d] = sig_mu - z[d] * f[d] - dz[d] * df[d];
        r_qv[d] = sig_mu - q[d] * v[d] - dq[d] * dv[d];
        rd_t[d] = r_d[d] + r_zf[d] * inv_f[d] - (r_qv[d] - q[d] * r_u[d]) * inv_v[d];
        x_rhs[d * n32 + tid] = w[d] * theta[d] * rd_t[d];
      }
      rows_sync(rw);
#pragma unroll
      for (int d = 0; d < D; ++d) acc += w[d] * theta[d] * rd_t[d] - x_rhs[d * n32 + src[d]];
      double a = live ? acc - r_p + r_sy * inv_y : 0.0;
      if (pass == 0) {
        double b2 = live ? 1.0 : 0.0;  // N b = 1: the border column that carries sum(dy) = r_t
        blk_solve<true>(tid, l, sm, a, b2);
        border = b2;
      } else {
        double unused = 0.0;
        blk_solve<false>(tid, l, sm, a, unused);
      }
      {
        double r[2] = {live ? a : 0.0, live ? border : 0.0};
        rows_reduce<2, 0u>(r, l, sm, warp, lane, red_phase);
        if (pass == 0) inv_border_sum = fast_rcp(r[1]);
        dt = (r[0] - r_t) * inv_border_sum;
      }
      dy = a - dt * border;
      ds = (r_sy - s * dy) * inv_y;
      x_dy[tid] = dy;
      rows_sync(rw);
      float rp = ratio_to_bound(s, ds), rd = ratio_to_bound(y, dy);
      // sums for the centring parameter: the complementarity after a step (ap, ad) is
      // kcomp mu + ap c_p + ad c_d + ap ad c_pd, so it can be reduced before the step is known
      double c_p = ds * y, c_d = s * dy, c_pd = ds * dy;
#pragma unroll
      for (int d = 0; d < D; ++d) {
        df[d] = theta[d] * (rd_t[d] - w[d] * (dy - x_dy[dst[d]]));
        dv[d] = r_u[d] - df[d];
        dz[d] = (r_zf[d] - z[d] * df[d]) * inv_f[d];
        dq[d] = (r_qv[d] - q[d] * dv[d]) * inv_v[d];
        rp = fminf(rp, fminf(ratio_to_bound(f[d], df[d]), ratio_to_bound(v[d], dv[d])));
        rd = fminf(rd, fminf(ratio_to_bound(z[d], dz[d]), ratio_to_bound(q[d], dq[d])));
        c_p += z[d] * df[d] + q[d] * dv[d];
        c_d += dz[d] * f[d] + dq[d] * v[d];
        c_pd += dz[d] * df[d] + dq[d] * dv[d];
      }
      if (pass == 0) {  // step lengths and the centring parameter from the affine step, one reduction
        double r[5] = {live ? -(double)rp : -3.0e38, live ? -(double)rd : -3.0e38, live ? c_p : 0.0,
                       live ? c_d : 0.0, live ? c_pd : 0.0};
        rows_reduce<5, 3u>(r, l, sm, warp, lane, red_phase);
        apf = -r[0];
        adf = -r[1];
        const double ap = fmin(apf, 1.0), ad = fmin(adf, 1.0);
        const double comp_aff = kcomp * mu + ap * r[2] + ad * r[3] + ap * ad * r[4];
        const double ratio = fmin(fmax(comp_aff * inv_mu, 0.0), 1.0);
        sig_mu = ratio * ratio * ratio * mu;
      } else {
        double r[2] = {live ? -(double)rp : -3.0e38, live ? -(double)rd : -3.0e38};
        rows_reduce<2, 3u>(r, l, sm, warp, lane, red_phase);
        apf = -r[0];
        adf = -r[1];
      }
    }
    const double ap = fmin(kEta * apf, 1.0), ad = fmin(kEta * adf, 1.0);
    t += ap * dt;
    if (live) {
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

  double bad = 0.0;
#pragma unroll
  for (int d = 0; d < D; ++d) {
    if (live && !((f[d] == f[d]) && fabs(f[d]) < 1e300)) bad = 1.0;
    f_out[d] = fmin(fmax(f[d], 0.0), 1.0);
  }
  {
    double r[1] = {bad};
    rows_reduce<1, 1u>(r, l, sm, warp, lane, red_phase);
    bad = r[0];
  }
  const bool finite = bad == 0.0;
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

}  // namespace lplb
