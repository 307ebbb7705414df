"""The per-group balancing LP: builders, float64 oracles and the CPU solver.

For one LP group with ``G`` ranks and ``D`` replicated bundles per rank, let
``w[j, d]`` be the load of rank ``j``'s bundle ``d`` and ``F[i]`` the load of rank
``i``'s non-replicated experts.  Variable ``f[j, d] in [0, 1]`` is the share of bundle
``(j, d)`` that stays on its origin ``j``; the rest goes to the replica holder
``o2r[j, d]``.  The LP is::

    min t   s.t.   load_i(f) = base_i + sum_k M[i, k] f_k <= t,   0 <= f <= 1

with ``M[origin(k), k] = +w_k``, ``M[holder(k), k] = -w_k`` and
``base_i = F_i + sum_{k held by i} w_k``.  This is the compact form of the
``(G + G*D) x (2*G*D + G + 2)`` equality system that the reference assembles
(reference ``lplb/resources/csrc-tmpl/minilp.cu:199-293``); ``standard_form`` rebuilds
that larger system for cross-checks.

Solvers:

* ``solve_highs``  – scipy/HiGHS simplex, the float64 ground truth.
* ``solve_ipm``    – batched Mehrotra predictor-corrector interior-point method on
  the compact form, written with plain tensor ops.  In float64 it is the dense torch
  oracle; in float32 it performs the same arithmetic, in the same order of steps, as
  the CUDA kernel, so it doubles as the CPU path of ``Planner.solve_probs`` and as the
  reference the kernel is tested against.
* ``affine_scaling_reference`` – the primal affine-scaling iteration with a big-M
  start and a fixed number of steps that the reference runs
  (reference ``lplb/resources/csrc-tmpl/minilp.cu:323-401``), restated on the standard
  form; used only to report how far that method lands from the optimum.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .topology import invert_r2o

__all__ = [
    "bundle_loads",
    "compact_form",
    "standard_form",
    "rank_loads",
    "solve_highs",
    "solve_ipm",
    "IpmResult",
    "affine_scaling_reference",
]


def bundle_loads(
    workload: torch.Tensor, phy2log: torch.Tensor, n_group: int, g: int, d: int, ll: int, c: int
) -> tuple[torch.Tensor, torch.Tensor]:
    """Fold per-expert loads into per-bundle loads ``w[NG, G, D]`` and fixed loads ``F[NG, G]``.

    ``workload`` is indexed by logical expert; ``phy2log`` gives each rank's slot order
    (reference ``lplb/resources/csrc-tmpl/minilp.cu:203-233``).
    """
    pl = ll + c * d
    own = phy2log.reshape(n_group, g, pl)[:, :, :ll].long()
    loads = workload.reshape(-1)[own]
    w = loads[:, :, : c * d].reshape(n_group, g, c, d).sum(2)
    fixed = loads[:, :, c * d :].sum(-1)
    return w, fixed


def compact_form(w: torch.Tensor, fixed: torch.Tensor, r2o: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Return ``(M [.., G, K], base [.., G])`` for batched ``w [.., G, D]``, ``fixed [.., G]``."""
    g, d = r2o.shape
    k = g * d
    o2r = invert_r2o(r2o.cpu()).long().reshape(-1).to(w.device)
    origin = torch.arange(g, device=w.device).repeat_interleave(d)
    wk = w.reshape(*w.shape[:-2], k)
    m = torch.zeros(*w.shape[:-2], g, k, dtype=w.dtype, device=w.device)
    cols = torch.arange(k, device=w.device)
    m[..., origin, cols] += wk
    m[..., o2r, cols] -= wk
    base = fixed.clone()
    base.index_add_(-1, o2r, wk)
    return m, base


def rank_loads(f: torch.Tensor, w: torch.Tensor, fixed: torch.Tensor, r2o: torch.Tensor) -> torch.Tensor:
    """Per-rank load ``[.., G]`` realised by shares ``f [.., G, D]``."""
    m, base = compact_form(w, fixed, r2o)
    return base + (m @ f.reshape(*f.shape[:-2], -1, 1).to(m.dtype)).squeeze(-1)


def standard_form(
    w: torch.Tensor, fixed: torch.Tensor, r2o: torch.Tensor, big_m: float = 1000.0
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The equality-form LP ``min c.x, A x = b, x >= 0`` of one group (float64).

    Columns: ``xo[G*D]`` (share kept), ``xr[G*D]`` (share sent), slacks ``s[G]``, ``t``,
    and one artificial column that makes ``x = 1`` feasible.
    """
    g, d = r2o.shape
    k = g * d
    nc, nv = g + k, 2 * k + g + 2
    a = torch.zeros(nc, nv, dtype=torch.float64)
    b = torch.zeros(nc, dtype=torch.float64)
    o2r = invert_r2o(r2o.cpu()).long()
    wk = w.reshape(-1).double()
    for j in range(g):
        for dd in range(d):
            col = j * d + dd
            a[j, col] = wk[col]
            a[int(o2r[j, dd]), k + col] = wk[col]
            a[g + col, col] = 1.0
            a[g + col, k + col] = 1.0
    a[:g, 2 * k : 2 * k + g] = torch.eye(g, dtype=torch.float64)
    a[:g, 2 * k + g] = -1.0
    b[:g] = -fixed.double()
    b[g:] = 1.0
    a[:, nv - 1] = b - a[:, : nv - 1].sum(1)
    c = torch.zeros(nv, dtype=torch.float64)
    c[nv - 2] = 1.0
    c[nv - 1] = big_m
    return a, b, c


def solve_highs(w: torch.Tensor, fixed: torch.Tensor, r2o: torch.Tensor) -> tuple[torch.Tensor, float]:
    """Ground-truth optimum of one group with HiGHS: ``(f [G, D], t*)``."""
    from scipy.optimize import linprog

    g, d = r2o.shape
    k = g * d
    m, base = compact_form(w.double(), fixed.double(), r2o)
    a_ub = np.concatenate([m.numpy(), -np.ones((g, 1))], axis=1)
    cost = np.zeros(k + 1)
    cost[k] = 1.0
    res = linprog(cost, A_ub=a_ub, b_ub=-base.numpy(), bounds=[(0, 1)] * k + [(None, None)], method="highs")
    if res.status != 0:
        raise RuntimeError(f"HiGHS failed: {res.message}")
    return torch.from_numpy(res.x[:k]).reshape(g, d), float(res.fun)


@dataclass
class IpmResult:
    f: torch.Tensor  #: ``[B, G, D]`` shares kept on the origin, inside ``[0, 1]``
    t: torch.Tensor  #: ``[B]`` max rank load realised by ``f`` (in the caller's units)
    gap: torch.Tensor  #: ``[B]`` final relative duality gap
    iters: torch.Tensor  #: ``[B]`` iterations used
    converged: torch.Tensor  #: ``[B]`` bool
    anchor: dict | None = None  #: warm-start state to hand to the next call (see ``solve_ipm``)
    warm: torch.Tensor | None = None  #: ``[B]`` bool, instances that started from the anchor


def _chol_factor(n: torch.Tensor) -> torch.Tensor:
    """Batched right-looking Cholesky with guarded pivots, ``n [B, G, G]`` SPD.

    A pivot that rounding drove below ``1e-30`` or to a non-finite value is replaced by
    a huge number, which zeroes that unknown in the solves instead of poisoning the
    rest with NaNs; the CUDA kernel applies the same guard.
    """
    a = n.clone()
    g = a.shape[-1]
    lower = torch.zeros_like(a)
    for j in range(g):
        piv = a[:, j, j]
        bad = ~(piv > 1e-30)
        piv = torch.where(bad, torch.full_like(piv, 1e30), piv)
        inv = torch.rsqrt(piv)
        col = a[:, :, j] * inv.unsqueeze(1)
        col[:, :j] = 0
        lower[:, :, j] = col
        a = a - col.unsqueeze(2) * col.unsqueeze(1)
    return lower


def _chol_apply(lower: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    """Solve ``L L^T x = rhs`` for ``rhs [B, G]`` by forward and backward substitution."""
    g = lower.shape[-1]
    x = rhs.clone()
    for j in range(g):
        x[:, j] = x[:, j] / lower[:, j, j]
        x[:, j + 1 :] -= lower[:, j + 1 :, j] * x[:, j : j + 1]
    for j in range(g - 1, -1, -1):
        x[:, j] = x[:, j] / lower[:, j, j]
        x[:, :j] -= lower[:, j, :j] * x[:, j : j + 1]
    return x


def solve_ipm(
    w: torch.Tensor,
    fixed: torch.Tensor,
    r2o: torch.Tensor,
    *,
    max_iters: int = 24,
    tol: float = 1e-4,
    dtype: torch.dtype = torch.float64,
    factor_dtype: torch.dtype | None = None,
    anchor: dict | None = None,
    warm_start: bool = False,
    guard: float = 0.1,
    snap_mu: float = 1e-3,
) -> IpmResult:
    """Batched primal-dual interior-point solve of the compact LP.

    ``w [B, G, D]``, ``fixed [B, G]`` in any non-negative units.  Loads are rescaled by
    the mean rank load so the optimum is O(1); ``tol`` bounds the relative duality gap
    ``(primal - dual) / primal``.

    Method.  Unknowns: shares ``f`` with upper slacks ``v = 1 - f``, level ``t``, rank
    slacks ``s = t - load(f)``, multipliers ``y`` (rank constraints, ``sum y = 1``), ``z``
    (``f >= 0``) and ``q`` (``f <= 1``).  The start ``f = v = 1/2``, ``y = 1/G``,
    ``z = q`` is primal *and* dual feasible because every column of ``M`` sums to zero,
    so no phase one or big-M column is needed; residuals are still carried in the Newton
    right-hand sides so rounding drift is corrected.  Each iteration eliminates
    everything but ``dy`` and ``dt``: ``N = M diag(theta) M^T + diag(s / y)`` with
    ``theta = 1 / (z/f + q/v)`` is a weighted graph Laplacian of the topology plus a
    positive diagonal, factored once by Cholesky and reused for the predictor, the
    corrector and the border column that carries ``sum dy = r_t``.  Step lengths keep
    every positive quantity positive with a 0.995 fraction to the boundary.

    Warm start (``warm_start=True``).  A cold solve saves its first iterate whose average
    complementarity is at most ``snap_mu`` as the *anchor* (returned in ``result.anchor``;
    pass it back in).  The next solve starts from the anchor when the new data leave it
    nearly primal feasible, ``max_i |t - load_i(f) - s_i| <= guard`` in units of the mean
    rank load, and cold otherwise (which refreshes the anchor).  Batches drawn from one
    distribution keep fitting the same anchor and converge in one or two iterations; a shift
    of the distribution trips the guard.  The residuals of the anchor are removed by the
    Newton steps like any other infeasibility.
    """
    g, d = r2o.shape
    k = g * d
    squeeze = w.dim() == 2
    if squeeze:
        w, fixed = w.unsqueeze(0), fixed.unsqueeze(0)
    nb = w.shape[0]
    dev = w.device  # every tensor below lives where the data lives (CPU oracle or the planner's GPU)
    w = w.to(dtype)
    fixed = fixed.to(dtype)
    scale = (w.sum((-1, -2)) + fixed.sum(-1)) / g
    empty = ~(scale > 0)  # nothing to balance: report f = 1 (keep everything on the origin)
    scale = torch.where(empty, torch.ones_like(scale), scale)
    m, base = compact_form(w / scale.view(nb, 1, 1), fixed / scale.view(nb, 1), r2o)
    mt = m.transpose(1, 2)
    one = torch.ones(nb, g, 1, dtype=dtype, device=dev)
    fdt = factor_dtype or dtype

    f = torch.full((nb, k), 0.5, dtype=dtype, device=dev)
    v = torch.full((nb, k), 0.5, dtype=dtype, device=dev)
    load = base + (m @ f.unsqueeze(-1)).squeeze(-1)
    spread = load.max(1).values - load.min(1).values
    t = load.max(1).values + 0.5 * spread + 0.05
    s = t.unsqueeze(1) - load
    y = torch.full((nb, g), 1.0 / g, dtype=dtype, device=dev)
    mu0 = (s * y).sum(1, keepdim=True) / g
    z = (mu0 / 0.5).expand(nb, k).clone()
    q = z.clone()

    use_warm = torch.zeros(nb, dtype=torch.bool, device=dev)
    if warm_start and anchor is not None:
        fa, va = anchor["f"].to(dtype), anchor["v"].to(dtype)
        sa, ta = anchor["s"].to(dtype), anchor["t"].to(dtype)
        rp = (ta.unsqueeze(1) - base - (m @ fa.unsqueeze(-1)).squeeze(-1) - sa).abs().max(1).values
        use_warm = anchor["valid"].bool() & ~empty & (rp <= guard)
        pick = use_warm.unsqueeze(1)
        f, v = torch.where(pick, fa, f), torch.where(pick, va, v)
        z, q = torch.where(pick, anchor["z"].to(dtype), z), torch.where(pick, anchor["q"].to(dtype), q)
        s, y = torch.where(pick, sa, s), torch.where(pick, anchor["y"].to(dtype), y)
        t = torch.where(use_warm, ta, t)
    new_anchor = None
    if warm_start:
        if anchor is not None:
            new_anchor = {key: val.clone() for key, val in anchor.items()}
        else:
            new_anchor = {
                "f": torch.zeros(nb, k, dtype=dtype, device=dev), "v": torch.zeros(nb, k, dtype=dtype, device=dev),
                "z": torch.zeros(nb, k, dtype=dtype, device=dev), "q": torch.zeros(nb, k, dtype=dtype, device=dev),
                "s": torch.zeros(nb, g, dtype=dtype, device=dev), "y": torch.zeros(nb, g, dtype=dtype, device=dev),
                "t": torch.zeros(nb, dtype=dtype, device=dev), "valid": torch.zeros(nb, dtype=torch.bool, device=dev),
            }
    saved = torch.zeros(nb, dtype=torch.bool, device=dev)
    # the feasible iterate with the smallest gap seen so far: what is returned if the loop
    # ends without meeting `tol` (a tolerance below what float arithmetic can certify)
    best_gap = torch.full((nb,), float("inf"), dtype=dtype, device=dev)
    best_f = f.clone()
    stopped = torch.zeros(nb, dtype=torch.bool, device=dev)

    done = empty.clone()
    iters = torch.zeros(nb, dtype=torch.int64, device=dev)
    gap = torch.where(empty, torch.zeros(nb, dtype=dtype, device=dev), torch.full((nb,), float("inf"), dtype=dtype, device=dev))
    eta = 0.995
    n_comp = g + 2 * k

    def max_step(val: torch.Tensor, dval: torch.Tensor) -> torch.Tensor:
        ratio = torch.where(dval < 0, -val / dval, torch.full_like(val, float("inf")))
        return ratio.min(1).values

    for _ in range(max_iters):
        mf = (m @ f.unsqueeze(-1)).squeeze(-1)
        r_p = t.unsqueeze(1) - base - mf - s
        r_u = 1.0 - f - v
        r_d = z - q - (mt @ y.unsqueeze(-1)).squeeze(-1)
        r_t = 1.0 - y.sum(1)
        mu = ((s * y).sum(1) + (z * f).sum(1) + (q * v).sum(1)) / n_comp
        # primal value of the current shares and the dual bound of the current multipliers
        primal = (base + mf).max(1).values
        dual = (y * base).sum(1) - q.sum(1) + torch.minimum(r_d, torch.zeros_like(r_d)).sum(1)
        gap_now = (primal - dual) / primal.abs().clamp_min(1e-12)
        infeas = torch.maximum(r_u.abs().max(1).values, r_t.abs())
        if new_anchor is not None:
            take = ~use_warm & ~saved & ~empty & (mu <= snap_mu)
            if bool(take.any()):
                for key, val in (("f", f), ("v", v), ("z", z), ("q", q), ("s", s), ("y", y), ("t", t)):
                    new_anchor[key][take] = val[take]
                new_anchor["valid"][take] = True
                saved = saved | take
        # at mu ~ 1e-13 the iterate is optimal to machine precision: stop instead of dividing by it
        better = (~done) & (gap_now < best_gap) & (infeas <= max(tol, 1e-9))
        best_gap = torch.where(better, gap_now, best_gap)
        best_f = torch.where(better.unsqueeze(1), f, best_f)
        newly = (~done) & (((gap_now <= tol) & (infeas <= tol)) | (mu <= 1e-13))
        gap = torch.where(done, gap, gap_now)
        done = done | newly
        if bool(done.all()):
            break
        iters = iters + (~done).long()

        theta = 1.0 / (z / f + q / v)
        n = (m * theta.unsqueeze(1)) @ mt + torch.diag_embed(s / y)
        n = torch.where(done.view(nb, 1, 1), torch.eye(g, dtype=dtype, device=dev).expand(nb, g, g), n)
        chol = _chol_factor(n.to(fdt))
        border = _chol_apply(chol, one.squeeze(-1).to(fdt)).to(dtype)
        border_sum = border.sum(1)

        def newton(r_sy: torch.Tensor, r_zf: torch.Tensor, r_qv: torch.Tensor):
            rd_t = r_d + r_zf / f - (r_qv - q * r_u) / v
            rhs = (m @ (theta * rd_t).unsqueeze(-1)).squeeze(-1) - r_p + r_sy / y
            a = _chol_apply(chol, rhs.to(fdt)).to(dtype)
            dt = (a.sum(1) - r_t) / border_sum
            dy = a - dt.unsqueeze(1) * border
            df = theta * (rd_t - (mt @ dy.unsqueeze(-1)).squeeze(-1))
            dv = r_u - df
            ds = (r_sy - s * dy) / y
            dz = (r_zf - z * df) / f
            dq = (r_qv - q * dv) / v
            return df, dv, dt, ds, dy, dz, dq

        # predictor
        df, dv, dt, ds, dy, dz, dq = newton(-s * y, -z * f, -q * v)
        ap = torch.minimum(torch.minimum(max_step(s, ds), max_step(f, df)), max_step(v, dv)).clamp_max(1.0)
        ad = torch.minimum(torch.minimum(max_step(y, dy), max_step(z, dz)), max_step(q, dq)).clamp_max(1.0)
        mu_aff = (
            ((s + ap[:, None] * ds) * (y + ad[:, None] * dy)).sum(1)
            + ((z + ad[:, None] * dz) * (f + ap[:, None] * df)).sum(1)
            + ((q + ad[:, None] * dq) * (v + ap[:, None] * dv)).sum(1)
        ) / n_comp
        sigma = (mu_aff / mu).clamp(0.0, 1.0) ** 3
        sm = (sigma * mu).unsqueeze(1)
        # corrector
        df, dv, dt, ds, dy, dz, dq = newton(sm - s * y - ds * dy, sm - z * f - dz * df, sm - q * v - dq * dv)
        ap = (eta * torch.minimum(torch.minimum(max_step(s, ds), max_step(f, df)), max_step(v, dv))).clamp_max(1.0)
        ad = (eta * torch.minimum(torch.minimum(max_step(y, dy), max_step(z, dz)), max_step(q, dq))).clamp_max(1.0)
        # A step that is not finite (an instance pushed far past convergence by a tolerance
        # tighter than the arithmetic allows) is not taken: that instance stops where it is.
        cand = (f + ap[:, None] * df, v + ap[:, None] * dv, t + ap * dt, s + ap[:, None] * ds,
                y + ad[:, None] * dy, z + ad[:, None] * dz, q + ad[:, None] * dq)
        finite = torch.ones(nb, dtype=torch.bool, device=dev)
        for c in cand:
            finite &= torch.isfinite(c.reshape(nb, -1)).all(1)
        stopped = stopped | (~done & ~finite)
        done = done | ~finite
        move = (~done) & finite

        def upd(old, new):
            return torch.where(move.view(-1, *([1] * (old.dim() - 1))), new, old)

        f, v, t, s, y, z, q = (upd(o, c) for o, c in zip((f, v, t, s, y, z, q), cand))

    certified = done & ~stopped
    f = torch.where(certified.unsqueeze(1), f, best_f)
    gap = torch.where(certified, gap, best_gap)
    f = torch.where(empty.unsqueeze(1), torch.ones_like(f), f.clamp(0.0, 1.0))
    load = base + (m @ f.unsqueeze(-1)).squeeze(-1)
    out = IpmResult(
        f=f.reshape(nb, g, d),
        t=load.max(1).values * scale,
        gap=gap,
        iters=iters,
        converged=certified,
        anchor=new_anchor,
        warm=use_warm,
    )
    return out


def affine_scaling_reference(
    w: torch.Tensor, fixed: torch.Tensor, r2o: torch.Tensor, steps: int = 5, dtype=np.float32
) -> tuple[torch.Tensor, float, bool]:
    """Primal affine scaling from ``x = 1`` with a big-M column, fixed step count.

    Restates the numerical method of the reference kernel on one group so its distance
    from the optimum can be reported.  ``d_max`` here is the true maximum over all
    variables (the reference keeps only each lane's last entry,
    reference ``lplb/resources/csrc-tmpl/minilp.cu:355-357``).  Returns
    ``(f [G, D], max rank load realised, accepted)`` with the reference's acceptance
    test (``minilp.cu:381-382``).
    """
    g, d = r2o.shape
    k = g * d
    peak = max(float(w.max()), float(fixed.max()), 1e-30)
    a64, b64, c64 = standard_form(w.double() / peak, fixed.double() / peak, r2o)
    a, b, c = a64.numpy().astype(dtype), b64.numpy().astype(dtype), c64.numpy().astype(dtype)
    x = np.ones(a.shape[1], dtype=dtype)
    d_max = dtype(0)
    for _ in range(steps):
        ax2 = a * (x * x)
        lhs = ax2 @ a.T
        rhs = ax2 @ c
        try:
            wv = np.linalg.solve(lhs.astype(dtype), rhs.astype(dtype)).astype(dtype)
        except np.linalg.LinAlgError:
            return torch.full((g, d), 0.5, dtype=torch.float64), float("nan"), False
        r = wv @ a
        dvec = x * (c - r)
        d_max = dvec.max()
        x = x * (1 - dtype(0.999) / d_max * dvec)
    resid = np.abs(a @ x - b).max()
    ok = bool(d_max < 0.1 and 0 <= x[-1] < 1e-4 and resid < 0.05)
    f = torch.from_numpy(x[:k].astype(np.float64)).reshape(g, d) if ok else torch.full((g, d), 0.5, dtype=torch.float64)
    realised = rank_loads(f.clamp(0, 1), w.double(), fixed.double(), r2o).max()
    return f, float(realised), ok
