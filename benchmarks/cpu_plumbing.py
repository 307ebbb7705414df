#!/usr/bin/env python
"""CPU-only walk through the whole planner, no GPU and no extension needed.

32 logical experts over 8 simulated ranks (Cube, 2 redundant experts per rank), loads from
4096 tokens x top-8 routing with logits ~ N(0,1) plus a per-expert bias ~ N(0,1.5), seed 0.
The embedded placement balancer re-places the experts, the Cube LP is solved by the dense
float64 torch interior-point method and checked against HiGHS, and the redirect is applied.

Usage: python benchmarks/cpu_plumbing.py
"""

import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube, lp  # noqa: E402


def main():
    g = torch.Generator().manual_seed(0)
    bias = torch.randn(32, generator=g) * 1.5
    idx = (torch.randn(4096, 32, generator=g) + bias).topk(8, dim=-1).indices
    counts = torch.bincount(idx.reshape(-1), minlength=32)
    planner = Planner(cube(), 32 + 16, 32, 8, device="cpu")
    pl = planner.n_local_routed_experts

    def rank_load(phys):
        load = torch.bincount(phys.reshape(-1) // pl, minlength=8).double()
        return float(load.max() / load.mean())

    natural = rank_load(planner.mapping.log2phy[idx.reshape(-1), 0].long())
    t0 = time.perf_counter()
    planner.update_redundancy_mapping(counts)
    placed_s = time.perf_counter() - t0
    placed = rank_load(planner.mapping.log2phy[idx.reshape(-1), 0].long())
    avail = torch.zeros(1, dtype=torch.int64)
    t0 = time.perf_counter()
    out = planner.run(idx, avail, 8)
    run_s = time.perf_counter() - t0
    w, fixed = lp.bundle_loads(counts.double(), planner.phy2log, 1, 8, 2, 4, 1)
    _, t_opt = lp.solve_highs(w[0], fixed[0], cube())
    ipm = lp.solve_ipm(w, fixed, cube(), tol=1e-9, max_iters=60)  # far tighter than the planner's 1e-4
    print(json.dumps({
        "max_over_mean": {"natural_placement": round(natural, 4), "after_placement": round(placed, 4),
                          "after_lp_redirect": round(rank_load(out), 4),
                          "lp_optimum_highs": round(t_opt / float(counts.sum() / 8), 4)},
        "ipm_vs_highs_relative_gap": abs(float(ipm.t[0]) - t_opt) / t_opt,
        "ipm_iterations": int(ipm.iters[0]),
        "groups_converged": int(avail),
        "seconds": {"update_redundancy_mapping": round(placed_s, 4), "run_cpu": round(run_s, 4)},
    }))


if __name__ == "__main__":
    main()
