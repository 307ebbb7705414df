"""Shared test utilities: reference-style workloads and the analytic balance check."""

from __future__ import annotations

import torch

from lplb_b200 import topology

# (name, r2o, n_logical, ep_size, redundants per rank, reorder with history, max/mean bound)
# Same six configurations and bounds as reference tests/test_solve.py:13-22.
SOLVE_CONFIGS = [
    ("cube-ep32", topology.cube(), 256, 32, 2, True, 1.07),
    ("cube-ep32-c2", topology.cube(), 256, 32, 4, False, 1.07),
    ("cube-ep64", topology.cube(), 256, 64, 2, True, 1.10),
    ("ring-ep32", topology.ring(8), 256, 32, 1, True, 1.07),
    ("hypercube-ep16", topology.hypercube(), 256, 16, 2, True, 1.03),
    ("torus8x4-ep32", topology.torus(8, 4), 256, 32, 2, False, 1.01),
]


def synthetic_loads(n_logical: int, seed: int, device="cpu"):
    """History ~ N(1, 0.15) * 2^20 and current load ~ N(1, 0.3) * 2^12, clamped at zero
    (the distributions of reference tests/test_solve.py:41-51)."""
    g = torch.Generator().manual_seed(seed)
    history = (torch.randn(n_logical, generator=g) * 0.15 + 1).clamp_min(0).mul(2**20).long()
    current = (torch.randn(n_logical, generator=g) * 0.3 + 1).clamp_min(0).mul(2**12).int()
    return history.to(device), current.to(device)


def balance_after(planner, phy2log, workload, probs) -> float:
    """max/mean rank load after applying shares analytically."""
    g, d = planner.group_size, planner.num_redundants
    c, ll = planner.combined_redundant_experts, planner.n_local_logical_routed_experts
    own = phy2log.reshape(planner.n_group, g, -1)[:, :, :ll].long().cpu()
    loads = workload.cpu().double()[own]
    w = loads[:, :, : c * d].reshape(planner.n_group, g, c, d).sum(2)
    fixed = loads[:, :, c * d :].sum(-1)
    from lplb_b200 import lp

    rank = lp.rank_loads(probs.cpu().double(), w, fixed, planner.r2o.cpu())
    return float(rank.max() / rank.mean())
