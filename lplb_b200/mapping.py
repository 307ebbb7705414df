"""Physical/logical expert maps for a redundancy topology.

Physical expert ids are rank-major: ``phys = ep_rank * Pl + slot``.  On every rank
slots ``0 .. Ll-1`` are its own logical experts and slots ``Ll .. Pl-1`` are replicas.
The first ``C*D`` own slots are the ones that get replicated; own slot ``j*D + d``
belongs to bundle ``d`` and its copy lives in slot ``Ll + j*D + d`` of the rank
``o2r[rank, d]``.

This module replaces the slow-path bookkeeping of the reference's
``Planner.update_redundancy_mapping`` (reference ``lplb/planner.py:115-182``): the
Python double loop that builds ``log2phy`` becomes two scatters, nothing is pinned to
``'cuda'``, and the per-logical-expert tables that the redirect kernel needs are
built once here instead of inside every kernel launch
(reference ``lplb/resources/csrc-tmpl/minilp.cu:466-496``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .eplb import rebalance_experts
from .topology import invert_r2o

__all__ = ["ExpertMapping", "build_mapping"]


@dataclass
class ExpertMapping:
    """All static maps derived from one placement decision.

    Shapes use ``E`` logical experts, ``P = ep_size * Pl`` physical experts.
    """

    phy2log: torch.Tensor  #: ``[P]`` int32, logical id held by each physical slot
    log2phy: torch.Tensor  #: ``[E, 2]`` int32, (original, replica or -1)
    logcnt: torch.Tensor  #: ``[E]`` int32, 1 or 2
    log2edge: torch.Tensor  #: ``[E]`` int32, flat index into ``probs[NG, G, D]`` or -1

    def to(self, device: torch.device | str) -> "ExpertMapping":
        return ExpertMapping(*(t.to(device) for t in (self.phy2log, self.log2phy, self.logcnt, self.log2edge)))


def build_mapping(
    r2o: torch.Tensor,
    n_group: int,
    n_local_logical: int,
    n_combined: int,
    workload: torch.Tensor | None = None,
    *,
    n_nodes: int = 1,
) -> ExpertMapping:
    """Place logical experts and derive every lookup table (CPU tensors).

    :param r2o: ``[G, D]`` topology.
    :param n_group: number of independent LP groups (``ep_size // G``).
    :param n_local_logical: ``Ll``, logical experts per rank.
    :param n_combined: ``C``, experts per replicated bundle.
    :param workload: optional ``[E]`` load history.  Without it experts keep their
        natural order.  With it they are first reordered across ranks by the embedded
        placement balancer (no replication), then each rank's experts are sorted by
        history, heaviest first, so the heaviest ``C*D`` are the replicated ones.
    :param n_nodes: node count handed to the placement balancer (the reference
        derives it from ``torch.cuda.device_count()``, reference ``lplb/planner.py:133``,
        which divides by zero without a GPU).
    """
    r2o_cpu = r2o.detach().to("cpu", torch.int64)
    g, d = r2o_cpu.shape
    ll, c = n_local_logical, n_combined
    ep_size = n_group * g
    n_logical = ep_size * ll
    n_rep = c * d
    if n_rep > ll:
        raise ValueError(f"{n_rep} replicated experts per rank exceed the {ll} local logical experts")
    pl = ll + n_rep

    if workload is None:
        own = torch.arange(n_logical, dtype=torch.int64).reshape(n_group, g, ll)
    else:
        hist = workload.detach().to("cpu").reshape(-1)
        if hist.numel() != n_logical:
            raise ValueError(f"workload has {hist.numel()} entries, expected {n_logical}")
        placed, _, _ = rebalance_experts(hist.unsqueeze(0), n_logical, n_group, n_nodes, ep_size)
        own = placed[0].reshape(n_group, g, ll)
        by_history = torch.sort(hist.to(torch.float64)[own], dim=-1, descending=True, stable=True).indices
        own = own.gather(-1, by_history)

    # Replica slots: rank i's slot (j, d) mirrors rank r2o[i, d]'s own slot (j, d).
    bundles = own[:, :, :n_rep].reshape(n_group, g, c, d)
    src = r2o_cpu.view(1, g, 1, d).expand(n_group, g, c, d)
    mirrored = bundles.gather(1, src).reshape(n_group, g, n_rep)
    phy2log = torch.cat([own, mirrored], dim=-1).reshape(-1)

    # Logical -> physical pairs, original first.
    phys = torch.arange(ep_size * pl, dtype=torch.int64).reshape(ep_size, pl)
    log2phy = torch.full((n_logical, 2), -1, dtype=torch.int64)
    log2phy[phy2log.reshape(ep_size, pl)[:, :ll].reshape(-1), 0] = phys[:, :ll].reshape(-1)
    log2phy[phy2log.reshape(ep_size, pl)[:, ll:].reshape(-1), 1] = phys[:, ll:].reshape(-1)
    if bool((log2phy[:, 0] < 0).any()):
        raise ValueError("placement does not cover every logical expert exactly once")
    logcnt = (log2phy >= 0).sum(1)

    # Which LP variable governs each replicated logical expert: (ep_rank, d) flattened.
    log2edge = torch.full((n_logical,), -1, dtype=torch.int64)
    rank_ids = torch.arange(ep_size).view(n_group, g, 1, 1).expand(n_group, g, c, d)
    dup_ids = torch.arange(d).view(1, 1, 1, d).expand(n_group, g, c, d)
    log2edge[bundles.reshape(-1)] = (rank_ids * d + dup_ids).reshape(-1)

    # Cross-check replica location against the inverse topology.
    o2r = invert_r2o(r2o_cpu).to(torch.int64)
    holder = (torch.arange(n_group).view(n_group, 1, 1, 1) * g + o2r.view(1, g, 1, d)).expand(n_group, g, c, d)
    slot = (ll + torch.arange(c).view(1, 1, c, 1) * d + torch.arange(d).view(1, 1, 1, d)).expand(n_group, g, c, d)
    expect = (holder * pl + slot).reshape(-1)
    if not torch.equal(log2phy[bundles.reshape(-1), 1], expect):
        raise AssertionError("replica slots disagree with the inverse topology")

    i32 = torch.int32
    return ExpertMapping(phy2log.to(i32), log2phy.to(i32), logcnt.to(i32), log2edge.to(i32))
