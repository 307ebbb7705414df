"""Embedded expert-placement balancer (the slow path that runs every N steps).

Given per-expert load statistics it decides which logical expert sits in which
physical slot so that ranks (and nodes) carry similar load.  The planner calls it
with ``num_replicas == num_logical`` so it only *reorders* experts; replication
is supported for completeness because the reference exposes it.

Behaviour follows the reference's embedded EPLB (reference ``lplb/eplb.py:6-190``):
longest-processing-time greedy packing into equal-cardinality packs, greedy
replication of the expert with the highest per-replica load, and a hierarchical
policy groups -> nodes -> GPUs.  The implementation is vectorised over layers
(one masked arg-min per placed item for all layers at once) instead of nested Python
loops per layer, and never touches a CUDA API, so it runs on GPU-less hosts.
"""

from __future__ import annotations

import torch

__all__ = [
    "balanced_packing",
    "replicate_experts",
    "rebalance_experts_hierarchical",
    "rebalance_experts",
]


def _invert_rows(perm: torch.Tensor) -> torch.Tensor:
    """Row-wise inverse of a batch of permutations ``[X, n]``."""
    out = torch.empty_like(perm)
    ar = torch.arange(perm.shape[1], dtype=perm.dtype).expand_as(perm)
    out.scatter_(1, perm, ar)
    return out


def balanced_packing(weight: torch.Tensor, num_packs: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Distribute ``n`` weighted items over ``num_packs`` packs of exactly
    ``n / num_packs`` items each, keeping pack weights close (LPT greedy).

    :param weight: ``[X, n]`` item weights, one independent problem per row.
    :return: ``(pack_index, rank_in_pack)``, both ``[X, n]`` int64 on CPU.

    Items are visited heaviest first (stable order among equals); each goes to the
    lightest pack that still has room, lowest pack id on ties
    (reference ``lplb/eplb.py:6-46``).
    """
    rows, n = weight.shape
    if n % num_packs != 0:
        raise ValueError(f"{n} items cannot fill {num_packs} equal packs")
    cap = n // num_packs
    if cap == 1:
        ident = torch.arange(n, dtype=torch.int64).expand(rows, n).clone()
        return ident, torch.zeros(rows, n, dtype=torch.int64)

    w = weight.detach().to("cpu", torch.float64)
    order = torch.sort(w, dim=1, descending=True, stable=True).indices
    load = torch.zeros(rows, num_packs, dtype=torch.float64)
    fill = torch.zeros(rows, num_packs, dtype=torch.int64)
    pack_index = torch.empty(rows, n, dtype=torch.int64)
    rank_in_pack = torch.empty(rows, n, dtype=torch.int64)
    row_ids = torch.arange(rows)
    inf = torch.tensor(float("inf"), dtype=torch.float64)
    for step in range(n):
        item = order[:, step]
        choice = torch.where(fill < cap, load, inf).argmin(dim=1)
        pack_index[row_ids, item] = choice
        rank_in_pack[row_ids, item] = fill[row_ids, choice]
        load[row_ids, choice] += w[row_ids, item]
        fill[row_ids, choice] += 1
    return pack_index, rank_in_pack


def replicate_experts(
    weight: torch.Tensor, num_phy: int
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Grow ``num_log`` experts to ``num_phy`` physical slots by repeatedly adding a
    replica to the expert whose per-replica load is highest.

    :return: ``(phy2log [X, num_phy], replica_rank [X, num_phy], logcnt [X, num_log])``

    With ``num_phy == num_log`` this is the identity, which is how the planner uses
    it (reference ``lplb/eplb.py:49-77``).
    """
    rows, num_log = weight.shape
    extra = num_phy - num_log
    if extra < 0:
        raise ValueError("num_phy must be >= the number of logical experts")
    w = weight.detach().to("cpu", torch.float64)
    logcnt = torch.ones(rows, num_log, dtype=torch.int64)
    phy2log = torch.empty(rows, num_phy, dtype=torch.int64)
    phy2log[:, :num_log] = torch.arange(num_log)
    replica_rank = torch.zeros(rows, num_phy, dtype=torch.int64)
    row_ids = torch.arange(rows)
    for slot in range(num_log, num_phy):
        hottest = (w / logcnt).argmax(dim=1)
        phy2log[:, slot] = hottest
        replica_rank[:, slot] = logcnt[row_ids, hottest]
        logcnt[row_ids, hottest] += 1
    return phy2log, replica_rank, logcnt


def rebalance_experts_hierarchical(
    weight: torch.Tensor,
    num_physical_experts: int,
    num_groups: int,
    num_nodes: int,
    num_gpus: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Three-stage placement: expert groups -> nodes, replicas within a node,
    physical experts -> GPUs of the node (reference ``lplb/eplb.py:80-148``).

    :return: ``(phy2log [L, P], replica_rank [L, P], logcnt [L, E])``
    """
    layers, num_log = weight.shape
    for what, a, b in (
        ("logical experts / groups", num_log, num_groups),
        ("groups / nodes", num_groups, num_nodes),
        ("gpus / nodes", num_gpus, num_nodes),
        ("physical experts / gpus", num_physical_experts, num_gpus),
    ):
        if a % b != 0:
            raise ValueError(f"{what}: {a} is not a multiple of {b}")
    experts_per_group = num_log // num_groups
    groups_per_node = num_groups // num_nodes
    log_per_node = num_log // num_nodes
    phy_per_node = num_physical_experts // num_nodes
    phy_per_gpu = num_physical_experts // num_gpus
    w = weight.detach().to("cpu", torch.float64)

    # Stage 1: whole expert groups to nodes.  "Node-major logical" (nlog) order lists
    # node 0's experts first, then node 1's, ...
    group_load = w.reshape(layers, num_groups, experts_per_group).sum(-1)
    node_of_group, pos_in_node = balanced_packing(group_load, num_nodes)
    group_base = (node_of_group * groups_per_node + pos_in_node) * experts_per_group
    log2nlog = (group_base.unsqueeze(-1) + torch.arange(experts_per_group)).reshape(layers, num_log)
    nlog2log = _invert_rows(log2nlog)

    # Stage 2: replicate inside each node; one independent row per (layer, node).
    node_load = w.gather(1, nlog2log).reshape(layers * num_nodes, log_per_node)
    phy2nlog, phy_rank, nlog_cnt = replicate_experts(node_load, phy_per_node)

    # Stage 3: spread each node's physical experts over its GPUs.
    phy_load = (node_load / nlog_cnt).gather(1, phy2nlog)
    gpu_of_phy, pos_on_gpu = balanced_packing(phy_load, num_gpus // num_nodes)
    slot_of_phy = gpu_of_phy * phy_per_gpu + pos_on_gpu
    phy_of_slot = _invert_rows(slot_of_phy)

    slot2nlog = phy2nlog.gather(1, phy_of_slot).reshape(layers, num_nodes, phy_per_node)
    slot2nlog = slot2nlog + (torch.arange(num_nodes) * log_per_node).view(1, num_nodes, 1)
    slot2log = nlog2log.gather(1, slot2nlog.reshape(layers, num_physical_experts))
    slot_rank = phy_rank.gather(1, phy_of_slot).reshape(layers, num_physical_experts)
    logcnt = nlog_cnt.reshape(layers, num_log).gather(1, log2nlog)
    return slot2log, slot_rank, logcnt


def rebalance_experts(
    weight: torch.Tensor,
    num_replicas: int,
    num_groups: int,
    num_nodes: int,
    num_gpus: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Entry point (reference ``lplb/eplb.py:151-190``).

    :param weight: ``[layers, num_logical_experts]`` load statistics.
    :param num_replicas: number of physical experts, a multiple of ``num_gpus``.
    :return: ``(phy2log [L, P], log2phy [L, E, max_replicas] padded with -1, logcnt [L, E])``

    Uses the hierarchical policy when groups divide evenly over nodes, otherwise a
    single global group on a single node.
    """
    if weight.dim() != 2:
        raise ValueError("weight must be [layers, num_logical_experts]")
    layers, num_log = weight.shape
    if num_groups % num_nodes == 0:
        phy2log, rank, logcnt = rebalance_experts_hierarchical(
            weight, num_replicas, num_groups, num_nodes, num_gpus
        )
    else:
        phy2log, rank, logcnt = rebalance_experts_hierarchical(weight, num_replicas, 1, 1, num_gpus)
    width = int(logcnt.max())
    log2phy = torch.full((layers, num_log * width), -1, dtype=torch.int64)
    log2phy.scatter_(1, phy2log * width + rank, torch.arange(num_replicas).expand(layers, -1))
    return phy2log, log2phy.reshape(layers, num_log, width), logcnt
