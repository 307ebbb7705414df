"""Plain PyTorch restatements of the planner kernels.

They run on any device, define the semantics the CUDA kernels are tested against, and
are what ``Planner`` executes when it is built on a CPU device.

* ``count_reference``   – histogram with a per-slice inclusive prefix
  (kernel: ``count_kernel`` in ``csrc/planner_kernels.cuh``).
* ``quotas_reference``  – integer number of each expert's local tokens that stay on the
  original, ``rint(share * total)``.
* ``redirect_reference`` – logical -> physical rewrite with the even-spread rule
  (kernel: ``redirect_kernel``).  Tokens of one expert are numbered in array order here;
  the kernels number them in an order that depends on atomics, so outputs agree as
  multisets per expert, not position by position.
"""

from __future__ import annotations

import torch

__all__ = ["slice_bounds", "count_reference", "quotas_reference", "redirect_reference"]

_BLOCK = 256


def slice_bounds(n: int, n_slices: int, align: int = _BLOCK) -> list[int]:
    """Token range boundaries of the kernels' CTA slices (``slice_begin`` in ``common.cuh``)."""
    per = -(-n // n_slices)
    per = -(-per // align) * align
    return [min(n, per * p) for p in range(n_slices + 1)]


def count_reference(idx: torch.Tensor, n_logical: int, n_slices: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``(counts [E], inclusive prefix over slices [n_slices, E])``, int32; ``-1`` is skipped."""
    flat = idx.reshape(-1).long()
    bounds = slice_bounds(flat.numel(), n_slices)
    rows = torch.zeros(n_slices, n_logical + 1, dtype=torch.int64, device=idx.device)
    for p in range(n_slices):
        part = flat[bounds[p] : bounds[p + 1]]
        valid = (part >= 0) & (part < n_logical)
        part = torch.where(valid, part, torch.full_like(part, n_logical))
        rows[p].scatter_add_(0, part, torch.ones_like(part))
    prefix = rows[:, :n_logical].cumsum(0).to(torch.int32)
    return prefix[-1].clone(), prefix


def quotas_reference(total: torch.Tensor, probs: torch.Tensor, log2edge: torch.Tensor) -> torch.Tensor:
    """Tokens of each expert kept on the original: all of them for unreplicated experts."""
    p = probs.reshape(-1).float()
    p = torch.where(torch.isnan(p), torch.full_like(p, 0.5), p).clamp(0, 1)
    edge = log2edge.long()
    share = torch.where(edge >= 0, p[edge.clamp_min(0)], torch.ones_like(total, dtype=torch.float32))
    q = torch.round(share * total.float()).to(torch.int64)  # round-half-even, like cvt.rni
    return torch.minimum(q.clamp_min(0), total.long())


def redirect_reference(
    idx: torch.Tensor, probs: torch.Tensor, log2phy: torch.Tensor, log2edge: torch.Tensor
) -> torch.Tensor:
    """Rewrite logical ids to physical ids; ``-1`` (and out-of-range ids) map to ``-1``."""
    n_logical = log2phy.shape[0]
    flat = idx.reshape(-1).long()
    valid = (flat >= 0) & (flat < n_logical)
    safe = torch.where(valid, flat, torch.zeros_like(flat))
    total = torch.zeros(n_logical, dtype=torch.int64, device=idx.device)
    total.scatter_add_(0, safe, valid.long())
    quota = quotas_reference(total, probs.to(idx.device), log2edge.to(idx.device))
    # ordinal of every token among the tokens of its expert, in array order
    order = torch.sort(torch.where(valid, flat, torch.full_like(flat, n_logical)), stable=True)
    starts = torch.zeros(n_logical + 2, dtype=torch.int64, device=idx.device)
    starts[1 : n_logical + 1] = total.cumsum(0)
    ordinal = torch.empty_like(flat)
    ordinal[order.indices] = torch.arange(flat.numel(), device=idx.device) - starts[order.values.clamp_max(n_logical)]
    tot = total[safe].clamp_min(1)
    quo = quota[safe]
    keep = (quo >= tot) | ((quo > 0) & ((ordinal * quo) % tot + quo >= tot))
    phys = log2phy.to(idx.device).long()
    keep = keep | (phys[safe, 1] < 0)
    out = torch.where(keep, phys[safe, 0], phys[safe, 1])
    out = torch.where(valid, out, torch.full_like(out, -1))
    return out.reshape(idx.shape).to(idx.dtype)
