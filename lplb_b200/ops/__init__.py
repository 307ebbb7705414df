"""Plain PyTorch statements of the planner's kernels (the numerics oracles and the CPU path)."""

from .reference import count_reference, quotas_reference, redirect_reference, slice_bounds

__all__ = ["count_reference", "quotas_reference", "redirect_reference", "slice_bounds"]
