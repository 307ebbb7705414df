"""Model-side consumers of the planner: the expert-parallel benchmark MoE layer."""

from .moe import MoELayer, interleave_gate_up

__all__ = ["MoELayer", "interleave_gate_up"]
