"""Benchmark MoE layer that consumes the planner's redirected indices.

SwiGLU experts (``hidden -> 2*inter -> hidden``), top-k routing, expert parallel over the
ranks of one NVLink domain.  A forward pass is::

    logical ids --Planner.run--> physical ids
    count pairs per physical expert, all-gather the counts over peer memory   (plan)
    push every (token, k) hidden state into its expert's rows on the target GPU (dispatch)
    grouped GEMM 1 on tcgen05 + SwiGLU epilogue
    grouped GEMM 2 on tcgen05, epilogue stores rows straight into the source GPU (combine)
    weighted sum over k

The reference ships no model; its ecosystem pairs the planner with DeepEP dispatch/combine
(reference ``scripts/run_ep16_cube8p2e.py:34-40``).  This layer exists to measure what the
balancing buys end to end: per-step time with no balancing, static placement only, and the
per-batch LP.
"""

from __future__ import annotations

import torch

from ..planner import Planner

__all__ = ["MoELayer", "interleave_gate_up"]


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, tile: int = 128) -> torch.Tensor:
    """``[I, H]`` gate and up projections -> ``[2I, H]`` in the kernel's row order: for every
    block of ``tile`` output features, the gate rows followed by the matching up rows."""
    i, h = gate.shape
    return torch.stack([gate.reshape(i // tile, tile, h), up.reshape(i // tile, tile, h)], dim=1).reshape(2 * i, h)


class MoELayer:
    """Expert-parallel SwiGLU MoE layer on the native engine.

    With ``group=None`` a single GPU hosts every physical expert of the (virtual)
    ``ep_size`` ranks; with a process group each rank hosts ``n_physical / ep_size``.
    Weights are random-init and derived from a per-logical-expert seed, so a replica holds
    the same values as its original without any weight traffic.
    """

    def __init__(
        self,
        planner: Planner,
        hidden: int,
        inter: int,
        topk: int,
        max_tokens: int,
        group: "torch.distributed.ProcessGroup | None" = None,
        capacity_factor: float = 2.0,
        seed: int = 0,
        weight_scale: float | None = None,
        capacity_rows: int | None = None,
    ) -> None:
        """``capacity_rows`` sets the receive buffer's size in rows directly (rounded up to a
        multiple of 128) instead of deriving it from ``max_tokens * topk * capacity_factor``.
        Pairs that would land beyond it are dropped by their senders, contribute nothing to
        the output and are reported (``check()`` returns the overflow code)."""
        from .. import _native

        if planner.device.type != "cuda":
            raise RuntimeError("MoELayer needs a CUDA device")
        native = _native.load()
        self.planner = planner
        self.hidden, self.inter, self.topk, self.max_tokens = hidden, inter, topk, max_tokens
        self.device = planner.device
        self.group = group
        self.seed = seed
        self.weight_scale = weight_scale if weight_scale is not None else hidden**-0.5
        if group is None:
            self.n_ranks, self.rank = 1, 0
            self.n_local = planner.n_routed_experts
        else:
            import torch.distributed as dist

            self.n_ranks, self.rank = group.size(), dist.get_rank(group)
            if self.n_ranks != planner.ep_size:
                raise ValueError("the process group must have one rank per EP rank")
            self.n_local = planner.n_local_routed_experts
        # a single GPU receives exactly its own pairs; with peers the LP bounds the imbalance,
        # and `capacity_factor` leaves room for it
        pairs = max_tokens * topk
        wanted = capacity_rows if capacity_rows is not None else int(pairs * (capacity_factor if group is not None else 1.0))
        capacity = int(-(-max(1, int(wanted)) // 128) * 128)
        self.capacity = capacity
        self.engine = native.MoeEngine(
            hidden, inter, self.n_local, self.n_ranks, self.rank, topk, max_tokens, capacity, self.device.index
        )
        handle = bytes(self.engine.alloc())
        if group is None:
            handles = [handle]
        else:
            import torch.distributed as dist

            handles = [None] * self.n_ranks
            dist.all_gather_object(handles, handle, group=group)
        self.engine.open([bytes(h) for h in handles])
        if group is not None:
            dist.barrier(group=group)
        self.fuse_dispatch = False
        self.send_ctas = 0  # fused dispatch only: this many CTAs send rows and run no tiles (0: sender warps in every CTA)
        self._placed_for: torch.Tensor | None = None
        self.place_weights()

    # ------------------------------------------------------------------ weights
    def logical_weights(self, expert: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``(gate [I, H], up [I, H], down [H, I])`` bf16 of one logical expert."""
        g = torch.Generator(device=self.device).manual_seed(self.seed * 100003 + expert)
        shape = dict(device=self.device, generator=g, dtype=torch.float32)
        gate = (torch.randn(self.inter, self.hidden, **shape) * self.weight_scale).bfloat16()
        up = (torch.randn(self.inter, self.hidden, **shape) * self.weight_scale).bfloat16()
        down = (torch.randn(self.hidden, self.inter, **shape) * self.inter**-0.5).bfloat16()
        return gate, up, down

    def place_weights(self) -> None:
        """(Re)materialise this rank's physical expert weights for the planner's current
        placement.  Call after ``Planner.update_redundancy_mapping``."""
        phy2log = self.planner.phy2log
        first = self.rank * self.n_local
        mine = phy2log[first : first + self.n_local].tolist()
        w13 = torch.empty(self.n_local, 2 * self.inter, self.hidden, dtype=torch.bfloat16, device=self.device)
        w2 = torch.empty(self.n_local, self.hidden, self.inter, dtype=torch.bfloat16, device=self.device)
        for slot, expert in enumerate(mine):
            gate, up, down = self.logical_weights(expert)
            w13[slot] = interleave_gate_up(gate, up)
            w2[slot] = down
        self.w13, self.w2 = w13, w2
        self.engine.set_weights(w13, w2)
        self._placed_for = phy2log.clone()

    # ------------------------------------------------------------------ routing policies
    def route(self, logical_idx: torch.Tensor, avail_counter: torch.Tensor, policy: str = "lplb") -> torch.Tensor:
        """Logical -> physical ids.  ``lplb``: per-batch LP; ``static``: always the original
        copy under the current placement (EPLB-style placement only); placement itself is
        whatever ``update_redundancy_mapping`` last produced (identity = no balancing)."""
        if policy == "lplb":
            return self.planner.run(logical_idx, avail_counter)
        if policy == "static":
            original = self.planner.mapping.log2phy[:, 0].to(logical_idx.dtype)
            safe = logical_idx.clamp_min(0)
            return torch.where(logical_idx >= 0, original[safe], torch.full_like(logical_idx, -1))
        raise ValueError(f"unknown routing policy {policy!r}")

    # ------------------------------------------------------------------ forward
    def forward_physical(
        self, x: torch.Tensor, phys_idx: torch.Tensor, weights: torch.Tensor, upto: int = 5, fuse_dispatch: bool | None = None
    ):
        """Run the layer on physical expert ids.  ``fuse_dispatch`` (default: the layer's
        setting) sends the rows from inside the first GEMM kernel, so the tensor cores start on
        an expert as soon as its rows have landed instead of after the whole dispatch."""
        if self._placed_for is None or not torch.equal(self._placed_for, self.planner.phy2log):
            raise RuntimeError("expert placement changed: call place_weights() first")
        n_cta = torch.cuda.get_device_properties(self.device).multi_processor_count
        fuse = self.fuse_dispatch if fuse_dispatch is None else fuse_dispatch
        if fuse:
            self.engine.set_send_ctas(int(self.send_ctas))
        return self.engine.forward(x.contiguous(), phys_idx.contiguous(), weights.float().contiguous(), n_cta, upto, fuse)

    def forward(self, x, logical_idx, weights, avail_counter, policy: str = "lplb"):
        return self.forward_physical(x, self.route(logical_idx, avail_counter, policy), weights)

    def check(self) -> int:
        """First error code raised by the layer's kernels (0 = none); synchronises.  In the
        bounds-checking build an index that left its array is reported as code 6 (the access
        was skipped; ``engine.status()[16:28]`` holds the record)."""
        status = self.engine.status().tolist()
        return int(status[0] or status[16])

    def reset(self) -> None:
        """Re-align the ranks after a timeout: clear every flag, counter and the status block
        and restart the launch numbering.  Collective: every rank calls it between steps."""
        # this rank's kernels store into the peers' buffers: they must have drained before any
        # peer clears its own
        torch.cuda.synchronize(self.device)
        if self.group is not None:
            import torch.distributed as dist

            dist.barrier(group=self.group)
        self.engine.reset()
        if self.group is not None:
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ reference
    def reference_forward(self, x: torch.Tensor, logical_idx: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Plain PyTorch fp32 evaluation of the same layer on logical experts (single process):
        bf16 inputs and weights, fp32 accumulation, bf16 rounding where the kernels round."""
        out = torch.zeros(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
        xf = x.float()
        for expert in logical_idx[logical_idx >= 0].unique().tolist():
            gate, up, down = self.logical_weights(expert)
            tok, k = (logical_idx == expert).nonzero(as_tuple=True)
            h = xf[tok]
            act = torch.nn.functional.silu(h @ gate.float().T) * (h @ up.float().T)
            y = (act.bfloat16().float() @ down.float().T).bfloat16().float()
            out.index_add_(0, tok, y * weights[tok, k].float().unsqueeze(1))
        return out.bfloat16()
