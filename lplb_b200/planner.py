"""Public API: the per-batch token re-router for expert-parallel MoE.

``Planner`` keeps the constructor arguments, method names and tensor shapes of the
reference's ``lplb.Planner`` (reference ``lplb/planner.py:38-266``) so that a training
loop written against it runs unchanged:

.. code-block:: python

    planner = Planner(r2o, n_physical, n_logical, group=ep_group)
    planner.update_redundancy_mapping(history)         # every N steps
    phys = planner.run(indices, avail_counter, n_sms)  # every batch

Differences that a user can observe, all deliberate:

* ``run`` is one kernel launch (histogram, NVLink statistics exchange, LP, redirect) when
  the statistics travel over peer memory or not at all; the three-stage pipeline with
  ``torch.distributed.all_reduce`` remains as ``comm="nccl"``.
* The shares come from a primal-dual interior-point method that stops on a duality-gap
  test (``tol``), not from five affine-scaling steps; they are always inside ``[0, 1]``.
* ``avail_counter`` may be int32 or int64 and counts converged groups per call.
* ``device``/``n_nodes`` are explicit, so everything up to and including the LP runs on
  a CPU device too (used by the CPU test-suite).
* Waits on other GPUs are bounded; their outcome is visible through ``check_status``.
"""

from __future__ import annotations

import contextlib
import logging
import os
from typing import Any

import torch

from . import lp as _lp
from .mapping import ExpertMapping, build_mapping
from .ops import reference as _ref
from .parallel.exchange import PeerExchangeUnavailable
from .topology import invert_r2o, validate_r2o

log = logging.getLogger("lplb_b200")

__all__ = ["Planner", "PlannerStatus"]

_NO_RANGE = contextlib.nullcontext()

_ERR_NAMES = {
    0: "ok",
    1: "grid_timeout",
    2: "peer_timeout",
    3: "lp_timeout",
    4: "bad_index",
    5: "lp_not_converged",
    6: "index_out_of_bounds",
}
_PHASE_NAMES = {0: "-", 1: "count", 2: "exchange", 3: "solve", 4: "redirect"}


class PlannerStatus(dict):
    """Decoded status block of the native engine (see ``csrc/common.cuh``)."""

    @property
    def ok(self) -> bool:
        return self["error"] == "ok"


class Planner:
    def __init__(
        self,
        redundant_to_original: torch.Tensor,
        n_routed_experts: int,
        n_logical_routed_experts: int,
        ep_size: int | None = None,
        group: "torch.distributed.ProcessGroup | None" = None,
        *,
        device: torch.device | str | None = None,
        n_nodes: int | None = None,
        comm: str = "auto",
        max_iters: int = 24,
        tol: float = 1e-4,
        peer_timeout_us: float = 1e6,
        grid_timeout_us: float = 1e6,
        allow_self_edges: bool = False,
        warm_start: bool = True,
        warm_guard: float = 0.1,
        warm_snap_mu: float = 1e-3,
        exchange_node_size: int = 0,
        solver: str = "auto",
    ) -> None:
        """
        :param redundant_to_original: ``[group_size, num_redundants]``; rank ``i``'s
            ``d``-th redundant slot is a copy of rank ``r2o[i, d]``'s ``d``-th
            replicated expert.  Every column must be a permutation of the ranks.  The
            real number of redundant experts per rank may be a multiple ``C`` of
            ``num_redundants``; ``C`` experts then share one LP variable.
        :param n_routed_experts: physical experts in total (logical + redundant).
        :param n_logical_routed_experts: logical experts in total.
        :param ep_size: EP ranks; defaults to ``group.size()``.
        :param group: EP process group.  ``None`` means statistics are not exchanged.
        :param device: where the planner's tensors live; default ``cuda`` if available.
        :param n_nodes: nodes seen by the placement balancer; default
            ``max(1, ep_size // gpus_per_host)``.
        :param comm: ``"p2p"`` exchanges statistics inside the kernel over NVLink peer
            memory, ``"nccl"`` uses ``torch.distributed.all_reduce`` between kernels,
            ``"none"`` never exchanges, ``"auto"`` picks ``p2p`` when every rank of the
            group is on this host and falls back to ``nccl``.
        :param max_iters, tol: interior-point iteration cap and relative duality gap.
        :param peer_timeout_us, grid_timeout_us: budgets of the in-kernel waits.
        :param warm_start: start every solve from a centred iterate saved by the last cold
            solve of the same group, as long as the new statistics still fit it (largest row
            residual at most ``warm_guard`` mean rank loads); typically one or two iterations
            instead of three to five when consecutive batches come from one distribution.
            Shares then depend on the planner's history, not only on the current batch; every
            rank keeps its own (normally identical) state.  ``update_redundancy_mapping``,
            ``reset_exchange`` and a step whose statistics exchange timed out discard the state
            (that step and the next one solve cold).  On by default; ``False`` solves every batch
            from scratch.
        :param exchange_node_size: run the in-kernel statistics exchange in two levels, inside
            nodes of this many consecutive ranks and then between nodes (the schedule for a
            topology that spans nodes, e.g. ``torus(2, 4)`` with 4); 0 = one all-to-all level.
        :param solver: device LP solver: ``"warp"`` keeps a group of up to 32 ranks (4 replicas
            per rank) in one warp's registers, ``"block"`` solves a group of up to 128 ranks
            (8 replicas per rank) with one thread block and the matrix in shared memory,
            ``"auto"`` uses the warp solver up to 8 ranks and the block solver above.  Larger
            groups run the same method as tensor ops on the planner's device.
        """
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())

        validate_r2o(redundant_to_original, allow_self_edges=allow_self_edges)
        self.r2o = redundant_to_original.to(self.device, torch.int32).contiguous()
        self.o2r = invert_r2o(redundant_to_original.cpu()).to(self.device)
        self.group_size, self.num_redundants = int(self.r2o.shape[0]), int(self.r2o.shape[1])

        self.n_routed_experts = int(n_routed_experts)
        self.n_logical_routed_experts = int(n_logical_routed_experts)
        if ep_size is None:
            if group is None:
                raise ValueError("ep_size must be provided when group is None")
            ep_size = group.size()
        self.ep_size = int(ep_size)
        if self.ep_size % self.group_size:
            raise ValueError(f"ep_size {self.ep_size} is not a multiple of the topology's {self.group_size} ranks")
        self.n_group = self.ep_size // self.group_size
        if self.n_routed_experts % self.ep_size or self.n_logical_routed_experts % self.ep_size:
            raise ValueError("expert counts must be multiples of ep_size")
        self.n_local_routed_experts = self.n_routed_experts // self.ep_size
        self.n_local_logical_routed_experts = self.n_logical_routed_experts // self.ep_size
        extra = self.n_local_routed_experts - self.n_local_logical_routed_experts
        if extra <= 0 or extra % self.num_redundants:
            raise ValueError(
                f"{extra} redundant experts per rank cannot be split over {self.num_redundants} topology slots"
            )
        self.combined_redundant_experts = extra // self.num_redundants

        if n_nodes is None:
            per_host = torch.cuda.device_count() if torch.cuda.is_available() else 0
            n_nodes = max(1, self.ep_size // per_host) if per_host else 1
        self.n_nodes = int(n_nodes)
        self.max_iters, self.tol = int(max_iters), float(tol)
        self.ep_group = group
        self.deep_ep_initialized = False  # name kept from the reference: "in-kernel exchange is live"
        self._n_sms_default: int | None = None
        self.warm_start, self.warm_guard, self.warm_snap_mu = bool(warm_start), float(warm_guard), float(warm_snap_mu)
        self._anchor: dict | None = None  # CPU path only; the engine keeps its own on the device
        self.exchange_node_size = int(exchange_node_size)
        self._host_out: tuple | None = None
        self._staged_probs: torch.Tensor | None = None
        self._status_mirror: list | None = None
        self._nvtx_on = self.device.type == "cuda" and os.environ.get("LPLB_B200_NVTX") == "1"

        self._engine = None
        self._native_solver = False
        if self.device.type == "cuda":
            from . import _native

            native = _native.load()  # raises if the extension is missing: no silent fallback on a GPU
            self._engine = native.PlannerEngine(
                self.n_group,
                self.group_size,
                self.num_redundants,
                self.n_local_logical_routed_experts,
                self.combined_redundant_experts,
                self.device.index,
            )
            if solver != "auto":
                self._engine.set_solver(solver)
            self._native_solver = bool(self._engine.has_native_solver())
            if not self._native_solver:
                log.warning(
                    "group of %d ranks x %d replicas exceeds the device solvers; the LP runs as tensor ops "
                    "with host synchronisation (slow path)",
                    self.group_size, self.num_redundants,
                )
            self._engine.set_topology(self.r2o, self.o2r)
            self._engine.set_params(self.max_iters, self.tol, float(peer_timeout_us), float(grid_timeout_us))
            self._engine.set_warm_start(bool(warm_start), float(warm_guard), float(warm_snap_mu))

        self.mapping: ExpertMapping
        self.phy2log: torch.Tensor
        self.update_redundancy_mapping()

        if comm not in ("auto", "p2p", "nccl", "none"):
            raise ValueError(f"unknown comm mode {comm!r}")
        self.comm = "none"
        if group is not None and comm != "none" and group.size() > 1:
            self.comm = "nccl"
            if comm in ("auto", "p2p") and self._engine is not None:
                # init_peer_exchange fails on every rank of the group or on none, so all ranks
                # take the same branch here and nobody mixes transports with its peers
                try:
                    self.init_peer_exchange()
                except PeerExchangeUnavailable as exc:
                    if comm == "p2p":
                        raise
                    log.warning("peer-memory exchange unavailable (%s); using torch.distributed.all_reduce", exc)

    # ------------------------------------------------------------------ communicator
    def init_peer_exchange(self) -> None:
        """Bring up the in-kernel NVLink statistics exchange (collective over the group).

        Allocates this rank's receive buffers, all-gathers CUDA-IPC handles through
        ``torch.distributed`` and maps every peer.  Raises ``PeerExchangeUnavailable`` on
        every rank if any rank cannot take part (a rank on another host, an allocation or a
        mapping that failed).  Counterpart of the reference's ``init_comm``
        (reference ``csrc/plugin.cpp:357-456``), minus NVSHMEM.
        """
        from .parallel.exchange import open_peer_exchange

        if self.deep_ep_initialized:
            return
        if self._engine is None or self.ep_group is None:
            raise RuntimeError("peer exchange needs a CUDA device and a process group")
        if self.exchange_node_size and self.ep_group.size() % self.exchange_node_size:
            raise ValueError("exchange_node_size must divide the number of ranks")
        open_peer_exchange(self._engine, self.ep_group, self.device)
        if self.exchange_node_size:
            self._engine.set_exchange_nodes(self.exchange_node_size)
        self.deep_ep_initialized = True
        self.comm = "p2p"

    def init_from_deep_ep(self, buffer: Any = None) -> None:
        """Switch to the in-kernel exchange (API of reference ``lplb/planner.py:104-113``).

        The reference borrows DeepEP's NVSHMEM state here.  This build needs nothing from
        the buffer: all ranks of one NVLink domain are reached through peer memory that
        the planner maps itself, so the argument is accepted and ignored.
        """
        self.init_peer_exchange()

    def invalidate_warm_start(self) -> None:
        """Forget the saved iterates; the next solve of every group starts cold."""
        self._anchor = None
        if self._engine is not None:
            self._engine.invalidate_warm_start()

    def reset_exchange(self) -> None:
        """Collective: re-zero epochs, flags and buffers on every rank (e.g. after a timeout)."""
        self._anchor = None
        if self._engine is None:
            return
        # this rank's launches store into the peers' buffers: drain them before any peer clears its own
        torch.cuda.synchronize(self.device)
        if self.ep_group is not None:
            torch.distributed.barrier(group=self.ep_group)
        self._engine.reset_exchange()
        if self.ep_group is not None:
            torch.distributed.barrier(group=self.ep_group)

    # ------------------------------------------------------------------ slow path
    def update_redundancy_mapping(
        self, workload: torch.Tensor | None = None
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Re-place experts from load history and rebuild every lookup table.

        Returns ``(phy2log [P], log2phy [E, 2], logcnt [E])`` int32 on the planner's
        device (reference ``lplb/planner.py:115-182``).  Moving the expert *weights* to
        match ``phy2log`` is the caller's job, as in the reference.
        """
        mapping = build_mapping(
            self.r2o,
            self.n_group,
            self.n_local_logical_routed_experts,
            self.combined_redundant_experts,
            workload,
            n_nodes=self.n_nodes,
        )
        assert mapping.phy2log.numel() == self.n_routed_experts
        self._anchor = None  # a new placement is a new LP
        self.mapping = mapping.to(self.device)
        self.phy2log = self.mapping.phy2log
        if self._engine is not None:
            self._engine.set_mapping(self.mapping.phy2log, self.mapping.log2phy, self.mapping.log2edge)
        return self.mapping.phy2log, self.mapping.log2phy, self.mapping.logcnt

    # ------------------------------------------------------------------ stages
    def _default_sms(self) -> int:
        if self._n_sms_default is None:
            if self.device.type == "cuda":
                self._n_sms_default = torch.cuda.get_device_properties(self.device).multi_processor_count
            else:
                self._n_sms_default = 8
        return self._n_sms_default

    def _default_ctas(self, n_idx: int) -> int:
        """CTAs of the single launch when the caller names none: one per SM for large batches,
        fewer for small ones.  A worker CTA should get at least 384 indices (1.5 per thread);
        below that more CTAs only add arrivals and atomics (4096 tokens x top-8 on a B200:
        25.0 us with 74 or 111 CTAs, 25.8 us with 148, 25.3 us with 38)."""
        return max(2, min(self._default_sms(), 1 + -(-int(n_idx) // 384)))

    def count_workload(self, idx: torch.Tensor, n_sms: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Count logical expert ids in ``idx`` (``-1`` is skipped).

        :return: ``(counts [E] int32, inclusive prefix over the n_sms token slices [n_sms, E])``
            (reference ``lplb/planner.py:184-194``).
        """
        if self._engine is not None:
            return self._engine.count_idx(idx.contiguous(), int(n_sms))
        return _ref.count_reference(idx, self.n_logical_routed_experts, int(n_sms))

    def solve_probs(self, workload: torch.Tensor, avail_counter: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Solve every group's LP for the given per-expert statistics.

        :param workload: ``numel == n_logical`` counts of this rank (summed over the
            group first when a communicator is set).
        :param avail_counter: one-element integer tensor, incremented once per group
            whose LP converged.
        :return: ``(probs [NG, G, D] float32, workload / max(workload) [NG, G, Ll] float32)``
            (reference ``lplb/planner.py:196-217`` returns the same pair).
        """
        shape = (self.n_group, self.group_size, self.n_local_logical_routed_experts)
        if self._engine is not None:
            wl = workload.reshape(-1).to(torch.int32).contiguous()
            if self.comm == "p2p":
                wl = self._engine.all_reduce_counts(wl)
            elif self.comm == "nccl":
                wl = wl.clone()
                torch.distributed.all_reduce(wl, group=self.ep_group)
            if self._native_solver:
                probs, normalised = self._engine.solve(wl, avail_counter)
                return probs, normalised.view(shape)
            # Groups beyond the device solvers (more than 128 ranks or 8 replicas per rank): the
            # same interior-point method as batched tensor ops on the planner's device.  Nothing
            # is copied to the host, but the iteration's loop control reads device flags, so this
            # path synchronises the host several times per call.
            w, fixed = _lp.bundle_loads(
                wl.double(), self.phy2log, self.n_group, self.group_size, self.num_redundants,
                self.n_local_logical_routed_experts, self.combined_redundant_experts,
            )
            res = _lp.solve_ipm(
                w, fixed, self.r2o, max_iters=self.max_iters, tol=self.tol, warm_start=self.warm_start,
                anchor=self._anchor, guard=self.warm_guard, snap_mu=self.warm_snap_mu,
            )
            self._anchor = res.anchor
            avail_counter += res.converged.sum().to(avail_counter.dtype)
            peak = wl.max().clamp_min(1).float()
            return res.f.float(), (wl.float() / peak).view(shape)

        wl = workload.reshape(-1).to(torch.int64)
        if self.comm == "nccl":
            wl = wl.clone()
            torch.distributed.all_reduce(wl, group=self.ep_group)
        w, fixed = _lp.bundle_loads(
            wl.double(),
            self.phy2log,
            self.n_group,
            self.group_size,
            self.num_redundants,
            self.n_local_logical_routed_experts,
            self.combined_redundant_experts,
        )
        res = _lp.solve_ipm(
            w, fixed, self.r2o.cpu(), max_iters=self.max_iters, tol=self.tol, warm_start=self.warm_start,
            anchor=self._anchor, guard=self.warm_guard, snap_mu=self.warm_snap_mu,
        )
        self._anchor = res.anchor
        avail_counter += int(res.converged.sum())
        peak = wl.max().clamp_min(1).float()
        return res.f.float().to(self.device), (wl.float() / peak).view(shape)

    def weighted_select_target(
        self,
        idx: torch.Tensor,
        o_weight: torch.Tensor,
        local_workload_by_sm: torch.Tensor,
        n_sms: int,
    ) -> torch.Tensor:
        """Rewrite logical ids to physical ids so that a share ``o_weight`` of every
        replicated expert's local tokens stays on the original
        (reference ``lplb/planner.py:219-243``).  ``n_sms`` must equal the value given to
        ``count_workload``."""
        if self._engine is not None:
            return self._engine.map_idx(
                idx.contiguous(), o_weight.float().contiguous(), local_workload_by_sm, int(n_sms)
            )
        return _ref.redirect_reference(idx, o_weight, self.mapping.log2phy, self.mapping.log2edge)

    # ------------------------------------------------------------------ hot path
    def run(
        self,
        idx: torch.Tensor,
        avail_counter: torch.Tensor,
        n_sms: int | None = None,
        out: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """Logical expert ids ``[-1, E)`` in, physical expert ids ``[-1, P)`` out, same shape
        (reference ``lplb/planner.py:245-266``).

        ``n_sms`` CTAs are launched (default: one per SM, fewer for batches of less than 384
        indices per SM, never fewer than two): one of them exchanges the statistics and solves
        the LPs, the others count and rewrite the indices.

        ``idx`` normally lives on the planner's GPU.  It may instead be a *pinned host* tensor:
        the kernel then reads it over PCIe itself (no separate host-to-device copy), and the
        result is written to ``out``, which may be a pinned host tensor as well (no separate
        device-to-host copy).  Without ``out`` a pinned buffer cached on the planner is
        returned; it is overwritten by the next such call.  The caller synchronises the stream
        before reading a host result."""
        pick_ctas = n_sms is None
        if n_sms is None:
            n_sms = self._default_sms()
        with self._nvtx("lplb_b200.planner.run"):
            # One launch, unless the statistics travel through torch.distributed, or several
            # groups need the thread-block solver: inside the one launch a single CTA would solve
            # them one after the other, the stand-alone solve kernel gives every group a CTA.
            fused = self._engine is not None and self._native_solver and self.comm != "nccl"
            if fused and self.n_group > 1 and self._engine.solver() == "block":
                fused = False
            if fused:
                if not idx.is_cuda and out is None:
                    key = (tuple(idx.shape), idx.dtype)
                    if self._host_out is None or self._host_out[0] != key:
                        self._host_out = (key, torch.empty(idx.shape, dtype=idx.dtype).pin_memory())
                    out = self._host_out[1]
                self._staged_probs = None
                if pick_ctas:
                    n_sms = self._default_ctas(idx.numel())
                return self._engine.run_fused(idx.contiguous(), avail_counter, int(n_sms), self.comm == "p2p", out)
            if not idx.is_cuda and self._engine is not None:
                idx = idx.to(self.device, non_blocking=True)
            local, by_sm = self.count_workload(idx, n_sms)
            probs, _ = self.solve_probs(local, avail_counter)
            self._staged_probs = probs
            res = self.weighted_select_target(idx, probs, by_sm, n_sms)
            if out is not None:
                out.copy_(res, non_blocking=True)
                return out
            return res

    def run_staged(self, idx: torch.Tensor, avail_counter: torch.Tensor, n_sms: int | None = None) -> torch.Tensor:
        """The three-launch pipeline regardless of ``comm`` (baseline for measurements)."""
        if n_sms is None:
            n_sms = self._default_sms()
        local, by_sm = self.count_workload(idx, n_sms)
        probs, _ = self.solve_probs(local, avail_counter)
        return self.weighted_select_target(idx, probs, by_sm, n_sms)

    @property
    def last_probs(self) -> torch.Tensor | None:
        """Shares ``[NG, G, D]`` computed by the most recent ``run``."""
        if self._staged_probs is not None or self._engine is None:
            return self._staged_probs
        return self._engine.last_probs()

    # ------------------------------------------------------------------ observability
    @staticmethod
    def _decode_status(raw: list[int]) -> PlannerStatus:
        out = PlannerStatus(
            error=_ERR_NAMES.get(raw[0], str(raw[0])),
            phase=_PHASE_NAMES.get(raw[1], str(raw[1])),
            detail=raw[2],
            calls=raw[3],
            lp_iters=raw[4],
            lp_failures=raw[5],
            timeouts=raw[6],
            bad_indices=raw[7],
            lp_gap=raw[8] * 1e-9,
        )
        if raw[0] == 6 or raw[11]:
            out.update(bounds_line=raw[2], bounds_index=raw[9], bounds_limit=raw[10], bounds_skipped=raw[11])
        return out

    def check_status(self, clear: bool = False) -> PlannerStatus:
        """Read the engine's status block (one small blocking device-to-host copy).

        ``lp_gap`` is the largest relative duality gap among the groups of the last launch,
        ``lp_iters`` the iterations of its slowest group; the other counters are cumulative."""
        if self._engine is None:
            return PlannerStatus(error="ok", phase="-", detail=0, calls=0, lp_iters=0, lp_failures=0, timeouts=0,
                                 bad_indices=0, lp_gap=0.0)
        out = self._decode_status(self._engine.status().cpu().tolist())
        if clear:
            self._engine.status().zero_()
        return out

    def poll_status(self) -> PlannerStatus | None:
        """Status without stalling the host: every call enqueues a copy of the status block into
        pinned host memory on the current stream and returns the decoded result of the most
        recent copy that has *completed* (``None`` until the first one has).  Meant to be
        called once per step from a training loop: the answer lags the device by a step or
        so and costs no synchronisation."""
        if self._engine is None:
            return self.check_status()
        if self._status_mirror is None:
            self._status_mirror = [
                (torch.empty(16, dtype=torch.int32).pin_memory(), torch.cuda.Event()) for _ in range(2)
            ]
            self._status_pending: list[int] = []
            self._status_last: PlannerStatus | None = None
        # newest completed copy wins; keep at most two in flight
        while self._status_pending and self._status_mirror[self._status_pending[0]][1].query():
            slot = self._status_pending.pop(0)
            self._status_last = self._decode_status(self._status_mirror[slot][0].tolist())
        if len(self._status_pending) < 2:
            slot = next(i for i in range(2) if i not in self._status_pending)
            buf, event = self._status_mirror[slot]
            buf.copy_(self._engine.status(), non_blocking=True)
            event.record()
            self._status_pending.append(slot)
        return self._status_last

    def _nvtx(self, name: str):
        """NVTX range around the hot path when LPLB_B200_NVTX=1 (for timeline profilers)."""
        if self._nvtx_on:
            return torch.cuda.nvtx.range(name)
        return _NO_RANGE

    def dump_lp(self, workload: torch.Tensor) -> dict[str, Any]:
        """Everything the solver sees for the given (already summed) statistics, on the host:
        bundle loads, fixed loads, the compact form ``M, base`` and the equality form
        ``A, b, c`` of every group, plus the float64 oracle's shares and optimum.  This is the
        inspectable counterpart of the reference's compile-time ``DEBUG_DUMP`` printf of
        ``A``, ``b``, ``c`` and ``x`` (reference ``lplb/resources/csrc-tmpl/minilp.cu:295-321``)."""
        wl = workload.detach().reshape(-1).to("cpu", torch.float64)
        r2o = self.r2o.cpu()
        w, fixed = _lp.bundle_loads(
            wl, self.phy2log.cpu(), self.n_group, self.group_size, self.num_redundants,
            self.n_local_logical_routed_experts, self.combined_redundant_experts,
        )
        m, base = _lp.compact_form(w, fixed, r2o)
        oracle = _lp.solve_ipm(w, fixed, r2o, tol=1e-9, max_iters=60)
        standard = [_lp.standard_form(w[g], fixed[g], r2o) for g in range(self.n_group)]
        return {
            "bundle_loads": w, "fixed_loads": fixed, "M": m, "base": base,
            "A": [t[0] for t in standard], "b": [t[1] for t in standard], "c": [t[2] for t in standard],
            "oracle_shares": oracle.f, "oracle_max_load": oracle.t, "oracle_iterations": oracle.iters,
        }

    def enable_trace(self, on: bool = True) -> None:
        """Make the fused kernel write per-phase ``globaltimer`` stamps (a few extra stores)."""
        if self._engine is not None:
            self._engine.enable_trace(bool(on))

    def phase_times_us(self) -> dict[str, float] | None:
        """Phase durations of the last fused ``run`` in microseconds; synchronises.

        ``count`` is the time until the first worker CTA had counted its slice, ``last_count``
        the further wait until all counts were in; ``exchange`` and ``solve`` belong to the solver
        CTA; ``redirect`` ends when the first worker has rewritten its slice, ``drain`` when the
        last one has.  With a peer exchange the ``exchange`` phase is split further, measured from its
        start: ``xchg_pushed`` (this rank's stores to all peers issued), ``xchg_first_peer`` and
        ``xchg_last_peer`` (first and last word of another rank seen), and ``xchg_last_peer_rank``;
        what lies between ``xchg_pushed`` and ``xchg_last_peer`` is wire time plus waiting for the
        slowest rank.  A two-level exchange reports its second level as ``xchg2_*``."""
        if self._engine is None or self._engine.trace() is None:
            return None
        t = self._engine.trace().cpu().tolist()
        out = {
            "count": (t[1] - t[0]) / 1e3,
            "last_count": (t[2] - t[1]) / 1e3,
            "exchange": (t[3] - t[2]) / 1e3,
            "solve": (t[4] - t[3]) / 1e3,
            "redirect": (t[5] - t[4]) / 1e3,
            "drain": (t[6] - t[5]) / 1e3,
            "total": (t[6] - t[0]) / 1e3,
        }
        if self.comm == "p2p":
            for base, tag in ((8, "xchg"), (12, "xchg2")):
                if t[base] and t[base] >= t[2]:
                    out[f"{tag}_pushed"] = (t[base] - t[2]) / 1e3
                    out[f"{tag}_first_peer"] = (t[base + 1] - t[2]) / 1e3
                    out[f"{tag}_last_peer"] = (t[base + 2] - t[2]) / 1e3
                    out[f"{tag}_last_peer_rank"] = int(t[base + 3])
        return out

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict[str, Any]:
        """Everything needed to resume with the same placement (the reference keeps no
        such state: its ``phy2log`` lives only on the object, ``lplb/planner.py:180``)."""
        return {
            "r2o": self.r2o.cpu(),
            "phy2log": self.mapping.phy2log.cpu(),
            "log2phy": self.mapping.log2phy.cpu(),
            "logcnt": self.mapping.logcnt.cpu(),
            "log2edge": self.mapping.log2edge.cpu(),
            "n_routed_experts": self.n_routed_experts,
            "n_logical_routed_experts": self.n_logical_routed_experts,
            "ep_size": self.ep_size,
        }

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if not torch.equal(state["r2o"].int(), self.r2o.cpu()):
            raise ValueError("checkpoint was written for a different topology")
        for key in ("n_routed_experts", "n_logical_routed_experts", "ep_size"):
            if int(state[key]) != getattr(self, key):
                raise ValueError(f"checkpoint {key}={state[key]} does not match this planner")
        self.mapping = ExpertMapping(
            state["phy2log"].int(), state["log2phy"].int(), state["logcnt"].int(), state["log2edge"].int()
        ).to(self.device)
        self.phy2log = self.mapping.phy2log
        self._anchor = None  # saved iterates belong to the placement that was replaced
        if self._engine is not None:
            self._engine.set_mapping(self.mapping.phy2log, self.mapping.log2phy, self.mapping.log2edge)
