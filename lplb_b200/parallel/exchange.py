"""Bootstrap of the in-kernel statistics exchange over NVLink peer memory.

``torch.distributed`` is used once, to all-gather one CUDA-IPC handle per rank; after
that the kernels talk to each other with plain stores, release/acquire flags and loads on
peer memory, and no host-side collective is on the per-batch path.  This covers the
intra-node tier of the reference's communicator (reference ``csrc/plugin.cpp:395-448``,
``lplb/resources/csrc-tmpl/minilp.cu:139-163``).  The reference's inter-node tier rides
on NVSHMEM, which this build does not use; a group that spans hosts stays on
``torch.distributed.all_reduce``.
"""

from __future__ import annotations

import contextlib
import os
import socket

import torch
import torch.distributed as dist

__all__ = ["host_identity", "same_host", "open_peer_exchange", "PeerExchangeUnavailable"]


def host_identity() -> str:
    """A string that is equal for two processes iff they share a machine (and boot)."""
    boot = ""
    try:
        with open("/proc/sys/kernel/random/boot_id") as fh:
            boot = fh.read().strip()
    except OSError:
        pass
    return f"{socket.gethostname()}:{boot}"


def same_host(group: dist.ProcessGroup) -> bool:
    ids: list[str | None] = [None] * group.size()
    dist.all_gather_object(ids, host_identity(), group=group)
    return len(set(ids)) == 1


class PeerExchangeUnavailable(RuntimeError):
    """Raised by ``open_peer_exchange`` on *every* rank of the group when any rank could not
    take part; ``reasons`` maps the failing ranks to their error text."""

    def __init__(self, reasons: dict[int, str]):
        self.reasons = dict(reasons)
        super().__init__("; ".join(f"rank {r}: {msg}" for r, msg in sorted(self.reasons.items())))


def _agree(group: dist.ProcessGroup, error: str | None) -> dict[int, str]:
    """All-gather every rank's local outcome (``None`` = fine); returns the failures."""
    seen: list[str | None] = [None] * group.size()
    dist.all_gather_object(seen, error, group=group)
    return {r: msg for r, msg in enumerate(seen) if msg is not None}


def open_peer_exchange(engine, group: dist.ProcessGroup, device: torch.device) -> None:
    """Collective over ``group``: allocate, exchange handles, map peers, synchronise.

    The outcome is the same on all ranks: either every rank returns with its peers mapped, or
    every rank raises :class:`PeerExchangeUnavailable` with its own buffers released.  A rank
    whose local step fails (no memory, a handle that cannot be opened, ``LPLB_B200_DISABLE_P2P=1``
    in its environment) still walks through every collective of the sequence, so the others are
    never left waiting and nobody ends up on a different transport than its peers.
    """
    world, rank = group.size(), dist.get_rank(group)
    if world < 2:
        raise RuntimeError("peer exchange needs at least two ranks")
    if world > 32:
        raise RuntimeError("peer exchange supports at most 32 ranks in one NVLink domain")
    use_cuda = device.type == "cuda"

    # step 1: local allocation, then one all-gather that carries host identity, handle and error
    error: str | None = None
    handle: bytes | None = None
    try:
        if os.environ.get("LPLB_B200_DISABLE_P2P") == "1":
            raise RuntimeError("disabled by LPLB_B200_DISABLE_P2P=1")
        with torch.cuda.device(device) if use_cuda else contextlib.nullcontext():
            handle = bytes(engine.alloc_exchange(world, rank))
    except Exception as exc:  # noqa: BLE001 - reported to the whole group below
        error = f"{type(exc).__name__}: {exc}"
    offers: list[tuple | None] = [None] * world
    dist.all_gather_object(offers, (host_identity(), handle, error), group=group)
    failures = {r: o[2] for r, o in enumerate(offers) if o[2] is not None}
    if not failures and len({o[0] for o in offers}) != 1:
        failures = {r: "ranks of the group live on different hosts" for r in range(world)}

    # step 2: map the peers (only if step 1 worked everywhere), then agree on the outcome
    if not failures:
        error = None
        try:
            with torch.cuda.device(device) if use_cuda else contextlib.nullcontext():
                engine.open_exchange([bytes(o[1]) for o in offers])
                if use_cuda:
                    torch.cuda.synchronize(device)
        except Exception as exc:  # noqa: BLE001
            error = f"{type(exc).__name__}: {exc}"
        failures = _agree(group, error)
    if failures:
        try:
            engine.close_exchange()
        except Exception:  # noqa: BLE001 - nothing was allocated, or it is already gone
            pass
        raise PeerExchangeUnavailable(failures)
    dist.barrier(group=group)
