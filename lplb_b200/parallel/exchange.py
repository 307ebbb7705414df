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

import os
import socket

import torch
import torch.distributed as dist

__all__ = ["host_identity", "same_host", "open_peer_exchange"]


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


def open_peer_exchange(engine, group: dist.ProcessGroup, device: torch.device) -> None:
    """Collective over ``group``: allocate, exchange handles, map peers, synchronise."""
    world, rank = group.size(), dist.get_rank(group)
    if world < 2:
        raise RuntimeError("peer exchange needs at least two ranks")
    if world > 32:
        raise RuntimeError("peer exchange supports at most 32 ranks in one NVLink domain")
    if not same_host(group):
        raise RuntimeError("ranks of the group live on different hosts")
    if os.environ.get("LPLB_B200_DISABLE_P2P") == "1":
        raise RuntimeError("disabled by LPLB_B200_DISABLE_P2P=1")
    with torch.cuda.device(device):
        handle = engine.alloc_exchange(world, rank)
        handles: list[bytes | None] = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        engine.open_exchange([bytes(h) for h in handles])
        torch.cuda.synchronize(device)
    dist.barrier(group=group)
