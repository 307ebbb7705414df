#!/usr/bin/env python
"""Distributed planner walk-through on one node (the counterpart of the reference's
``scripts/run_ep16_cube8p2e.py``, which needs two nodes and DeepEP).

Run with one rank per GPU, e.g. on 8 GPUs:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/run_ep8_cube.py

Each rank builds a ``Planner`` on the world group (in-kernel NVLink statistics exchange),
re-places experts from a broadcast history, solves the LP for its own random statistics,
checks that every group converged, prints the balance before/after and times the solve
kernel with ``bench_kineto``.  With fewer than 8 ranks a ring topology is used.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube, lp, ring  # noqa: E402
from lplb_b200.utils.timing import bench_kineto  # noqa: E402


def main(n_logical_per_rank: int = 32) -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    r2o = cube() if world == 8 else ring(world)
    red = r2o.shape[1]
    n_logical = n_logical_per_rank * world
    planner = Planner(r2o, n_logical + red * world, n_logical, group=dist.group.WORLD, device=dev)
    planner.init_from_deep_ep(None)  # already live with comm="auto"; kept to show the reference's call

    torch.manual_seed(42 + rank)
    history = (torch.randn(n_logical, device=dev) * 0.15 + 1).clamp_min(0).mul(2**20).int()
    dist.broadcast(history, src=0)
    phy2log, _, _ = planner.update_redundancy_mapping(history)

    current = (torch.randn(n_logical, device=dev) + 1).clamp_min(0).mul(2**12).int()
    avail = torch.zeros((), dtype=torch.int32, device=dev)
    probs, normalised = planner.solve_probs(current, avail)  # exchanges the statistics in-kernel
    assert int(avail) == planner.n_group, "an LP group did not converge"

    total = current.clone()
    dist.all_reduce(total)
    g, d = planner.group_size, planner.num_redundants
    w, fixed = lp.bundle_loads(total.cpu().double(), phy2log.cpu(), planner.n_group, g, d,
                               planner.n_local_logical_routed_experts, planner.combined_redundant_experts)
    before = lp.rank_loads(torch.ones_like(w), w, fixed, r2o)
    after = lp.rank_loads(probs.cpu().double(), w, fixed, r2o)
    seconds = bench_kineto(lambda: planner.solve_probs(current, avail), "solve_kernel", 200)
    if rank == 0:
        print(f"ranks {world}, experts {n_logical}+{red * world}")
        print(f"balance max/mean: {float(before.max() / before.mean()):.4f} -> {float(after.max() / after.mean()):.4f}")
        print(f"solve kernel: {seconds * 1e6:.1f} us average over 200 calls; status {planner.check_status()['error']}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
