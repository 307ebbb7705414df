"""Two CPU ranks over gloo: the host-side logic of a distributed planner (statistics
all-reduce, identical shares on every rank, state dict) without any GPU."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    planner = Planner(cube(), 64 + 16, 64, 8, dist.group.WORLD, device="cpu", comm="auto")
    assert planner.comm == "nccl"  # no peer memory on a CPU device: torch.distributed carries the statistics
    g = torch.Generator().manual_seed(100 + rank)
    history = torch.randint(100, 1000, (64,), generator=torch.Generator().manual_seed(1))
    planner.update_redundancy_mapping(history)
    for step in range(3):
        idx = torch.randint(-1, 64, (512, 4), generator=g)
        avail = torch.zeros(1, dtype=torch.int64)
        counts, by_sm = planner.count_workload(idx, 4)
        probs, normalised = planner.solve_probs(counts, avail)
        assert int(avail) == 1
        total = counts.clone()
        dist.all_reduce(total)
        gathered = [torch.empty_like(probs) for _ in range(world)]
        dist.all_gather(gathered, probs)
        assert all(torch.equal(p, probs) for p in gathered)
        single = Planner(cube(), 64 + 16, 64, 8, device="cpu")
        single.load_state_dict(planner.state_dict())
        want, _ = single.solve_probs(total, torch.zeros(1, dtype=torch.int64))
        assert torch.allclose(want, probs, atol=1e-6)
        out = planner.run(idx, avail, 4)
        assert out.shape == idx.shape and bool(((out == -1) == (idx == -1)).all())
    dist.barrier()
    if rank == 0:
        print("CPU_DIST_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
