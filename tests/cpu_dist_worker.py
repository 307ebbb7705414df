"""Two CPU ranks over gloo: the host-side logic of a distributed planner (statistics
all-reduce, identical shares on every rank, state dict) without any GPU."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube  # noqa: E402


class FakeEngine:
    """Stands in for the native engine's exchange calls; `fail_in` makes one of them raise."""

    def __init__(self, fail_in=None):
        self.fail_in, self.opened, self.closed = fail_in, None, 0

    def alloc_exchange(self, world, rank):
        if self.fail_in == "alloc":
            raise MemoryError("no memory for the receive buffers")
        return bytes([rank]) * 64

    def open_exchange(self, handles):
        if self.fail_in == "open":
            raise RuntimeError("peer handle cannot be mapped")
        self.opened = list(handles)

    def close_exchange(self):
        self.closed += 1


def check_bootstrap_outcome_is_collective(rank, world):
    """One rank fails locally (environment switch, allocation, mapping): every rank must get
    PeerExchangeUnavailable naming that rank, nobody hangs, nobody keeps buffers; with no
    failure every rank ends with all handles."""
    from lplb_b200.parallel.exchange import PeerExchangeUnavailable, open_peer_exchange

    cpu = torch.device("cpu")
    group = dist.group.WORLD
    for failing_rank, how in ((1, "env"), (0, "alloc"), (1, "open")):
        engine = FakeEngine(fail_in=how if rank == failing_rank and how != "env" else None)
        if how == "env" and rank == failing_rank:
            os.environ["LPLB_B200_DISABLE_P2P"] = "1"
        try:
            open_peer_exchange(engine, group, cpu)
        except PeerExchangeUnavailable as exc:
            assert list(exc.reasons) == [failing_rank], exc.reasons
            assert engine.closed == 1
        else:
            raise AssertionError(f"rank {rank}: bootstrap succeeded although rank {failing_rank} failed ({how})")
        finally:
            os.environ.pop("LPLB_B200_DISABLE_P2P", None)
    engine = FakeEngine()
    open_peer_exchange(engine, group, cpu)
    assert engine.opened == [bytes([r]) * 64 for r in range(world)] and engine.closed == 0


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # cold solves: the shares are compared with a fresh single-process planner below
    planner = Planner(cube(), 64 + 16, 64, 8, dist.group.WORLD, device="cpu", comm="auto", warm_start=False)
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
    check_bootstrap_outcome_is_collective(rank, world)
    dist.barrier()
    if rank == 0:
        print("CPU_DIST_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
