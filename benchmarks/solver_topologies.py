#!/usr/bin/env python
"""`Planner.solve_probs` latency per topology on one GPU: how the LP solvers scale with the
group size (8 to 128 ranks) and the number of replicas per rank.  `--solvers warp,block` times
both device solvers where both cover the shape; `auto` is what the library picks.

Eight logical experts per rank; every call sees a fresh load vector, 4096 * max(0, N(1, 0.3))
per expert times a per-call factor N(1, 0.05) (consecutive batches of one distribution); one
call per event pair (so the ~6 us launch + event floor is included), 256 MiB L2 flush between
calls.  Each topology is timed cold and with `warm_start=True`.

    python benchmarks/solver_topologies.py [--only hypercube,torus8x4] [--calls 30] [--modes cold]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, topology  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="ring8,cube,hypercube,torus2x4,torus8x4")
    ap.add_argument("--calls", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--modes", default="cold,warm", help="cold: warm_start off; warm: warm_start on")
    ap.add_argument("--solvers", default="auto", help="comma list of auto, warp, block")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    from lplb_b200.utils.timing import ClockSampler, physical_gpu_index

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    rows = []
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.__enter__()
    for name in args.only.split(","):
        r2o = topology.by_name(name)
        g, d = r2o.shape
        n_logical = 8 * g
        gen = torch.Generator(device=dev).manual_seed(g * 10 + d)
        base = (torch.randn(n_logical, device=dev, generator=gen) * 0.3 + 1).clamp_min(0) * 4096
        total = args.warmup + args.calls
        noise = 1 + 0.05 * torch.randn(total, n_logical, device=dev, generator=gen)
        loads = (base * noise).clamp_min(0).int()
        row = {"topology": name, "group_size": g, "replicas_per_rank": d}
        for solver, mode in [(s, m) for s in args.solvers.split(",") for m in args.modes.split(",")]:
            warm = mode == "warm"
            try:
                planner = Planner(r2o, n_logical + d * g, n_logical, g, device=dev, warm_start=warm, solver=solver)
            except RuntimeError:
                continue  # this solver does not cover the shape
            mode = mode if args.solvers == "auto" else f"{mode}_{solver}"
            avail = torch.zeros(1, dtype=torch.int32, device=dev)
            times, iters = [], []
            for it in range(total):
                flush.fill_(it & 255)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                planner.solve_probs(loads[it], avail)
                b.record()
                torch.cuda.synchronize()
                if it >= args.warmup:
                    times.append(a.elapsed_time(b) * 1e3)
                    iters.append(planner.check_status()["lp_iters"])
            row[f"solve_probs_us_p50_{mode}"] = round(statistics.median(times), 1)
            row[f"lp_iterations_mean_{mode}"] = round(sum(iters) / len(iters), 2)
            row[f"all_converged_{mode}"] = int(avail) == total
        rows.append(row)
        print(json.dumps(rows[-1]))
    sampler.__exit__(None, None, None)
    print(json.dumps({"clocks": sampler.summary()}))
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        with open(args.json, "w") as fh:
            json.dump({"rows": rows, "clocks": sampler.summary(),
                       "timing": "CUDA events around one call, L2 flushed between calls"}, fh, indent=1)


if __name__ == "__main__":
    main()
