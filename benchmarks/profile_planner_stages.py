#!/usr/bin/env python
"""Small driver for profiler captures of the stand-alone planner kernels (count, solve,
redirect): EP8 Cube, 256 + 16 experts, 4096 tokens x top-8, a handful of launches.

    python benchmarks/profile_planner_stages.py
    ncu --set full --clock-control none -k regex:"count_kernel|solve_kernel|redirect_kernel" -s 9 -c 3 \
        -o planner_stages python benchmarks/profile_planner_stages.py
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube  # noqa: E402


def main():
    dev = torch.device("cuda", 0)
    planner = Planner(cube(), 272, 256, 8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    bias = torch.randn(256, device=dev, generator=g)
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for step in range(4):
        idx = (torch.randn(4096, 256, device=dev, generator=g) + bias).bfloat16().topk(8, dim=-1).indices
        if step == 0:
            planner.update_redundancy_mapping(torch.bincount(idx.reshape(-1), minlength=256))
        flush.fill_(step)
        out = planner.run_staged(idx, avail)
    torch.cuda.synchronize()
    print("ok", int(avail), tuple(out.shape))


if __name__ == "__main__":
    main()
