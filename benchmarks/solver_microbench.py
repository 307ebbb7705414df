#!/usr/bin/env python
"""Single-GPU LP solver microbenchmark.

Seeded random instances of the EP8 Cube LP (2 redundant experts per rank, 16 logical
experts per rank): per-expert loads are drawn from a multinomial over 128 experts,
32768 tokens x top-8, with Dirichlet(0.3) expert probabilities; on every rank the two
heaviest experts are the replicated ones.  Reports

* the latency of one ``solve_probs`` call that solves a single group (the case a
  training step sees), timed with CUDA events, L2 flushed between calls;
* the throughput of batched calls (64 groups per launch);
* the objective gap of the returned shares against the float64 oracle, and the gap of
  the reference's five-step affine-scaling method restated on the CPU, for comparison.

Usage: python benchmarks/solver_microbench.py [--instances 10000] [--json out.json]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube, lp  # noqa: E402


def draw(rng, n):
    cnt = np.stack([
        -np.sort(-rng.multinomial(32768 * 8, rng.dirichlet(np.full(128, 0.3))).reshape(8, 16), axis=1) for _ in range(n)
    ])
    return cnt  # [n, 8, 16], heaviest first on every rank


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--instances", type=int, default=10000)
    ap.add_argument("--latency-calls", type=int, default=200)
    ap.add_argument("--affine-sample", type=int, default=200)
    ap.add_argument("--tol", type=float, default=1e-4)
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(0)
    batch = 64
    n_batches = -(-args.instances // batch)
    r2o = cube()

    # unrelated instances follow one another, so every solve starts from scratch
    big = Planner(r2o, (128 + 16) * batch, 128 * batch, 8 * batch, device=dev, tol=args.tol, warm_start=False)
    one = Planner(r2o, 128 + 16, 128, 8, device=dev, tol=args.tol, warm_start=False)
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    gaps, iters_hist, batch_us = [], [], []
    first = None
    for b in range(n_batches):
        cnt = draw(rng, batch)
        if first is None:
            first = cnt
        current = torch.from_numpy(cnt.reshape(-1)).int().to(dev)
        big.solve_probs(current, avail)  # warm-up of this shape
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.fill_(b & 0xFF)
        start.record()
        probs, _ = big.solve_probs(current, avail)
        end.record()
        torch.cuda.synchronize()
        batch_us.append(start.elapsed_time(end) * 1e3)
        w = torch.from_numpy(cnt[:, :, :2].astype(np.float64))
        fixed = torch.from_numpy(cnt[:, :, 2:].sum(-1).astype(np.float64))
        realised = lp.rank_loads(probs.cpu().double(), w, fixed, r2o).max(-1).values
        oracle = lp.solve_ipm(w, fixed, r2o, tol=1e-7, max_iters=40)
        gaps.extend(((realised - oracle.t) / oracle.t).tolist())
        iters_hist.append(big.check_status()["lp_iters"])
    gaps = np.array(gaps[: args.instances])

    # latency of a single-group call
    lat = []
    for k in range(args.latency_calls + 10):
        current = torch.from_numpy(first[k % batch].reshape(-1)).int().to(dev)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.fill_(k & 0xFF)
        start.record()
        one.solve_probs(current, avail)
        end.record()
        torch.cuda.synchronize()
        if k >= 10:
            lat.append(start.elapsed_time(end) * 1e3)

    # the reference's method, restated on the CPU, on a sample
    ref_gaps, ref_ok = [], 0
    for i in range(min(args.affine_sample, batch)):
        w = torch.from_numpy(first[i, :, :2].astype(np.float64))
        fixed = torch.from_numpy(first[i, :, 2:].sum(-1).astype(np.float64))
        _, t_opt = lp.solve_highs(w, fixed, r2o)
        _, t_ref, ok = lp.affine_scaling_reference(w, fixed, r2o)
        ref_ok += ok
        ref_gaps.append((t_ref - t_opt) / t_opt)

    result = {
        "instances": int(len(gaps)),
        "tol": args.tol,
        "single_group_call_us": {"p50": round(statistics.median(lat), 2), "min": round(min(lat), 2), "mean": round(statistics.mean(lat), 2)},
        "batched_64_groups_call_us": {"p50": round(statistics.median(batch_us), 2), "per_instance_us": round(statistics.median(batch_us) / batch, 3)},
        "objective_gap_vs_float64": {"mean": float(gaps.mean()), "max": float(gaps.max()), "min": float(gaps.min())},
        "max_iterations": int(max(iters_hist)),
        "reference_method_cpu_restatement": {
            "sample": len(ref_gaps), "accepted": int(ref_ok),
            "gap_mean": float(np.mean(ref_gaps)), "gap_max": float(np.max(ref_gaps)),
        },
        "timing": "CUDA events around one solve_probs call (H2D of the counts excluded), 256 MiB L2 flush before each",
    }
    print(json.dumps(result))
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        with open(args.json, "w") as fh:
            json.dump(result, fh, indent=1)


if __name__ == "__main__":
    main()
