#!/usr/bin/env python
"""Torus topology sweep over batch size on 8 GPUs, emulated as 2 "nodes" of 4.

Topology torus(2, 4): every rank keeps one replica of an expert of its intra-node neighbour
and one of its inter-node neighbour.  64 logical experts per GPU (512 + 16 in total), top-8,
Zipf(s = 1.1) expert popularity (Gumbel top-k sampling), tokens per rank swept from 128 to
16,384.  For every batch size the script reports

  planner_us        Planner.run device time, max over ranks
  layer_ms_eplb     MoE layer step with placement-only balancing
  layer_ms_lplb     the same step with the per-batch LP (Planner.run inside the timed region)
  load_*            max/mean rank load under both policies

and the smallest batch size from which the LP wins.

Launch: python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/bench_torus_sweep.py [--json out.json]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, ring, torus  # noqa: E402
from lplb_b200.models.moe import MoELayer  # noqa: E402
from lplb_b200.utils.timing import ClockSampler, physical_gpu_index  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts-per-rank", type=int, default=64)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--sizes", default="128,256,512,1024,2048,4096,8192,16384")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--zipf", type=float, default=1.1)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    r2o = torus(2, 4) if world == 8 else (torus(2, world // 2) if world >= 4 else ring(world))
    red = r2o.shape[1]
    n_logical = args.experts_per_rank * world
    sizes = [int(s) for s in args.sizes.split(",")]
    planner = Planner(r2o, n_logical + red * world, n_logical, world, group, device=dev, comm="p2p", n_nodes=2,
                      exchange_node_size=world // 2 if world >= 4 else 0)  # two "nodes": two-level exchange
    layer = MoELayer(planner, args.hidden, args.inter, args.topk, max(sizes), group=group, capacity_factor=3.0)
    pl = planner.n_local_routed_experts

    gp = torch.Generator(device=dev).manual_seed(5)
    popularity = 1.0 / torch.arange(1, n_logical + 1, device=dev, dtype=torch.float64) ** args.zipf
    popularity = (popularity / popularity.sum())[torch.randperm(n_logical, device=dev, generator=gp)]
    log_p = popularity.log().float()
    planner.update_redundancy_mapping((popularity * 1e9).long())  # placement from the long-run statistics
    layer.place_weights()
    x_all = torch.randn(max(sizes), args.hidden, device=dev, generator=gp).bfloat16()
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def rank_max(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return t.tolist()

    rows = []
    for tokens in sizes:
        total = args.warmup + args.steps
        idxs, ws = [], []
        for s in range(total):
            g = torch.Generator(device=dev).manual_seed(7919 * s + 104729 * rank + tokens)
            gumbel = -torch.log(-torch.log(torch.rand(tokens, n_logical, device=dev, generator=g).clamp_min(1e-20)))
            idx = (log_p + gumbel).topk(args.topk, dim=-1).indices
            idxs.append(idx)
            ws.append(torch.full((tokens, args.topk), 1.0 / args.topk, device=dev))
        x = x_all[:tokens]
        res = {"tokens_per_rank": tokens}
        sampler = ClockSampler(physical_gpu_index(local), period_s=0.002)
        sampler.__enter__()
        # planner alone: all steps enqueued behind a device-side sleep (the host is ahead of the
        # GPU, so host jitter stays outside the event pairs); the first launch behind the sleep is
        # untimed and absorbs the ranks' different wake-up times, after which every step starts
        # from the alignment the previous step's exchange left plus the skew of one L2 flush
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(total)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(total)]
        dist.barrier(group=group)
        torch.cuda.synchronize(dev)
        torch.cuda._sleep(20_000_000)
        planner.run(idxs[0], avail)
        for s in range(total):
            flush.fill_(s & 255)
            starts[s].record()
            planner.run(idxs[s], avail)
            ends[s].record()
        torch.cuda.synchronize(dev)
        t_pl = [a.elapsed_time(b) * 1e3 for a, b in list(zip(starts, ends))[args.warmup:]]
        res["planner_us"] = round(statistics.median(rank_max(t_pl)), 2)
        # and the way a caller without such alignment sees it: launched right after a host barrier
        t_pl = []
        for s in range(total):
            flush.fill_(s & 255)
            dist.barrier(group=group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            planner.run(idxs[s], avail)
            b.record()
            torch.cuda.synchronize(dev)
            if s >= args.warmup:
                t_pl.append(a.elapsed_time(b) * 1e3)
        res["planner_us_after_host_barrier"] = round(statistics.median(rank_max(t_pl)), 2)
        for policy in ("eplb", "lplb"):
            times, loads = [], []
            for s in range(total):
                flush.fill_(s & 255)
                dist.barrier(group=group)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                phys = layer.route(idxs[s], avail, "lplb" if policy == "lplb" else "static")
                layer.forward_physical(x, phys, ws[s])
                b.record()
                torch.cuda.synchronize(dev)
                if s >= args.warmup:
                    times.append(a.elapsed_time(b))
                    load = torch.bincount(phys.reshape(-1) // pl, minlength=world).double()
                    dist.all_reduce(load, group=group)
                    loads.append(float(load.max() / load.mean()))
            res[f"layer_ms_{policy}"] = round(statistics.median(rank_max(times)), 4)
            res[f"load_{policy}"] = round(statistics.fmean(loads), 4)
        sampler.__exit__(None, None, None)
        per_rank = [None] * world
        dist.all_gather_object(per_rank, sampler.summary(), group=group)
        res["clocks_per_rank"] = per_rank
        rows.append(res)
    status = (layer.check(), planner.check_status()["error"])
    if rank == 0:
        wins = [r["tokens_per_rank"] for r in rows if r["layer_ms_lplb"] < r["layer_ms_eplb"]]
        out = {
            "n_gpus": world,
            "topology": f"torus(2,{world // 2})" if world >= 4 else f"ring{world}",
            "experts": n_logical + red * world,
            "zipf_s": args.zipf,
            "sweep": rows,
            "lplb_beats_eplb_from_tokens_per_rank": min(wins) if wins else None,
            "status": status,
            "timing": "CUDA events, median over steps of the max over ranks, L2 flushed before each step; layer steps "
                      "start after a host barrier; planner_us: steps enqueued behind a device sleep, only the flush between them",
        }
        print(json.dumps(out))
        if args.json:
            os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
            with open(args.json, "w") as fh:
                json.dump(out, fh, indent=1)
    dist.barrier(group=group)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
