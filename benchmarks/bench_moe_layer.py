#!/usr/bin/env python
"""End-to-end MoE layer over N GPUs: what does balancing buy?

DeepSeek-V3-like layer: hidden 7168, SwiGLU 7168 -> 2048 -> 7168, 32 logical experts per
rank plus the topology's redundant slots (256 + 16 experts on the 8-rank Cube), top-8,
8192 tokens per rank with hidden states ~ N(0,1), random-init bf16 weights.  Gate logits
~ N(0,1) plus a per-expert bias ~ N(0, skew), seeded per step.

Three policies are timed on the same inputs (device time, max over ranks, per step):
  none    natural expert placement, every token goes to the original expert
  eplb    placement re-balanced from history, every token goes to the original expert
  lplb    same placement plus the per-batch LP (Planner.run inside the timed region)
and the stages of the lplb run are separated by running the pipeline up to each stage.

Launch: python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/bench_moe_layer.py [--tokens 8192] [--steps 8]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import Planner, cube, ring  # noqa: E402
from lplb_b200.models.moe import MoELayer  # noqa: E402
from lplb_b200.utils.timing import ClockSampler, physical_gpu_index  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--skew", type=float, default=1.0)
    ap.add_argument("--capacity-factor", type=float, default=3.0)
    ap.add_argument("--fuse-dispatch", action="store_true", help="send rows from inside the first GEMM kernel")
    ap.add_argument("--send-ctas", type=int, default=0, help="with --fuse-dispatch: CTAs that only send rows")
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world < 2:
        raise SystemExit("needs at least 2 ranks; see benchmarks/bench_moe_rank.py for one GPU")
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    r2o = cube() if world == 8 else ring(world)
    red = r2o.shape[1]
    n_logical = args.experts_per_rank * world
    planner = Planner(r2o, n_logical + red * world, n_logical, world, group, device=dev, comm="p2p")
    layer = MoELayer(planner, args.hidden, args.inter, args.topk, args.tokens, group=group,
                     capacity_factor=args.capacity_factor)
    layer.fuse_dispatch = args.fuse_dispatch
    layer.send_ctas = args.send_ctas
    pl = planner.n_local_routed_experts

    total = args.warmup + args.steps
    gb = torch.Generator(device=dev).manual_seed(17)
    bias = torch.randn(n_logical, device=dev, generator=gb) * args.skew
    xs, idxs, ws = [], [], []
    for s in range(total):
        g = torch.Generator(device=dev).manual_seed(7919 * s + 104729 * rank + 1)
        logits = (torch.randn(args.tokens, n_logical, device=dev, generator=g) + bias).bfloat16()
        w, idx = torch.softmax(logits.float(), -1).topk(args.topk, dim=-1)
        idxs.append(idx)
        ws.append(w.contiguous())
    x = torch.randn(args.tokens, args.hidden, device=dev, generator=gb).bfloat16()
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def rank_max(v):
        t = torch.tensor(v, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return t

    clocks = {}
    max_rows = {}

    def run_policy(policy, upto=5):
        """Per-step device ms (max over ranks, mean over steps) and the max/mean rank load.
        SM clock, board power and throttle reasons are sampled on every rank while it runs."""
        with ClockSampler(physical_gpu_index(local), period_s=0.002) as sampler:
            out = _run_policy(policy, upto)
        per_rank = [None] * world
        dist.all_gather_object(per_rank, sampler.summary(), group=group)
        clocks[f"{policy}_upto{upto}"] = per_rank
        return out

    def _run_policy(policy, upto):
        times, loads, rows = [], [], []
        for s in range(total):
            flush.fill_(s & 255)
            dist.barrier(group=group)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            phys = layer.route(idxs[s], avail, "lplb" if policy == "lplb" else "static")
            layer.forward_physical(x, phys, ws[s], upto)
            b.record()
            torch.cuda.synchronize(dev)
            if s >= args.warmup:
                times.append(a.elapsed_time(b))
                load = torch.bincount(phys.reshape(-1) // pl, minlength=world).double()
                dist.all_reduce(load, group=group)
                loads.append(float(load.max() / load.mean()))
                rows.append(float(load.max()))
        per_step = rank_max(times)
        max_rows[f"{policy}_upto{upto}"] = sum(rows) / len(rows)
        return float(per_step.mean()), sum(loads) / len(loads)

    results = {}
    # none: natural placement
    planner.update_redundancy_mapping(None)
    layer.place_weights()
    results["none"] = run_policy("none")
    # placement from history (the first two steps' statistics, summed over ranks)
    hist = torch.zeros(n_logical, dtype=torch.int64, device=dev)
    for s in range(2):
        hist += torch.bincount(idxs[s].reshape(-1), minlength=n_logical)
    dist.all_reduce(hist, group=group)
    planner.update_redundancy_mapping(hist)
    layer.place_weights()
    results["eplb"] = run_policy("eplb")
    results["lplb"] = run_policy("lplb")
    stages = [run_policy("lplb", upto=u)[0] for u in (1, 2, 3, 4)]
    status = layer.check()

    if rank == 0:
        n_rows = args.tokens * args.topk
        remote = n_rows * (world - 1) / world * args.hidden * 2
        lp_ms, lp_load = results["lplb"]
        dispatch_ms = stages[1] - stages[0]
        # roofline denominators: the driver-measured peaks of this pool when the file is there
        peaks = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback figures"}
        peaks_file = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
        if os.path.exists(peaks_file):
            with open(peaks_file) as fh:
                measured = json.load(fh)
            peaks = {"bf16_tflops": measured["bf16_tflops"], "bf16_tflops_sustained": measured["bf16_tflops_sustained"],
                     "source": "MEASURED_PEAKS.json"}
        rows_hot = max_rows["lplb_upto5"]  # rows on the most loaded rank, which sets the step time
        flop1 = rows_hot * 2.0 * args.hidden * 2 * args.inter
        flop2 = rows_hot * 2.0 * args.inter * args.hidden
        gemm1_ms = stages[2] - (stages[0] if args.fuse_dispatch else stages[1])
        gemm2_ms = stages[3] - stages[2]

        def roof(flops, nvlink_bytes, ms):
            """Achieved / roofline for a kernel inside the step loop: compute against the sustained
            (power-capped) and the burst cuBLAS rate, NVLink at the nominal 900 GB/s per direction and
            at the 770 GB/s that a peer copy reaches on this pool."""
            out = {"ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1)}
            for cname, cpeak in (("sustained", peaks["bf16_tflops_sustained"]), ("burst", peaks["bf16_tflops"])):
                for lname, link in (("900", 900.0), ("770", 770.0)):
                    bound_ms = max(flops / (cpeak * 1e12), nvlink_bytes / (link * 1e9)) * 1e3
                    out[f"achieved_over_roofline_{cname}_nvlink{lname}"] = round(bound_ms / ms, 3)
            return out

        roofline = {
            "peaks": dict(peaks, nvlink_gbs_nominal=900.0, nvlink_gbs_measured_peer_copy=770.0),
            "rows_on_most_loaded_rank": round(rows_hot, 1),
            "gemm2_with_combine": roof(flop2, remote, gemm2_ms),
        }
        if args.fuse_dispatch:
            roofline["dispatch_with_gemm1"] = roof(flop1, remote, gemm1_ms)
        else:
            roofline["gemm1_swiglu"] = roof(flop1, 0.0, gemm1_ms)
        out = {
            "n_gpus": world,
            "fuse_dispatch": args.fuse_dispatch,
            "send_ctas": args.send_ctas,
            "topology": "cube" if world == 8 else f"ring{world}",
            "shape": {"hidden": args.hidden, "inter": args.inter, "experts": n_logical + red * world,
                      "topk": args.topk, "tokens_per_rank": args.tokens, "skew": args.skew},
            "layer_ms_max_over_ranks": {k: round(v[0], 4) for k, v in results.items()},
            "rank_load_max_over_mean": {k: round(v[1], 4) for k, v in results.items()},
            "lplb_stage_ms": {
                "route_count_plan": round(stages[0], 4),
                "dispatch_alone": round(dispatch_ms, 4),
                ("dispatch_and_gemm1_fused" if args.fuse_dispatch else "gemm1_swiglu"): round(
                    stages[2] - (stages[0] if args.fuse_dispatch else stages[1]), 4),
                "gemm2_combine": round(stages[3] - stages[2], 4),
                "reduce": round(lp_ms - stages[3], 4),
            },
            "dispatch_nvlink_gbs_per_direction": round(remote / (dispatch_ms * 1e-3) / 1e9, 1),
            "dispatch_frac_of_770_gbs": round(remote / (dispatch_ms * 1e-3) / 1e9 / 770.0, 3),
            "speedup_lplb_vs_none": round(results["none"][0] / lp_ms, 3),
            "speedup_lplb_vs_eplb": round(results["eplb"][0] / lp_ms, 3),
            "status": status,
            "roofline": roofline,
            "clocks_per_run_and_rank": clocks,
            "timing": "CUDA events per step around route + layer, 256 MiB L2 flush and a barrier before each step",
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
