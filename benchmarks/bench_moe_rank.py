#!/usr/bin/env python
"""One rank's share of the end-to-end MoE layer on a single B200.

Shape of one EP8 rank of the DeepSeek-V3-like layer: hidden 7168, SwiGLU 7168 -> 2048 -> 7168,
34 physical experts, 8192 tokens x top-8 = 65,536 expert rows.  Every stage is timed with
CUDA events (L2 flushed before each), and the two grouped GEMMs are reported against the
measured cuBLAS bf16 throughput of this GPU.

Usage: python benchmarks/bench_moe_rank.py [--tokens 8192] [--iters 10] [--skew 0.0]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lplb_b200 import _native  # noqa: E402
from lplb_b200.models.moe import interleave_gate_up  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=34)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skew", type=float, default=0.0, help="std of the per-expert logit bias")
    ap.add_argument("--fuse-dispatch", action="store_true")
    ap.add_argument("--send-ctas", type=int, default=0, help="with --fuse-dispatch: CTAs that only send rows")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    native = _native.load()
    h, i, e, k, t = args.hidden, args.inter, args.experts, args.topk, args.tokens
    eng = native.MoeEngine(h, i, e, 1, 0, k, t, -(-t * k // 128) * 128, 0)
    eng.open([bytes(eng.alloc())])
    g = torch.Generator(device=dev).manual_seed(0)
    w13 = torch.empty(e, 2 * i, h, dtype=torch.bfloat16, device=dev)
    w2 = torch.empty(e, h, i, dtype=torch.bfloat16, device=dev)
    for s in range(e):
        gate = (torch.randn(i, h, device=dev, generator=g) * h**-0.5).bfloat16()
        up = (torch.randn(i, h, device=dev, generator=g) * h**-0.5).bfloat16()
        w13[s] = interleave_gate_up(gate, up)
        w2[s] = (torch.randn(h, i, device=dev, generator=g) * i**-0.5).bfloat16()
    eng.set_weights(w13, w2)
    eng.set_send_ctas(args.send_ctas)
    x = torch.randn(t, h, device=dev, generator=g).bfloat16()
    logits = torch.randn(t, e, device=dev, generator=g) + args.skew * torch.randn(e, device=dev, generator=g)
    wts, idx = torch.softmax(logits, -1).topk(k, dim=-1)
    n_cta = torch.cuda.get_device_properties(dev).multi_processor_count
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def timed(upto):
        vals = []
        for it in range(args.iters + 2):
            flush.fill_(it & 255)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.forward(x, idx, wts, n_cta, upto, args.fuse_dispatch)
            b.record()
            torch.cuda.synchronize()
            if it >= 2:
                vals.append(a.elapsed_time(b))
        return statistics.median(vals)

    cum = [timed(u) for u in (1, 2, 3, 4, 5)]
    status = eng.status().tolist()
    stage = {
        "count_plan_ms": cum[0],
        "dispatch_ms": cum[1] - cum[0],
        "gemm1_swiglu_ms": cum[2] - cum[1],
        "gemm2_combine_ms": cum[3] - cum[2],
        "reduce_ms": cum[4] - cum[3],
        "total_ms": cum[4],
    }
    if args.fuse_dispatch:  # stage 2 ran the stand-alone dispatch; stage 3 ran dispatch and GEMM 1 in one kernel
        stage["dispatch_and_gemm1_fused_ms"] = cum[2] - cum[0]
    rows = t * k
    f1, f2 = 2.0 * rows * h * 2 * i, 2.0 * rows * i * h
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
    except OSError:
        pass
    peak = peaks.get("bf16_tflops", 1590.0)
    result = {
        "shape": {"hidden": h, "inter": i, "experts": e, "topk": k, "tokens": t, "rows": rows, "skew": args.skew},
        "stage_ms": {k_: round(v, 4) for k_, v in stage.items()},
        "gemm1_tflops": round(f1 / (stage["gemm1_swiglu_ms"] * 1e-3) / 1e12, 1),
        "gemm2_tflops": round(f2 / (stage["gemm2_combine_ms"] * 1e-3) / 1e12, 1),
        "gemm1_frac_of_measured_bf16_peak": round(f1 / (stage["gemm1_swiglu_ms"] * 1e-3) / 1e12 / peak, 3),
        "gemm2_frac_of_measured_bf16_peak": round(f2 / (stage["gemm2_combine_ms"] * 1e-3) / 1e12 / peak, 3),
        "dispatch_gbs": round(rows * h * 2 * 2 / (stage["dispatch_ms"] * 1e-3) / 1e9, 1),
        "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback 1590 TFLOP/s",
        "status": status[:2],
    }
    print(json.dumps(result))
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        with open(args.json, "w") as fh:
            json.dump(result, fh, indent=1)


if __name__ == "__main__":
    main()
