#!/usr/bin/env python
"""Headline benchmark: ``planner.run`` latency on DeepSeek-V3-shaped gating, EP8 Cube.

256 logical + 16 redundant experts (2 per rank of the 8-rank Cube), top-8, 4096 tokens
per rank.  Indices are the top-k of bf16 logits ~ N(0,1) plus a per-expert bias ~ N(0,1)
that is redrawn every 50 steps; everything is seeded per step.  With N < 8 GPUs the LP
still covers the 8-rank Cube (``ep_size=8``); the N real ranks each contribute 4096
tokens and exchange their statistics, so per-GPU work is fixed ("weak" scaling).

The planner runs in the library's default configuration (warm-started LP).  The step
counter starts so that a bias redraw, with its expert re-placement (untimed slow path) and
the cold solves that follow it, falls in the middle of the timed steps.  The same steps are
timed once more with ``warm_start=False`` and reported as ``value_cold_us``.

``python bench.py --gpus N --steps K --warmup W`` prints one JSON line on rank 0.
For N > 1 launch through ``python -m torch.distributed.run --nproc-per-node N``.
``--impl reference`` runs the unmodified reference from ``baseline/_ref`` instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LOGICAL = 256
EP_SIZE = 8
RED_PER_RANK = 2
TOKENS_PER_RANK = 4096
TOP_K = 8
BIAS_PERIOD = 50
PUBLISHED_SOLVER_US = 100.0  # reference README.md:70, solver only, unstated hardware
METRIC = "planner.run us (device, max over ranks), EP8 Cube, 4096 tokens/rank x top-8"


def first_step(steps: int, warmup: int) -> int:
    """Number of the first (warm-up) step: chosen so that a bias redraw falls in the middle of
    the timed steps, or after at most 25 of them in a long run."""
    lead = min(steps // 2, BIAS_PERIOD // 2)
    start = BIAS_PERIOD - lead - warmup
    while start < 0:
        start += BIAS_PERIOD
    return start


def make_indices(step: int, rank: int, device: torch.device) -> torch.Tensor:
    """Logical expert ids ``[4096, 8]`` int64 for one step of one rank."""
    gb = torch.Generator(device=device).manual_seed(1_000_003 * (step // BIAS_PERIOD) + 17)
    bias = torch.randn(N_LOGICAL, device=device, generator=gb)
    gl = torch.Generator(device=device).manual_seed(7919 * step + 104_729 * rank + 1)
    logits = torch.randn(TOKENS_PER_RANK, N_LOGICAL, device=device, generator=gl) + bias
    return logits.bfloat16().topk(TOP_K, dim=-1).indices


from lplb_b200.utils.timing import ClockSampler, physical_gpu_index  # noqa: E402


def dist_setup(n_gpus: int):
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if n_gpus > 1 and world != n_gpus:
        raise SystemExit(
            f"--gpus {n_gpus} needs {n_gpus} ranks: launch with python -m torch.distributed.run "
            f"--nnodes=1 --nproc-per-node {n_gpus} --master-addr 127.0.0.1 bench.py --gpus {n_gpus}"
        )
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    return rank, world, local, group


def rank_max(values: torch.Tensor, group) -> torch.Tensor:
    if group is not None:
        import torch.distributed as dist

        dist.all_reduce(values, op=dist.ReduceOp.MAX, group=group)
    return values


def post_balance(planner_like, out: torch.Tensor, group, pl: int) -> float:
    """max/mean physical-rank load over the whole job after redirect."""
    load = torch.bincount(out.reshape(-1).clamp_min(0) // pl, weights=(out.reshape(-1) >= 0).double(), minlength=EP_SIZE)
    if group is not None:
        import torch.distributed as dist

        dist.all_reduce(load, group=group)
    return float(load.max() / load.mean())


def run_ours(args) -> dict:
    from lplb_b200 import Planner, cube

    rank, world, local, group = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    n_routed = N_LOGICAL + RED_PER_RANK * EP_SIZE
    extra = {"warm_start": False} if args.cold else {}  # otherwise the library default
    planner = Planner(cube(), n_routed, N_LOGICAL, EP_SIZE, group, device=dev, comm=args.comm, **extra)
    n_sms = args.n_sms or None  # None: the library picks (one CTA per SM, fewer for small batches)
    pl = planner.n_local_routed_experts

    total_steps = args.warmup + args.steps
    step0 = first_step(args.steps, args.warmup) if args.first_step < 0 else args.first_step
    idx_dev = [make_indices(step0 + s, rank, dev) for s in range(total_steps)]  # position s = step step0 + s
    idx_pinned = [t.cpu().pin_memory() for t in idx_dev]
    out_pinned = torch.empty_like(idx_pinned[0]).pin_memory()
    avail = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # 2x the 126 MB L2
    redraws_timed = sum(1 for s in range(args.warmup, total_steps) if (step0 + s) % BIAS_PERIOD == 0)

    def barrier():
        if group is not None:
            import torch.distributed as dist

            dist.barrier(group=group)
        torch.cuda.synchronize(dev)

    def replace_experts(who, pos: int) -> None:
        """Slow path, outside every timed region: re-place experts from the statistics of the
        first steps of the bias period that starts at position `pos` (summed over ranks)."""
        hist = torch.zeros(N_LOGICAL, dtype=torch.int64, device=dev)
        for s in range(pos, min(pos + 8, total_steps)):
            hist += torch.bincount(idx_dev[s].reshape(-1), minlength=N_LOGICAL)
        if group is not None:
            import torch.distributed as dist

            dist.all_reduce(hist, group=group)
        who.update_redundancy_mapping(hist)

    sleep_cycles = int(0.012 * torch.cuda.get_device_properties(dev).clock_rate * 1e3) if hasattr(
        torch.cuda.get_device_properties(dev), "clock_rate") else 20_000_000
    gate_logits = [torch.randn(TOKENS_PER_RANK, N_LOGICAL, device=dev).bfloat16() for _ in range(4)]

    def timed_chunks(who, fn, gate=False):
        """Run fn(position) for every timed step between CUDA events.  Steps are enqueued in
        chunks (one bias period at most) behind a ~10 ms device-side sleep, so the host is far
        ahead of the GPU and host scheduling jitter cannot open gaps inside an event pair.  The
        first launch behind each sleep is an untimed step: the ranks leave their sleeps at
        different times, its in-kernel exchange absorbs that, and every timed step then starts
        from the alignment the previous step's exchange left, plus the skew of one L2 flush.
        Nothing but the flush runs between two steps.  With `gate=True` every step is preceded,
        outside its event pair, by the top-k over that step's gate logits, the kernels that
        come right before the planner in a MoE layer; they displace the solver's code from the
        instruction caches, which is what the planner sees inside a real pipeline."""
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        k = 0
        while k < args.steps:
            pos = args.warmup + k
            if (step0 + pos) % BIAS_PERIOD == 0:
                replace_experts(who, pos)
            n = min(args.steps - k, BIAS_PERIOD - (step0 + pos) % BIAS_PERIOD)
            barrier()
            torch.cuda._sleep(sleep_cycles)
            fn(max(0, pos - 1))  # untimed: absorbs the ranks' different wake-up times
            for j in range(k, k + n):
                flush.fill_(j & 0xFF)  # evict L2 between timed iterations
                if gate:
                    gate_logits[(args.warmup + j) % len(gate_logits)].topk(TOP_K, dim=-1)
                starts[j].record()
                fn(args.warmup + j)
                ends[j].record()
            k += n
        barrier()
        ms = torch.tensor([a.elapsed_time(b) for a, b in zip(starts, ends)], dtype=torch.float64, device=dev)
        return rank_max(ms, group)

    # ---- device-timed kernel path -------------------------------------------------------
    replace_experts(planner, 0)
    for s in range(args.warmup):
        flush.fill_(s & 0xFF)
        planner.run(idx_dev[s], avail, n_sms)
    last_out = {}

    def fused_step(pos):
        last_out["out"] = planner.run(idx_dev[pos], avail, n_sms)

    with ClockSampler(physical_gpu_index(local)) as clocks:
        per_step_ms = timed_chunks(planner, fused_step)
    out = last_out["out"]
    ms_per_step = float(per_step_ms.mean())
    status = planner.check_status()
    if args.dump and rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(args.dump)), exist_ok=True)
        with open(args.dump, "w") as fh:
            fh.write("\n".join(f"{v * 1e3:.3f}" for v in per_step_ms.tolist()))

    # LP optimum of the last step's global statistics (float64 HiGHS) for the quality claim
    counts = torch.bincount(idx_dev[-1].reshape(-1), minlength=N_LOGICAL)
    if group is not None:
        import torch.distributed as dist

        dist.all_reduce(counts, group=group)
    from lplb_b200 import lp as _lp

    w_b, f_b = _lp.bundle_loads(counts.cpu().double(), planner.phy2log.cpu(), 1, EP_SIZE, RED_PER_RANK, N_LOGICAL // EP_SIZE, 1)
    _, t_opt = _lp.solve_highs(w_b[0], f_b[0], cube())
    optimum_ratio = t_opt / float(counts.sum() / EP_SIZE)
    balance_after = post_balance(planner, out, group, pl)
    naive = planner.mapping.log2phy[idx_dev[-1].reshape(-1), 0].long()
    balance_before = post_balance(planner, naive, group, pl)
    mapping_after_timed = planner.state_dict()

    # ---- the same steps with the other warm-start setting ----------------------------------------
    other = Planner(cube(), n_routed, N_LOGICAL, EP_SIZE, group, device=dev, comm=args.comm,
                    warm_start=not planner.warm_start)
    replace_experts(other, 0)
    for s in range(args.warmup):
        other.run(idx_dev[s], avail, n_sms)
    other_ms = float(timed_chunks(other, lambda pos: other.run(idx_dev[pos], avail, n_sms)).mean())
    # ---- the default configuration again, each step right behind the gate's top-k kernels ------------
    in_pipeline_ms = float(timed_chunks(planner, fused_step, gate=True).mean())
    warm_us, cold_us = (ms_per_step * 1e3, other_ms * 1e3) if planner.warm_start else (other_ms * 1e3, ms_per_step * 1e3)

    # ---- three-launch pipeline with torch.distributed.all_reduce, same inputs ----------------
    staged = Planner(
        cube(), n_routed, N_LOGICAL, EP_SIZE, group, device=dev,
        comm="nccl" if group is not None else "none", **extra,
    )
    replace_experts(staged, 0)
    for s in range(args.warmup):
        staged.run_staged(idx_dev[s], avail, n_sms)
    staged_ms = float(timed_chunks(staged, lambda pos: staged.run_staged(idx_dev[pos], avail, n_sms)).mean())
    planner.load_state_dict(mapping_after_timed)

    # ---- end to end through the public API: pinned H2D, run, D2H, every step -----------------
    idx_stage = torch.empty_like(idx_dev[0])
    for s in range(args.warmup):
        idx_stage.copy_(idx_pinned[s], non_blocking=True)
        out_pinned.copy_(planner.run(idx_stage, avail, n_sms), non_blocking=True)
        torch.cuda.synchronize(dev)
    barrier()
    t0 = time.perf_counter()
    for k in range(args.steps):
        idx_stage.copy_(idx_pinned[args.warmup + k], non_blocking=True)
        out_pinned.copy_(planner.run(idx_stage, avail, n_sms), non_blocking=True)
        torch.cuda.synchronize(dev)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    e2e_ms = float(rank_max(torch.tensor([e2e_ms], dtype=torch.float64, device=dev), group)[0])
    barrier()

    # ---- the same end-to-end step with the transfers done by the kernel itself ------------------
    # Planner.run takes the pinned host indices directly (its loads cross PCIe) and writes the
    # result into pinned host memory: same bytes per step, no copy-engine launches.
    zc_ms = None
    if planner.comm in ("p2p", "none"):
        for s in range(args.warmup):
            planner.run(idx_pinned[s], avail, n_sms, out=out_pinned)
            torch.cuda.synchronize(dev)
        barrier()
        t0 = time.perf_counter()
        for k in range(args.steps):
            planner.run(idx_pinned[args.warmup + k], avail, n_sms, out=out_pinned)
            torch.cuda.synchronize(dev)
        zc_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        zc_ms = float(rank_max(torch.tensor([zc_ms], dtype=torch.float64, device=dev), group)[0])
        barrier()

    # ---- the same launch replayed from a CUDA graph (device time, same events and L2 flush) -----
    # Extra information only; `value` stays the eagerly launched number.  Skipped unless the
    # capture succeeded on every rank, so that all ranks keep launching in step.
    graph_ms = None
    if planner.comm in ("p2p", "none"):
        idx_static, out_static = idx_dev[0].clone(), torch.empty_like(idx_dev[0])
        graph, ok = torch.cuda.CUDAGraph(), 1
        try:
            with torch.cuda.graph(graph):
                planner.run(idx_static, avail, n_sms, out=out_static)
        except Exception:
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=dev)
        if group is not None:
            import torch.distributed as dist

            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag) == 1:
            def graph_step(pos):
                graph.replay()

            # the work does not depend on the values, but keep the data realistic
            idx_static.copy_(idx_dev[args.warmup])
            graph_ms = float(timed_chunks(planner, graph_step).mean())

    # ---- per-phase device times from the kernel's own stamps (median over the timed steps) -------
    planner.enable_trace(True)
    rows = []
    for k in range(min(args.steps, 50)):
        flush.fill_(k & 0xFF)
        planner.run(idx_dev[args.warmup + k], avail, n_sms)
        rows.append(planner.phase_times_us())
    planner.enable_trace(False)
    keys = [key for key in rows[0] if all(key in r for r in rows)]
    phases = {key: round(statistics.median(r[key] for r in rows), 2) for key in keys}

    value_us = ms_per_step * 1e3
    result = {
        "metric": METRIC,
        "value": round(value_us, 3),
        "unit": "us",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 6),
        "higher_is_better": False,
        "scaling": "weak",
        "vs_baseline": round(value_us / PUBLISHED_SOLVER_US, 4),
        "dtype": "int64 indices, bf16 gate logits, fp64 LP",
        "data": "synthetic",
        "impl": "lplb_b200",
        "config": {
            "model": "DeepSeek-V3-shaped gate: 256 logical + 16 redundant experts, top-8",
            "global_batch": TOKENS_PER_RANK * world,
            "seq_len": 1,
            "tokens_per_rank": TOKENS_PER_RANK,
            "parallelism": f"ep8-cube LP over {world} rank(s)",
            "comm": planner.comm,
            "lp_warm_start": planner.warm_start,
            "planner_configuration": "library defaults" if not args.cold and args.comm == "auto" else "non-default flags",
            "n_sms": n_sms or planner._default_ctas(TOKENS_PER_RANK * TOP_K),
            "l2": "256 MiB buffer written between timed iterations",
            "first_step": step0,
            "bias_redraws_inside_timed_steps": redraws_timed,
            "slow_path": "update_redundancy_mapping runs at every bias redraw (every 50 steps, one of them inside "
                         "the timed steps), between timed chunks; the cold solves after it are timed",
            "launch": "timed steps are enqueued behind a 12 ms device sleep so host jitter stays outside the event "
                      "pairs; the first launch behind each sleep is an untimed step; only the L2 flush runs "
                      "between steps (value_behind_gate_topk_us: also the gate's top-k kernels, untimed)",
        },
        "clocks": clocks.summary(),
        "e2e": {
            "value": round((zc_ms if zc_ms is not None else e2e_ms) * 1e3, 3),
            "unit": "us",
            "h2d_bytes_per_step": idx_pinned[0].numel() * idx_pinned[0].element_size(),
            "d2h_bytes_per_step": out_pinned.numel() * out_pinned.element_size(),
            "how": "host wall clock per step: Planner.run(pinned host indices, out=pinned host buffer) + stream "
                   "synchronize; the kernel itself moves both buffers over PCIe" if zc_ms is not None else
                   "host wall clock per step: pinned H2D copy, Planner.run, D2H copy to pinned memory, synchronize",
            "with_copy_engine_transfers_us": round(e2e_ms * 1e3, 3),
        },
        "gpu_launches": args.steps * (1 if planner.comm in ("p2p", "none") else 3),
        "value_warm_us": round(warm_us, 3),
        "value_cold_us": round(cold_us, 3),
        "value_behind_gate_topk_us": round(in_pipeline_ms * 1e3, 3),
        "staged_nccl_pipeline_us": round(staged_ms * 1e3, 3),
        "cuda_graph_replay_us": None if graph_ms is None else round(graph_ms * 1e3, 3),
        "balance_max_over_mean": {
            "before": round(balance_before, 5),
            "after": round(balance_after, 5),
            "lp_optimum_float64": round(optimum_ratio, 5),
        },
        "lp_iters_last": status["lp_iters"],
        "lp_gap_last": status["lp_gap"],
        "status": status["error"],
        "p50_us": round(float(per_step_ms.median()) * 1e3, 3),
        "p90_us": round(float(per_step_ms.quantile(0.9)) * 1e3, 3),
        "max_us": round(float(per_step_ms.max()) * 1e3, 3),
        "min_us": round(float(per_step_ms.min()) * 1e3, 3),
        "phases_us_median": phases,
    }
    if group is not None:
        import torch.distributed as dist

        dist.destroy_process_group()
    return result if rank == 0 else {}


REFERENCE_DRIVER = r'''
import ctypes, json, os, sys, time
# The reference's extension is linked against the toolkit's nvJitLink; torch brings an older one
# with the same soname.  Load the newer one first so that both resolve to it.
if JITLINK:
    ctypes.CDLL(JITLINK, mode=ctypes.RTLD_GLOBAL)
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
sys.path.insert(0, ROOT)
import torch
import bench
from lplb import Planner            # the unmodified reference
args = bench.parse_args(ARGV)
rank, world, local, group = bench.dist_setup(args.gpus)
dev = torch.device("cuda", local)
r2o = torch.tensor([[3, 0, 1, 2, 7, 4, 5, 6], [6, 7, 4, 5, 0, 1, 2, 3]]).T.int().cuda()
planner = Planner(r2o, bench.N_LOGICAL + bench.RED_PER_RANK * bench.EP_SIZE, bench.N_LOGICAL, bench.EP_SIZE, group)
n_sms = args.n_sms or torch.cuda.get_device_properties(dev).multi_processor_count
total = args.warmup + args.steps
step0 = bench.first_step(args.steps, args.warmup)
idx = [bench.make_indices(step0 + s, rank, dev) for s in range(total)]
hist = torch.zeros(bench.N_LOGICAL, dtype=torch.int64, device=dev)
for s in range(min(8, total)):
    hist += torch.bincount(idx[s].reshape(-1), minlength=bench.N_LOGICAL)
if group is not None:
    torch.distributed.all_reduce(hist, group=group)
planner.update_redundancy_mapping(hist)
avail = torch.zeros((), dtype=torch.int32, device=dev)
flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
for s in range(args.warmup):
    planner.run(idx[s], avail, n_sms)
starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
torch.cuda.synchronize()
with bench.ClockSampler(bench.physical_gpu_index(local)) as clocks:
    for k in range(args.steps):
        pos = args.warmup + k
        if (step0 + pos) % bench.BIAS_PERIOD == 0:  # slow path at the bias redraw, outside the event pairs
            hist.zero_()
            for s in range(pos, min(pos + 8, total)):
                hist += torch.bincount(idx[s].reshape(-1), minlength=bench.N_LOGICAL)
            if group is not None:
                torch.distributed.all_reduce(hist, group=group)
            planner.update_redundancy_mapping(hist)
        flush.fill_(k & 0xFF)
        starts[k].record()
        out = planner.run(idx[args.warmup + k], avail, n_sms)
        ends[k].record()
    torch.cuda.synchronize()
ms = torch.tensor([a.elapsed_time(b) for a, b in zip(starts, ends)], dtype=torch.float64, device=dev)
ms = float(bench.rank_max(ms, group).mean())
if rank == 0:
    print("REFERENCE_JSON " + json.dumps({
        "impl": "reference", "metric": bench.METRIC, "value": round(ms * 1e3, 3), "unit": "us",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": round(ms * 1e3 / bench.PUBLISHED_SOLVER_US, 4),
        "dtype": "int64 indices, fp32 LP", "data": "synthetic", "clocks": clocks.summary(),
        "config": {"model": "DeepSeek-V3-shaped gate: 256 logical + 16 redundant experts, top-8",
                   "global_batch": bench.TOKENS_PER_RANK * world, "seq_len": 1, "parallelism": "ep8-cube"}}))
'''


def find_jitlink() -> str:
    """The toolkit's libnvJitLink.so.12: the copy shipped beside the reference install, else the
    one next to the nvcc on PATH or under CUDA_HOME; "" if none is found."""
    import shutil

    candidates = [os.path.join(ROOT, "baseline", "_ref", "_libs", "libnvJitLink.so.12")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH")):
        if home:
            candidates.append(os.path.join(home, "lib64", "libnvJitLink.so.12"))
    nvcc = shutil.which("nvcc")
    if nvcc:
        candidates.append(os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "lib64", "libnvJitLink.so.12"))
    return next((c for c in candidates if os.path.exists(c)), "")


def run_reference(argv: list[str]) -> dict:
    """Run the unmodified reference in a child process; report why if it cannot run."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref", "lplb")
    if not os.path.isdir(ref_dir):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (offline pip install of the reference checkout was not done)"}
    if not os.path.isdir(os.path.join(ref_dir, "resources", "mathdx")):
        # The one blocker that cannot be fixed offline; nothing of the reference is run without it
        # (its run-time compile of minilp.cu can only fail, and did so with a crash of the child
        # process instead of an error message on a GPU box).
        return {"impl": "reference", "unavailable": "lplb/resources/mathdx is absent: all four kernels sit in minilp.cu, "
                "which includes cublasdx.hpp and cusolverdx.hpp (MathDx 25.06.0, fetched by download-mathdx.sh from the "
                "network); no copy of MathDx exists on this machine, so the reference's kernels cannot be compiled"}
    env = dict(os.environ)
    env.setdefault("LPLB_CACHE_PATH", os.path.join(ROOT, "baseline", "_ref", "_jit_cache"))
    code = f"ROOT = {ROOT!r}\nARGV = {argv!r}\nJITLINK = {find_jitlink()!r}\n" + REFERENCE_DRIVER
    try:
        proc = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"impl": "reference", "unavailable": "reference run exceeded 900 s"}
    for line in proc.stdout.splitlines():
        if line.startswith("REFERENCE_JSON "):
            return json.loads(line[len("REFERENCE_JSON "):])
    tail = [ln.strip() for ln in (proc.stderr or proc.stdout).splitlines() if ln.strip()]
    reason = tail[-1] if tail else f"exit code {proc.returncode}"
    mathdx = os.path.isdir(os.path.join(ref_dir, "resources", "mathdx"))
    note = "" if mathdx else " [lplb/resources/mathdx is absent: the kernels include cublasdx.hpp/cusolverdx.hpp, fetched by download-mathdx.sh from the network]"
    return {"impl": "reference", "unavailable": (reason[:300] + note)}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--comm", choices=["auto", "p2p", "nccl", "none"], default="auto")
    ap.add_argument("--n-sms", type=int, default=0, help="CTAs used by the planner kernels (default: the library picks)")
    ap.add_argument("--cold", action="store_true", help="headline with Planner(warm_start=False) instead of the default")
    ap.add_argument("--first-step", type=int, default=-1, help="number of the first warm-up step (default: chosen "
                    "so that a bias redraw falls inside the timed steps)")
    ap.add_argument("--dump", default="", help="write the per-step device times (us) to this file")
    return ap.parse_args(argv)


def main():
    args = parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        result = run_reference(sys.argv[1:])
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(result), flush=True)
        return
    result = run_ours(args)
    if result:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
