"""bench.py's reference arm must answer with one JSON line even where the reference cannot run."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "3", "--warmup", "3"],
        capture_output=True, text=True, timeout=600, cwd=ROOT,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference"
    assert "unavailable" in out or {"metric", "value", "unit", "n_gpus"} <= set(out)


def test_bench_defaults_follow_the_contract():
    sys.path.insert(0, ROOT)
    import bench

    args = bench.parse_args([])
    assert args.gpus == 1 and args.warmup >= 3 and args.steps > 0 and args.impl == "ours"
    assert bench.N_LOGICAL == 256 and bench.EP_SIZE == 8 and bench.TOKENS_PER_RANK == 4096 and bench.TOP_K == 8


def test_a_bias_redraw_falls_inside_the_timed_steps():
    sys.path.insert(0, ROOT)
    import bench

    for steps, warmup in ((20, 5), (200, 20), (3, 3), (40, 5), (20, 60)):
        first = bench.first_step(steps, warmup)
        assert first >= 0
        timed = range(first + warmup, first + warmup + steps)
        redraws = [s for s in timed if s % bench.BIAS_PERIOD == 0]
        assert redraws, (steps, warmup, first)
        # not at the very first timed step: the steps before it run on the old distribution
        assert redraws[0] > timed[0] or steps < 2


def test_clock_sampler_reads_a_fake_nvml(monkeypatch):
    """The sampler only reads: clock, power and event reasons, through whatever NVML binding is importable."""
    import sys
    import time
    import types

    from lplb_b200.utils.timing import ClockSampler

    calls = []
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("gpu", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965
    fake.nvmlDeviceGetClockInfo = lambda h, kind: 1500
    fake.nvmlDeviceGetPowerUsage = lambda h: 987_000
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    with ClockSampler(3, period_s=0.001) as sampler:
        time.sleep(0.02)
    out = sampler.summary()
    assert out["sm_mhz"] == 1500 and out["sm_max_mhz"] == 1965 and out["power_w"] == 987
    assert out["reasons"] == ["sw_power_cap"] and out["samples"] >= 1
    assert set(dir(fake)) >= {"nvmlInit"} and calls == ["init"]  # nothing but reads were asked of it


def test_cpu_plumbing_walkthrough_reaches_the_lp_optimum():
    """The GPU-free walk-through (placement, LP, redirect on 8 simulated ranks) ends at the HiGHS optimum."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run(
        [sys.executable, os.path.join(root, "benchmarks", "cpu_plumbing.py")],
        capture_output=True, text=True, timeout=300, env=env, cwd=root,
    )
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    ratios = line["max_over_mean"]
    assert ratios["after_placement"] < ratios["natural_placement"]
    assert ratios["after_lp_redirect"] <= ratios["lp_optimum_highs"] + 2e-3
    assert line["ipm_vs_highs_relative_gap"] < 1e-4 and line["groups_converged"] == 1
