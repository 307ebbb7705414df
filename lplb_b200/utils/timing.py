"""Device-side timing helpers.

``ClockSampler`` reads SM clock, power and throttle reasons through NVML (read-only) while a
timed region runs.  ``time_cuda`` brackets each call with CUDA events on the launching stream, after warm-up,
optionally evicting L2 between calls, and reports percentiles.  ``bench_kineto`` measures
named kernels with ``torch.profiler`` and can export a Chrome trace; it covers what the
reference's test helper of the same name does (reference ``tests/utils.py:46-94``) and
reads the kernel times from the profiler's event list instead of parsing its text table.
"""

from __future__ import annotations

import contextlib
import os
import statistics
import sys
import threading
import time
from typing import Callable, Sequence

import torch

__all__ = ["L2Flusher", "time_cuda", "bench_kineto", "suppress_output", "ClockSampler", "physical_gpu_index"]


@contextlib.contextmanager
def suppress_output():
    """Silence stdout and stderr at the file-descriptor level (profiler chatter included),
    like the helper in the reference's test utilities (reference ``tests/utils.py:16-43``)."""
    sys.stdout.flush()
    sys.stderr.flush()
    saved = os.dup(1), os.dup(2)
    with open(os.devnull, "w") as null:
        os.dup2(null.fileno(), 1)
        os.dup2(null.fileno(), 2)
        try:
            yield
        finally:
            os.dup2(saved[0], 1)
            os.dup2(saved[1], 2)
            os.close(saved[0])
            os.close(saved[1])


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""

    def __init__(self, device: torch.device | str = "cuda", mib: int = 256):
        self.buf = torch.empty(mib * 1024 * 1024, dtype=torch.uint8, device=device)
        self.n = 0

    def __call__(self) -> None:
        self.n += 1
        self.buf.fill_(self.n & 0xFF)


def time_cuda(fn: Callable[[], object], iters: int = 100, warmup: int = 10, flush_l2: bool = True) -> dict:
    """Per-call device time in microseconds: mean, p50, p90, min, max."""
    flusher = L2Flusher() if flush_l2 else None
    for _ in range(warmup):
        fn()
    pairs = []
    for _ in range(iters):
        if flusher:
            flusher()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        pairs.append((a, b))
    torch.cuda.synchronize()
    us = sorted(a.elapsed_time(b) * 1e3 for a, b in pairs)
    return {
        "mean": statistics.fmean(us),
        "p50": us[len(us) // 2],
        "p90": us[min(len(us) - 1, int(len(us) * 0.9))],
        "min": us[0],
        "max": us[-1],
        "iters": iters,
    }


def bench_kineto(
    fn: Callable[[], object],
    kernel_names: str | Sequence[str],
    num_tests: int = 30,
    trace_path: str | None = None,
) -> float | list[float]:
    """Average device time in seconds of the kernels whose name contains each given string."""
    single = isinstance(kernel_names, str)
    names = [kernel_names] if single else list(kernel_names)
    schedule = torch.profiler.schedule(wait=0, warmup=1, active=1, repeat=1)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA], schedule=schedule) as prof:
        for _ in range(2):
            for _ in range(num_tests):
                fn()
            torch.cuda.synchronize()
            prof.step()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    out = []
    events = prof.key_averages()
    for name in names:
        hits = [ev for ev in events if name in ev.key]
        if len(hits) != 1:
            raise RuntimeError(f"{len(hits)} profiler entries match kernel name {name!r}")
        ev = hits[0]
        total_us = getattr(ev, "device_time_total", None)
        if total_us is None:
            total_us = ev.cuda_time_total
        out.append(total_us / max(ev.count, 1) * 1e-6)
    return out[0] if single else out


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.power_w: list[float] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        names = {
            0x8: "hw_slowdown",
            0x40: "hw_thermal_slowdown",
            0x20: "sw_thermal_slowdown",
            0x4: "sw_power_cap",
            0x80: "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {
            "sm_mhz": int(statistics.median(self.samples)),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            "power_w": int(statistics.median(self.power_w)) if self.power_w else None,
        }


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            pass
    return local
