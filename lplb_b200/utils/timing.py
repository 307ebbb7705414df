"""Device-side timing helpers.

``time_cuda`` brackets each call with CUDA events on the launching stream, after warm-up,
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
from typing import Callable, Sequence

import torch

__all__ = ["L2Flusher", "time_cuda", "bench_kineto", "suppress_output"]


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
