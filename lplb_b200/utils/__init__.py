"""Timing and observability helpers (CUDA-event timing, L2 flush, profiler wrapper, NVML sampler)."""

from .timing import ClockSampler, L2Flusher, bench_kineto, physical_gpu_index, suppress_output, time_cuda

__all__ = ["ClockSampler", "L2Flusher", "bench_kineto", "physical_gpu_index", "suppress_output", "time_cuda"]
