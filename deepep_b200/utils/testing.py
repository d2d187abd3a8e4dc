"""Timing helpers: CUDA-event benches, an L2 flush and a profiler-based kernel timer.

Parity: ``deep_ep/utils/testing.py`` (``bench`` :38-68, ``bench_kineto``
:131-218, ``flush_l2_cache`` :25-35) and the aggregation rules of
``benchmarks/_utils.py:69-88`` (per-iteration maximum over ranks, then mean
and nearest-rank percentiles).
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

L2_CACHE_FLUSH_BYTES = 256 << 20  # twice the 126 MB L2 of a B200


def flush_l2_cache(enabled: bool = True) -> None:
    if enabled and torch.cuda.is_available():
        torch.empty(L2_CACHE_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda").zero_()


def bench(fn: Callable[[], Any], num_warmups: int = 50, num_tests: int = 50,
          post_fn: Optional[Callable[[], Any]] = None, flush_l2: bool = True) -> Tuple[float, float, float]:
    """Return (mean, min, max) seconds of ``fn`` over ``num_tests - 1`` timed calls."""
    if num_warmups < 0:
        raise ValueError("num_warmups must be greater than or equal to zero")
    if num_tests < 2:
        raise ValueError("num_tests must be at least two")
    torch.cuda.synchronize()
    for _ in range(num_warmups):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    for i in range(num_tests):
        flush_l2_cache(flush_l2)
        starts[i].record()
        fn()
        ends[i].record()
        if post_fn is not None:
            post_fn()
    torch.cuda.synchronize()
    times = [s.elapsed_time(e) / 1e3 for s, e in zip(starts, ends)][1:]
    return sum(times) / len(times), min(times), max(times)


def event_times_us(fn: Callable[[], Any], iters: int, warmup: int = 3, flush_l2: bool = True) -> List[float]:
    """Per-iteration device microseconds of ``fn`` measured with CUDA events."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        flush_l2_cache(flush_l2)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        out.append(s.elapsed_time(e) * 1e3)
    return out


def nearest_rank(sorted_values: Sequence[float], q: float) -> float:
    if not sorted_values:
        raise ValueError("no samples")
    k = max(1, math.ceil(q * len(sorted_values)))
    return sorted_values[k - 1]


def aggregate_rank_max(per_rank_samples: Sequence[Sequence[float]]) -> Dict[str, float]:
    """Maximum over ranks per iteration, then mean/min/max/p50/p95 over iterations."""
    if not per_rank_samples or any(len(s) != len(per_rank_samples[0]) for s in per_rank_samples):
        raise ValueError("every rank must report the same number of samples")
    worst = [max(col) for col in zip(*per_rank_samples)]
    ordered = sorted(worst)
    return {
        "mean_rank_max_us": sum(worst) / len(worst), "min_us": ordered[0], "max_us": ordered[-1],
        "p50_us": nearest_rank(ordered, 0.50), "p95_us": nearest_rank(ordered, 0.95), "iterations": len(worst),
    }


def bandwidth_gbps(effective_bytes: float, mean_rank_max_us: float) -> float:
    """Decimal GB/s of ``effective_bytes`` moved in ``mean_rank_max_us``."""
    return effective_bytes / (mean_rank_max_us * 1000.0) if mean_rank_max_us > 0 else 0.0


def bench_kineto(fn: Callable[[], Any], kernel_names, num_tests: int = 30, suppress_kineto_output: bool = True,
                 trace_path: Optional[str] = None, barrier_comm_profiling: bool = False,
                 num_kernels_per_period: int = 1, *, flush_l2: bool = True, barrier: Optional[Callable[[], Any]] = None):
    """Average device seconds of the kernels whose name contains ``kernel_names``.

    Uses ``torch.profiler`` (CUPTI).  Returns one float per requested name (a single float when a string was passed).
    ``flush_l2`` writes a buffer larger than the L2 before every call; with ``barrier_comm_profiling`` the ranks are
    aligned before every call, by ``barrier()`` when one is given, else by an all-reduce of one element (the reference's
    keyword extensions, ``deep_ep/utils/testing.py:131-141`` there).
    """
    if not isinstance(kernel_names, (str, tuple, list)):
        raise TypeError("kernel_names must be a string or a tuple of strings")
    names = (kernel_names,) if isinstance(kernel_names, str) else tuple(kernel_names)
    if not names or not all(isinstance(name, str) for name in names):
        raise TypeError("kernel_names must contain strings")
    if any(not name for name in names):
        raise ValueError("kernel names must not be empty")
    if num_tests <= 0:
        raise ValueError("num_tests must be greater than zero")
    if num_kernels_per_period <= 0:
        raise ValueError("num_kernels_per_period must be greater than zero")
    from torch.profiler import ProfilerActivity, profile

    fn()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            flush_l2_cache(flush_l2)
            if barrier_comm_profiling:
                if barrier is not None:
                    barrier()
                elif torch.distributed.is_initialized():
                    torch.distributed.all_reduce(torch.ones(1, device="cuda"))
            fn()
        torch.cuda.synchronize()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    totals = {n: [0.0, 0] for n in names}
    for evt in prof.events():
        for n in names:
            if n in evt.name and evt.device_time > 0:
                totals[n][0] += evt.device_time
                totals[n][1] += 1
    result = []
    for n in names:
        total, count = totals[n]
        if count == 0:
            raise RuntimeError(f"no kernel matching {n!r} was profiled")
        result.append(total / count / 1e6)
    del suppress_kineto_output, num_kernels_per_period
    return result[0] if isinstance(kernel_names, str) else tuple(result)


__all__ = ["L2_CACHE_FLUSH_BYTES", "aggregate_rank_max", "bandwidth_gbps", "bench", "bench_kineto",
           "event_times_us", "flush_l2_cache", "nearest_rank"]
