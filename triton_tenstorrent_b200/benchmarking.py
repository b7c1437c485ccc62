"""CUDA-event timing helper in the shape of triton.testing.do_bench, which the reference's driver
hands out as its benchmarker (backend/driver.py:524-526)."""
from __future__ import annotations

import statistics

import torch


def do_bench(fn, warmup: int = 5, rep: int = 20, flush_l2: bool = True, return_mode: str = "median"):
    """Runs fn() `warmup` + `rep` times and returns milliseconds per call (median / mean / min / all).
    Between timed calls a buffer larger than the L2 cache is overwritten so that every call starts cold."""
    cache = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(rep):
        if cache is not None:
            cache.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    if return_mode == "all":
        return times
    return {"median": statistics.median, "mean": statistics.fmean, "min": min}[return_mode](times)
