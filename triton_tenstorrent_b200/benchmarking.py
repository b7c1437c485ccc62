"""CUDA-event timing helper in the shape of triton.testing.do_bench, which the reference's driver
hands out as its benchmarker (backend/driver.py:524-526)."""
from __future__ import annotations

import statistics

import torch


def do_bench(fn, warmup: int = 5, rep: int = 20, grad_to_none=None, quantiles=None, flush_l2: bool = True,
             return_mode: str = "median"):
    """Runs fn() `warmup` + `rep` times and returns milliseconds per call (median / mean / min / max / all), or, with
    `quantiles` (what Triton's autotuner passes), the list of those quantiles of the measured times.
    Between timed calls a buffer larger than the L2 cache is overwritten so that every call starts cold.
    `grad_to_none` is accepted for call compatibility with triton.testing.do_bench and cleared the same way."""
    cache = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(rep):
        if grad_to_none is not None:
            for x in grad_to_none:
                x.grad = None
        if cache is not None:
            cache.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    if quantiles is not None:
        qs = torch.quantile(torch.tensor(times, dtype=torch.float64), torch.tensor(list(quantiles), dtype=torch.float64)).tolist()
        return qs[0] if len(qs) == 1 else qs
    if return_mode == "all":
        return times
    return {"median": statistics.median, "mean": statistics.fmean, "min": min, "max": max}[return_mode](times)
