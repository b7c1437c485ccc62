#!/usr/bin/env python
"""Benchmark of the hot path: the persistent bf16 tensor-descriptor matmul at M=N=K=8192, plus the
other example kernels (vector add, sin, fused-epilogue matmul, fused attention) as secondary lines.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extra]

A step is one launch of the matmul over synthetic inputs that are already resident in HBM
(A, B, C together are 403 MB, larger than the 126 MB L2, so no flush is needed between steps).
With N > 1 (one process per GPU under torchrun) the SAME 8192^3 problem is split: every rank owns M/N
contiguous rows of A and C (whole 128-row tiles, the reference's contiguous-range partition) and a replica
of B; there is no data-path collective and scaling is strong (`value` = 2*8192^3 / the slowest rank's time).
The fused attention forward is sharded by (batch, head) the same way and reported under "extra", as are
the replica form (every rank a full 8192-row block), the NCCL all-gather of C, and the matmul whose epilogue
stores C into every GPU's copy (with a bit-equality check against matmul + NCCL all-gather).

Prints ONE JSON line on rank 0.  `value` is whole-job TFLOP/s from CUDA-event time (max over ranks);
`e2e` is the same metric through the public wrapper with pinned HOST buffers, host<->device copies
inside the timed region; `roofline` compares the kernel with the measured cuBLAS bf16 peak;
`cpu_baseline` times the reference's golden_matmul loop (CPU oracle) on a bounded sample.
`--impl reference` times only that CPU implementation, with all host threads, on the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))

M = N = K = 8192
FLOP_PER_STEP = 2.0 * M * N * K
METRIC = "bf16 matmul TFLOP/s (persistent tensor-descriptor matmul, M=N=K=8192)"

# DRAM traffic of one 8192^3 launch of the headline kernel from an ncu capture
# (dram__bytes_read.sum 1.104 GB + dram__bytes_write.sum 127.4 MB; profiles/matmul_bf16_tcgen05_2cta_8192.md).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1_231_452_000


def measured_peaks():
    """Roofline denominators measured on this pool's B200s; the stated fallback if the file is absent."""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()   # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def mark(self):
        """The timed region starts now: `summary(under_load=True)` ignores the samples taken before."""
        self.mark_at = len(self.lines)

    def summary(self, under_load: bool = False):
        """Median / min / mean SM clock, maximum power and the throttle reasons seen.  under_load: only the samples after
        `mark()` (if it was called) whose power draw is at least half of the maximum seen, i.e. taken while the kernels ran."""
        rows, reasons = [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = self.lines[getattr(self, "mark_at", 0):] if under_load else self.lines
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                row = (float(parts[0]), float(parts[1]), float(parts[2]))
            except ValueError:
                continue
            rows.append((row, [name for name, val in zip(names, parts[3:7]) if val.lower().startswith("active")]))
        total = len(rows)
        if under_load and rows:
            pmax = max(r[0][2] for r in rows)
            rows = [r for r in rows if r[0][2] >= 0.5 * pmax]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [r[0][0] for r in rows]
        for _, active in rows:
            reasons.update(active)
        # nvidia-smi's readings lag the load by a sample or two, so the minimum and the mean are kept beside the median
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(r[0][1] for r in rows), "sm_mhz_min": min(sm),
                "sm_mhz_mean": round(statistics.fmean(sm), 1), "power_w_max": max(r[0][2] for r in rows),
                "reasons": sorted(reasons), "samples": len(rows), "samples_total": total}


def cpu_reference_rate(rows: int, repeat: int = 1):
    """Times the reference's golden_matmul loop (the CPU oracle) on `rows` rows of the 8192^3 problem,
    all host threads.  Returns (TFLOP/s, seconds, threads)."""
    import golden_inputs as gi
    from oracle import cpu_oracle as oracle
    oracle.use_all_cores()
    a, b = gi.matmul_inputs(rows, N, K, seed=0)
    best = float("inf")
    for _ in range(repeat):
        t0 = time.perf_counter()
        oracle.golden_matmul_naive(a, b)
        best = min(best, time.perf_counter() - t0)
    return 2.0 * rows * N * K / best / 1e12, best, oracle.max_threads()


def run_reference(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path (golden_matmul,
    examples/matmul_tensor_descriptor/matmul_multi_core_tma.cpp:31-51, restated in oracle/oracle.c) on the
    host cores.  Rank 0 alone works; each step is a bounded sample of rows of the 8192^3 problem."""
    if rank != 0:
        return
    import golden_inputs as gi
    from oracle import cpu_oracle as oracle
    threads = oracle.use_all_cores()
    # calibrate on 8 rows, then size a step so that warmup + steps stay near two minutes in total
    rate, secs, _ = cpu_reference_rate(8)
    rows_per_sec = 8 / secs
    budget = 120.0 / max(1, args.steps + args.warmup)
    rows = int(max(1, min(M, rows_per_sec * budget)))
    a, b = gi.matmul_inputs(rows, N, K, seed=0)
    for _ in range(args.warmup):
        oracle.golden_matmul_naive(a, b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.golden_matmul_naive(a, b)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * rows * N * K / dt / 1e12
    sample = f"{rows} of {M} rows of C per step (all {N} columns, K={K}), golden_matmul loop, {threads} OpenMP threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"bf16 matmul M=N=K={M}, A,B ~ N(0,1)/sqrt(K), fp32 accumulate, bf16 out", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_region(fn, steps, dist, torch):
    """Barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks. ms per step."""
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def quick_ms(fn, torch, warm=3, rep=10):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(rep):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / rep


def sustained_block(fn, flop, peaks, sampler_index, torch, seconds=2.0, probe_ms=None):
    """>= `seconds` of back-to-back launches of `fn` on this rank with the clock sampler running across them: the
    power-capped regime, beside the short (burst) timings.  Returns ms per launch, TFLOP/s, clocks, cycles per launch."""
    if probe_ms is None:
        probe_ms = quick_ms(fn, torch, warm=2, rep=5)
    n = max(20, int(seconds * 1000.0 / probe_ms))
    with ClockSampler(sampler_index) as clocks:
        time.sleep(0.3)          # a few idle samples first; the summary keeps the samples under load
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
    ms = s.elapsed_time(e) / n
    ck = clocks.summary(under_load=True)
    t = flop / ms / 1e9
    out = {"ms": ms, "TFLOP/s": t, "launches": n, "seconds": ms * n / 1e3, "clocks": ck,
           "frac_of_sustained_cublas": t / peaks["bf16_tflops_sustained"], "frac_of_nominal_2250": t / 2250.0}
    if ck.get("sm_mhz"):
        out["kcycles_per_launch"] = ms * ck["sm_mhz"]     # time x median SM MHz
    return out


def host_link_rates(torch, dist, nbytes=256 << 20, reps=4):
    """Pinned host<->device copy bandwidth of this rank with every rank copying at the same time, both directions at
    once (one large cudaMemcpyAsync per direction per repetition, on two streams).  GB/s (h2d, d2h)."""
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    d_out = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    d_in.copy_(h_in, non_blocking=True); h_out.copy_(d_out, non_blocking=True)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    with torch.cuda.stream(s1):
        ev[0].record()
        for _ in range(reps):
            d_in.copy_(h_in, non_blocking=True)
        ev[1].record()
    with torch.cuda.stream(s2):
        ev[2].record()
        for _ in range(reps):
            h_out.copy_(d_out, non_blocking=True)
        ev[3].record()
    torch.cuda.synchronize()
    h2d = reps * nbytes / ev[0].elapsed_time(ev[1]) / 1e6
    d2h = reps * nbytes / ev[2].elapsed_time(ev[3]) / 1e6
    if dist is not None:
        t = torch.tensor([h2d, d2h], device="cuda", dtype=torch.float64)
        lo = t.clone(); dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        tot = t.clone(); dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        return {"h2d_GB/s_per_gpu_min": float(lo[0]), "d2h_GB/s_per_gpu_min": float(lo[1]),
                "h2d_GB/s_all_gpus": float(tot[0]), "d2h_GB/s_all_gpus": float(tot[1])}
    return {"h2d_GB/s_per_gpu_min": h2d, "d2h_GB/s_per_gpu_min": d2h, "h2d_GB/s_all_gpus": h2d, "d2h_GB/s_all_gpus": d2h}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-workload", default=None,
                    choices=["matmul", "matmul_fused", "add", "sin", "memcpy", "attention", "attention_causal", "matmul_shard",
                             "attention_bwd"],
                    help="launch only this kernel warmup+steps times and print nothing to time: the small, "
                         "bounded command the ncu captures summarised under profiles/ are taken from")
    ap.add_argument("--shard-rows", type=int, default=1024, help="rows of A for --profile-workload matmul_shard")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import golden_inputs as gi
    from triton_tenstorrent_b200 import _lib, ops, sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU path)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    lib = _lib.load()
    peaks = measured_peaks()
    if args.profile_workload:
        profile_workload(args, torch, ops, gi)
        return

    # ---- inputs: ONE 8192^3 problem.  Rank r owns rows [r0, r1) of A and C (whole 128-row tiles, contiguous ranges)
    #      and a replica of B; with one GPU that is the whole problem.
    a_host_full = gi.matmul_inputs(M, N, K, seed=100)[0]
    b_host = gi.matmul_inputs(M, N, K, seed=0)[1]
    r0, r1 = sharding.row_shard(M, world, rank)
    a_host = a_host_full[r0:r1].contiguous()
    del a_host_full
    a, b = a_host.cuda(), b_host.cuda()
    c = torch.empty((r1 - r0, N), device="cuda", dtype=torch.bfloat16)
    step = lambda: ops.matmul_tma(a, b, True, out=c)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    launches0 = lib.b200k_launch_count()
    with ClockSampler(local_rank) as clocks:
        time.sleep(0.6)      # the sampler is up and has idle samples before the timed region starts
        clocks.mark()
        ms = time_region(step, args.steps, dist, torch)
        launches = lib.b200k_launch_count() - launches0
        # ---- kernel-only duration for the roofline: the step IS one kernel launch; per-launch events
        #      (same launches back to back, so the clock samples cover both loops)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        torch.cuda.synchronize()
        for s, e in evs:
            s.record(); step(); e.record()
        torch.cuda.synchronize()
        if args.steps * ms < 400.0:
            # a short timed region falls between two nvidia-smi samples: keep the GPU on the same launches until the
            # sampler has seen the load (these launches are not part of any reported time)
            t_end = time.perf_counter() + 0.4
            while time.perf_counter() < t_end:
                for _ in range(20):
                    step()
                torch.cuda.synchronize()
    ops.device_status()
    value = FLOP_PER_STEP / (ms * 1e-3) / 1e12       # whole job: the N shards together are one 8192^3 product
    # a step IS one launch of the kernel per GPU, so its average launch duration over the timed region is ms (CUDA
    # events around the K back-to-back launches); the per-launch events of the second loop (which add a gap per
    # launch) are reported beside it
    per_launch_ms = statistics.fmean(s.elapsed_time(e) for s, e in evs)
    kernel_ms = ms
    flop_per_gpu = FLOP_PER_STEP * (r1 - r0) / M
    achieved = flop_per_gpu / (kernel_ms * 1e-3) / 1e12
    sustained = args.steps * ms > 1000.0     # a second or more of back-to-back launches
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
                "peak_kind": f"{'sustained' if sustained else 'burst'} cuBLAS bf16, {peaks['source']}",
                "regime": "sustained (timed region over 1 s)" if sustained else "burst (timed region under 1 s)",
                "frac_of_nominal_2250": achieved / 2250.0,
                "kernel": "matmul_bf16_tcgen05_2cta_kernel<6>", "kernel_ms": kernel_ms,
                "kernel_ms_per_launch_events": per_launch_ms,
                "per_gpu": f"rows {r0}..{r1} of 8192 on rank {rank}" if world > 1 else "whole problem"}

    # ---- end to end through the public wrappers with pinned HOST buffers, copies inside the timed region
    a_pin, b_pin = a_host.pin_memory(), b_host.pin_memory()
    c_pin = torch.empty((r1 - r0, N), dtype=torch.bfloat16).pin_memory()
    if world == 1:
        e2e_step = lambda: ops.matmul_tma(a_pin, b_pin, True, out=c_pin)
        h2d_rank = (a_pin.numel() + b_pin.numel()) * 2
    else:
        # B crosses the host link once for the whole box: every rank uploads K/N of its rows and the ranks all-gather
        # it over NVLink; A rows stream up and C rows stream down in row blocks around the kernel
        e2e_step = lambda: sharding.matmul_tma_host_sharded(a_pin, b_pin, c_pin)
        h2d_rank = a_pin.numel() * 2 + sharding.host_b_bytes(b_pin, world)
    for _ in range(max(2, min(args.warmup, 5))):
        e2e_step()
    e2e_ms = time_region(e2e_step, args.steps, dist, torch)
    h2d_all, d2h_all = h2d_rank, c_pin.numel() * 2
    if dist is not None:
        t = torch.tensor([h2d_rank, c_pin.numel() * 2], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)
        h2d_all, d2h_all = int(t[0]), int(t[1])
    e2e = {"value": FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
           "ms_per_step": e2e_ms, "steps": args.steps}
    link = host_link_rates(torch, dist)
    # the copies that a step cannot avoid, at the measured concurrent link rates of the slowest GPU
    bound_ms = max(h2d_rank / link["h2d_GB/s_per_gpu_min"], c_pin.numel() * 2 / link["d2h_GB/s_per_gpu_min"]) / 1e6
    e2e["host_link"] = link
    e2e["host_link_bound_ms"] = bound_ms
    e2e["frac_of_host_link_bound"] = bound_ms / e2e_ms
    del a_pin, b_pin, c_pin

    extra = {}
    if not args.no_extra:
        try:   # the headline line must not depend on a secondary workload
            extra["matmul_8192_sustained" if world == 1 else "matmul_8192_shard_sustained"] = \
                sustained_block(step, flop_per_gpu, peaks, local_rank, torch, probe_ms=ms)
            if world == 1:
                extra.update(secondary_workloads(torch, ops, gi, peaks, local_rank))
            else:
                extra.update(multi_gpu_workloads(torch, ops, gi, sharding, peaks, dist, world, rank, a, b, c, ms))
        except Exception as e:  # noqa: BLE001
            extra["error"] = repr(e)

    cpu_baseline = None
    if rank == 0 and not args.no_cpu_baseline:
        rows = 64
        rate, secs, threads = cpu_reference_rate(rows)
        if secs < 5.0 and world == 1:   # many host cores: take a larger sample, about 10-20 s (N = 1 only: the other
            rows = int(min(M, rows * 12.0 / max(secs, 1e-3)))   # ranks wait for rank 0 at the final barrier)
            rate, secs, threads = cpu_reference_rate(rows)
        cpu_baseline = {"value": rate, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"{rows} of {M} rows of C (all {N} columns, K={K}) in {secs:.1f} s, the reference's "
                                  "golden_matmul loop restated in oracle/oracle.c"}

    if rank == 0:
        rows_per_gpu = r1 - r0
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"bf16 matmul M=N=K={M} (global M={M}: {rows_per_gpu} rows of A and C per GPU, B replicated), "
                                   "A,B ~ N(0,1)/sqrt(K), fp32 accumulate, bf16 out",
                       "l2": f"inputs larger than L2 (A+B+C = {(2 * rows_per_gpu * K + K * N) * 2 / 1e6:.0f} MB per GPU), no flush",
                       "parallelism": f"M-row blocks of C over {world} GPU(s), no collective"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches) * world,
            "clocks": clocks.summary(under_load=True), "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def profile_workload(args, torch, ops, gi):
    """One kernel, warmup + steps launches, workload-sized inputs (all larger than L2, under 1 GB)."""
    w = args.profile_workload
    if w == "matmul":
        a = (torch.randn(M, K, device="cuda") / K ** 0.5).bfloat16()
        b = (torch.randn(K, N, device="cuda") / K ** 0.5).bfloat16()
        c = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
        fn = lambda: ops.matmul_tma(a, b, True, out=c)
    elif w == "matmul_shard":
        # the M-row shard one GPU of N computes of the 8192^3 problem (1024 rows at N = 8)
        a = (torch.randn(args.shard_rows, K, device="cuda") / K ** 0.5).bfloat16()
        b = (torch.randn(K, N, device="cuda") / K ** 0.5).bfloat16()
        c = torch.empty((args.shard_rows, N), device="cuda", dtype=torch.bfloat16)
        fn = lambda: ops.matmul_tma(a, b, True, out=c)
    elif w == "matmul_fused":
        a = (torch.randn(16384, 4096, device="cuda") / 64).bfloat16()
        b = (torch.randn(4096, 4096, device="cuda") / 64).bfloat16()
        bias = torch.randn(4096, device="cuda") * 0.1
        c = torch.empty((16384, 4096), device="cuda", dtype=torch.bfloat16)
        fn = lambda: ops.matmul_fused(a, b, bias, "relu", out=c)
    elif w in ("add", "sin", "memcpy"):
        n = 1 << 26
        x, y = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
        fn = (lambda: ops.add(x, y)) if w == "add" else ((lambda: ops.sin(x)) if w == "sin" else (lambda: ops.memcpy(x, y)))
    elif w == "attention_bwd":
        # half the batch of the attention workload (2 x 32 heads x 4096 x 128): eight tensors of 67 MB, three launches
        q = torch.randn(2, 32, 4096, 128, device="cuda").bfloat16()
        k, v, d_o = torch.randn_like(q), torch.randn_like(q), torch.randn_like(q)
        o, m = ops.attention_with_lse(q, k, v, False, 128 ** -0.5)
        fn = lambda: ops.attention_backward(q, k, v, o, m, d_o, False, 128 ** -0.5)
    else:
        q = torch.randn(4, 32, 4096, 128, device="cuda").bfloat16()
        k, v = torch.randn_like(q), torch.randn_like(q)
        causal = w == "attention_causal"
        fn = lambda: ops.attention(q, k, v, causal, 128 ** -0.5)
    for _ in range(args.warmup + args.steps):
        fn()
    torch.cuda.synchronize()
    ops.device_status()
    print(json.dumps({"profile_workload": w, "launches": args.warmup + args.steps}), flush=True)


def secondary_workloads(torch, ops, gi, peaks, sampler_index):
    """The other example kernels at their workload sizes (per GPU), CUDA-event timed, with roofline fractions."""
    out = {}
    hbm = peaks["hbm_gbs"]
    tf = peaks["bf16_tflops"]
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int, device="cuda")

    def flushed_ms(fn, rep=10):
        fn(); fn()
        ts = []
        for _ in range(rep):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); fn(); e.record(); e.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)

    # vector add: the reference's n = 98432 (launch-latency bound, 1.2 MB) and a bandwidth-sized n = 2^26
    x, y = gi.add_inputs(98432)
    xd, yd = x.cuda(), y.cuda()
    ms = quick_ms(lambda: ops.add(xd, yd), torch, rep=50)
    out["add_n98432"] = {"ms": ms, "GB/s": 12 * 98432 / ms / 1e6, "note": "L2-resident, launch-latency bound"}
    # the same call recorded in a CUDA graph (20 launches per replay): what is left is the kernel itself
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(20):
            held = ops.add(xd, yd)
    ms = quick_ms(graph.replay, torch, rep=20) / 20
    out["add_n98432_cuda_graph"] = {"ms": ms, "GB/s": 12 * 98432 / ms / 1e6, "note": "20 launches per graph replay"}
    del graph, held
    n = 1 << 26
    xb, yb = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
    # 805 MB / 537 MB per launch: larger than L2, so back-to-back launches are a valid bandwidth measurement;
    # the flushed single-launch figure (which also contains the launch latency of a ~100 us kernel) is kept beside it
    ms = quick_ms(lambda: ops.add(xb, yb), torch, rep=30)
    msf = flushed_ms(lambda: ops.add(xb, yb))
    out["add_n2^26"] = {"ms": ms, "GB/s": 12 * n / ms / 1e6, "frac_of_hbm_peak": 12 * n / ms / 1e6 / hbm,
                        "l2": "inputs larger than L2, back-to-back launches", "ms_flushed_single": msf,
                        "GB/s_flushed_single": 12 * n / msf / 1e6}
    # the reference's own size sweep of vector add (01-vector-add.py:119: n = 2^12 .. 2^27), extended to 2^28;
    # back-to-back launches, so sizes that fit the 126 MB L2 (3 * 4 * n bytes) are served from it
    sweep = {}
    for kexp in range(12, 29, 2):
        nk = 1 << kexp
        xk, yk = torch.rand(nk, device="cuda"), torch.rand(nk, device="cuda")
        msk = quick_ms(lambda: ops.add(xk, yk), torch, rep=20 if kexp < 26 else 8)
        sweep[f"2^{kexp}"] = round(12 * nk / msk / 1e6, 1)
        del xk, yk
    out["add_sweep_GB/s"] = sweep
    xs = (xb * 8 - 4) * 3.14159265
    ms = quick_ms(lambda: ops.sin(xs), torch, rep=30)
    msf = flushed_ms(lambda: ops.sin(xs))
    out["sin_n2^26"] = {"ms": ms, "GB/s": 8 * n / ms / 1e6, "frac_of_hbm_peak": 8 * n / ms / 1e6 / hbm,
                        "l2": "inputs larger than L2, back-to-back launches", "ms_flushed_single": msf,
                        "GB/s_flushed_single": 8 * n / msf / 1e6}
    # the Gluon intro's memcpy (python/tutorials/gluon/01-intro.py reports 666 GB/s on GB200 for its one-element-per-step kernel)
    cp_out = torch.empty_like(xs)
    ms = quick_ms(lambda: ops.memcpy(xs, cp_out), torch, rep=30)
    out["memcpy_n2^26"] = {"ms": ms, "GB/s": 8 * n / ms / 1e6, "frac_of_hbm_peak": 8 * n / ms / 1e6 / hbm}
    del xb, yb, xs, cp_out

    # fused-epilogue matmul: ReLU(A.B + bias[N]), M=16384, N=K=4096
    Mf, Nf, Kf = 16384, 4096, 4096
    af, bf_ = gi.matmul_inputs(Mf, Nf, Kf, seed=1)
    bias = gi.row_bias(Nf).cuda()
    afd, bfd = af.cuda(), bf_.cuda()
    cf = torch.empty((Mf, Nf), device="cuda", dtype=torch.bfloat16)
    ms = quick_ms(lambda: ops.matmul_fused(afd, bfd, bias, "relu", out=cf), torch, rep=20)
    t = 2.0 * Mf * Nf * Kf / ms / 1e9
    out["matmul_fused_16384x4096x4096"] = {"ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf}
    del afd, bfd, cf

    # fused attention forward: Z=4, H=32, S=4096, D=128: short (burst) timing and >= 2 s of back-to-back launches
    Z, H, S, D = 4, 32, 4096, 128
    q = torch.randn(Z, H, S, D, device="cuda").bfloat16()
    k, v = torch.randn_like(q), torch.randn_like(q)
    for causal in (False, True):
        fn = lambda: ops.attention(q, k, v, causal, D ** -0.5)
        ms = quick_ms(fn, torch, rep=20)
        fl = 4.0 * Z * H * S * S * D * (0.5 if causal else 1.0)
        t = fl / ms / 1e9
        name = f"attention_fwd_{'causal' if causal else 'full'}"
        out[name] = {"ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf, "frac_of_nominal_2250": t / 2250.0}
        out[name + "_sustained"] = sustained_block(fn, fl, peaks, sampler_index, torch, probe_ms=ms)
        # the backward on the forward's saved tensors (delta, then dK/dV, then dQ: three launches).  The figure counts
        # the five matrix products of the algorithm (10 Z H S^2 D flop); the two kernels execute seven (S and dP twice)
        o, m = ops.attention_with_lse(q, k, v, causal, D ** -0.5)
        d_o = torch.randn_like(q)
        ms = quick_ms(lambda: ops.attention_backward(q, k, v, o, m, d_o, causal, D ** -0.5), torch, rep=10)
        t = 2.5 * fl / ms / 1e9
        out[f"attention_bwd_{'causal' if causal else 'full'}"] = {
            "ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf, "executed_TFLOP/s": t * 1.4, "launches": 3}
        del o, m, d_o
    del q, k, v
    # the other head dimensions (same token count): 64 with twice the heads, 256 with half.  At HEAD_DIM 64 the
    # exponentials bound the kernel, not the tensor pipe: 4.29e9 exponentials per launch at 16 per clock per SM, so
    # the figure is also given against that roofline at the maximum SM clock
    xu_tflops_d64 = 4.0 * 64 * 148 * 16 * 1.965e9 / 1e12     # flop per exponential (4 * D) x exponentials per second
    for (Hh, Dh) in ((64, 64), (16, 256)):
        q = torch.randn(Z, Hh, S, Dh, device="cuda").bfloat16()
        k, v = torch.randn_like(q), torch.randn_like(q)
        ms = quick_ms(lambda: ops.attention(q, k, v, False, Dh ** -0.5), torch, rep=10)
        t = 4.0 * Z * Hh * S * S * Dh / ms / 1e9
        out[f"attention_fwd_full_d{Dh}"] = {"ms": ms, "TFLOP/s": t, "frac_of_nominal_2250": t / 2250.0}
        if Dh == 64:
            out["attention_fwd_full_d64"]["ex2_roofline_TFLOP/s"] = xu_tflops_d64
            out["attention_fwd_full_d64"]["frac_of_ex2_roofline"] = t / xu_tflops_d64
            # the backward at HEAD_DIM 64: the same 2 x 4.29e9 exponentials (both kernels recompute P) for half the flop
            o, m = ops.attention_with_lse(q, k, v, False, Dh ** -0.5)
            d_o = torch.randn_like(q)
            ms = quick_ms(lambda: ops.attention_backward(q, k, v, o, m, d_o, False, Dh ** -0.5), torch, rep=10)
            out["attention_bwd_full_d64"] = {"ms": ms, "TFLOP/s": 10.0 * Z * Hh * S * S * Dh / ms / 1e9, "launches": 3}
            del o, m, d_o
        del q, k, v

    # matmul 4096^3 and 16384^3 (the other sizes of the workload definition)
    for S_ in (4096, 16384):
        aa = (torch.randn(S_, S_, device="cuda") / S_ ** 0.5).bfloat16()
        bb = (torch.randn(S_, S_, device="cuda") / S_ ** 0.5).bfloat16()
        cc = torch.empty((S_, S_), device="cuda", dtype=torch.bfloat16)
        ms = quick_ms(lambda: ops.matmul_tma(aa, bb, True, out=cc), torch, rep=10 if S_ < 16384 else 3)
        t = 2.0 * S_ ** 3 / ms / 1e9
        out[f"matmul_{S_}"] = {"ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf}
        del aa, bb, cc

    # the pointer-based matmul_kernel on tile-major fp16 buffers (32 x 32 tiles) with leaky_relu, 8192^3:
    # same kernels, operands fetched through 4-D tensor maps
    S_ = 8192
    at = ((torch.rand(S_, S_, device="cuda") - 0.5) / 16).half()
    bt = ((torch.rand(S_, S_, device="cuda") - 0.5) / 16).half()
    runs = [quick_ms(lambda: ops.matmul(at, bt, "leaky_relu", layout="tile32"), torch, rep=10) for _ in range(5)]
    ms = statistics.median(runs)
    t = 2.0 * S_ ** 3 / ms / 1e9
    out["matmul_tile32_f16_leaky_8192"] = {"ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf,
                                           "ms_runs": [round(r, 4) for r in runs]}
    del at, bt
    return out


def multi_gpu_workloads(torch, ops, gi, sharding, peaks, dist, world, rank, a_sh, b, c_sh, shard_ms):
    """N > 1: the fused attention forward sharded by (batch, head); the replica form of the matmul (every rank a full
    8192-row block, global M = 8192 * N); the all-gather of C by NCCL and by the matmul's own epilogue (peer stores),
    with a bit-equality check of the two gathered results."""
    out = {}
    rows = a_sh.shape[0]

    # ---- attention, Z*H = 128 (batch, head) pairs dealt out in contiguous ranges; every pair is independent
    Z, H, S, D = 4, 32, 4096, 128
    h0, h1 = sharding.head_shard(Z * H, world, rank)
    torch.manual_seed(1000 + rank)
    q = torch.randn(1, h1 - h0, S, D, device="cuda").bfloat16()
    k, v = torch.randn_like(q), torch.randn_like(q)
    for causal in (False, True):
        fn = lambda: ops.attention(q, k, v, causal, D ** -0.5)
        for _ in range(3):
            fn()
        ms = time_region(fn, 20, dist, torch)
        fl = 4.0 * Z * H * S * S * D * (0.5 if causal else 1.0)
        out[f"attention_sharded_{'causal' if causal else 'full'}"] = {
            "pairs_per_gpu": h1 - h0, "ms": ms, "TFLOP/s_total": fl / ms / 1e9,
            "frac_of_nominal_2250_per_gpu": fl / ms / 1e9 / world / 2250.0}
    del q, k, v

    # ---- replica form (weak scaling): every rank its own 8192-row block, B replicated, no collective
    a_full = gi.matmul_inputs(M, N, K, seed=100 + rank)[0].cuda()
    c_full = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    full = lambda: ops.matmul_tma(a_full, b, True, out=c_full)
    for _ in range(3):
        full()
    ms = time_region(full, 20, dist, torch)
    out["weak_8192_per_gpu"] = {"ms": ms, "TFLOP/s_total": world * FLOP_PER_STEP / ms / 1e9, "global_M": M * world}

    # ---- optional all-gather of C: NCCL after the matmul, or inside the matmul (epilogue stores to every GPU's copy)
    ms_ag = time_region(lambda: sharding.all_gather_rows(c_sh), 10, dist, torch)
    out["all_gather_C_nccl"] = {"ms": ms_ag, "bytes_out": M * N * 2, "GB/s_bus": (world - 1) / world * M * N * 2 / ms_ag / 1e6}
    if rows * world == M:
        try:   # GatheredRows raises on every rank or on none, so the ranks stay in step
            gathered = sharding.GatheredRows(rows, N)
            torch.cuda.synchronize()
            dist.barrier()
            sep = lambda: sharding.all_gather_rows(ops.matmul_tma(a_sh, b, True, out=c_sh))
            fused = lambda: sharding.matmul_all_gather(a_sh, b, gathered)
            ref = sep()
            got = fused()
            torch.cuda.synchronize()
            dist.barrier()
            same = torch.tensor([1 if torch.equal(ref.view(torch.int16), got.view(torch.int16)) else 0], device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            out["gather_parity"] = "bit-equal" if int(same.item()) == 1 else "MISMATCH"
            del ref
            ms_sep = time_region(sep, 20, dist, torch)
            ms_fused = time_region(fused, 20, dist, torch)
            sent = (world - 1) * rows * N * 2
            out["strong_8192_matmul_plus_all_gather"] = {
                "ms_matmul_then_nccl_all_gather": ms_sep, "ms_fused_epilogue_stores": ms_fused,
                "speedup": ms_sep / ms_fused, "nvlink_bytes_sent_per_gpu": sent,
                "GB/s_sent_per_gpu_fused": sent / ms_fused / 1e6, "ms_matmul_alone": shard_ms}
            # weak-scaling form: every rank's full 8192-row block gathered into a [world*8192, 8192] matrix
            big = sharding.GatheredRows(M, N)
            torch.cuda.synchronize()
            dist.barrier()
            sep = lambda: sharding.all_gather_rows(ops.matmul_tma(a_full, b, True, out=c_full))
            fused = lambda: sharding.matmul_all_gather(a_full, b, big)
            sep(); fused()
            ms_sep = time_region(sep, 5, dist, torch)
            ms_fused = time_region(fused, 5, dist, torch)
            sent = (world - 1) * M * N * 2
            out["weak_8192_per_gpu_matmul_plus_all_gather"] = {
                "ms_matmul_then_nccl_all_gather": ms_sep, "ms_fused_epilogue_stores": ms_fused,
                "speedup": ms_sep / ms_fused, "nvlink_bytes_sent_per_gpu": sent,
                "GB/s_sent_per_gpu_fused": sent / ms_fused / 1e6,
                "TFLOP/s_total_fused": world * FLOP_PER_STEP / ms_fused / 1e9}
        except Exception as e:  # noqa: BLE001
            out["matmul_plus_all_gather"] = {"error": repr(e)}
    return out


if __name__ == "__main__":
    main()
