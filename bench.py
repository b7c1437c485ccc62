#!/usr/bin/env python
"""Benchmark of the hot path: the persistent bf16 tensor-descriptor matmul at M=N=K=8192, plus the
other example kernels (vector add, sin, fused-epilogue matmul, fused attention) as secondary lines.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extra]

A step is one launch of the matmul over synthetic inputs that are already resident in HBM
(A, B, C together are 403 MB, larger than the 126 MB L2, so no flush is needed between steps).
With N > 1 (one process per GPU under torchrun) every rank owns one 8192-row block of A and C and a
replica of B: the global problem is [8192*N, 8192] x [8192, 8192], there is no data-path collective,
scaling is weak.  The optional NCCL all-gather of C and the strong-scaling split of a single 8192^3
problem are timed separately and reported under "extra".

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
METRIC = "bf16 matmul TFLOP/s (persistent tensor-descriptor matmul, M=N=K=8192 per GPU)"

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

    def summary(self):
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # nvidia-smi's readings lag the load by a sample or two, so the minimum and the mean are kept beside the median
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "sm_mhz_min": min(sm),
                "sm_mhz_mean": round(statistics.fmean(sm), 1), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}


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
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-workload", default=None,
                    choices=["matmul", "matmul_fused", "add", "sin", "attention", "attention_causal"],
                    help="launch only this kernel warmup+steps times and print nothing to time: the small, "
                         "bounded command the ncu captures summarised under profiles/ are taken from")
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

    # ---- inputs: every rank owns one 8192-row block of A and C, and a replica of B
    a_host = gi.matmul_inputs(M, N, K, seed=100 + rank)[0]
    b_host = gi.matmul_inputs(M, N, K, seed=0)[1]
    a, b = a_host.cuda(), b_host.cuda()
    c = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    step = lambda: ops.matmul_tma(a, b, True, out=c)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    launches0 = lib.b200k_launch_count()
    with ClockSampler(local_rank) as clocks:
        ms = time_region(step, args.steps, dist, torch)
        launches = lib.b200k_launch_count() - launches0
        # ---- kernel-only duration for the roofline: the step IS one kernel launch; per-launch events
        #      (same launches back to back, so the clock samples cover both loops)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        torch.cuda.synchronize()
        for s, e in evs:
            s.record(); step(); e.record()
        torch.cuda.synchronize()
    ops.device_status()
    value = world * FLOP_PER_STEP / (ms * 1e-3) / 1e12
    # a step IS one launch of the kernel, so its average launch duration over the timed region is ms (CUDA events
    # around the K back-to-back launches); the per-launch events of the second loop (which add a gap per launch)
    # are reported beside it
    per_launch_ms = statistics.fmean(s.elapsed_time(e) for s, e in evs)
    kernel_ms = ms
    achieved = FLOP_PER_STEP / (kernel_ms * 1e-3) / 1e12
    sustained = args.steps * ms > 1000.0     # a second or more of back-to-back launches
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_kind": f"{'sustained' if sustained else 'burst'} cuBLAS bf16, {peaks['source']}",
                "frac_of_burst": achieved / peaks["bf16_tflops"],
                "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"], "frac_of_nominal_2250": achieved / 2250.0,
                "kernel": "matmul_bf16_tcgen05_2cta_kernel<6>", "kernel_ms": kernel_ms,
                "kernel_ms_per_launch_events": per_launch_ms}

    # ---- end to end through the public wrapper with pinned host buffers
    a_pin, b_pin = a_host.pin_memory(), b_host.pin_memory()
    c_pin = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    e2e_step = lambda: ops.matmul_tma(a_pin, b_pin, True, out=c_pin)
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_ms = time_region(e2e_step, e2e_steps, dist, torch)
    e2e = {"value": world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": (a_pin.numel() + b_pin.numel()) * 2, "d2h_bytes_per_step": c_pin.numel() * 2,
           "ms_per_step": e2e_ms, "steps": e2e_steps}
    del a_pin, b_pin, c_pin

    extra = {}
    if not args.no_extra:
        try:   # the headline line must not depend on a secondary workload
            extra = secondary_workloads(torch, ops, gi, peaks, dist, world, rank, a, b, c, sharding)
        except Exception as e:  # noqa: BLE001
            extra = {"error": repr(e)}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = 64
        rate, secs, threads = cpu_reference_rate(rows)
        if secs < 5.0:   # many host cores: take a larger sample, about 10-20 s
            rows = int(min(M, rows * 12.0 / max(secs, 1e-3)))
            rate, secs, threads = cpu_reference_rate(rows)
        cpu_baseline = {"value": rate, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"{rows} of {M} rows of C (all {N} columns, K={K}) in {secs:.1f} s, the reference's "
                                  "golden_matmul loop restated in oracle/oracle.c"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"bf16 matmul M=N=K={M} per GPU (global M={M * world}, B replicated), "
                                   "A,B ~ N(0,1)/sqrt(K), fp32 accumulate, bf16 out",
                       "l2": "inputs larger than L2 (A+B+C = 403 MB per GPU), no flush",
                       "parallelism": f"M-row blocks of C over {world} GPU(s), no collective"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches) * world,
            "clocks": clocks.summary(), "extra": extra,
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
    elif w == "matmul_fused":
        a = (torch.randn(16384, 4096, device="cuda") / 64).bfloat16()
        b = (torch.randn(4096, 4096, device="cuda") / 64).bfloat16()
        bias = torch.randn(4096, device="cuda") * 0.1
        c = torch.empty((16384, 4096), device="cuda", dtype=torch.bfloat16)
        fn = lambda: ops.matmul_fused(a, b, bias, "relu", out=c)
    elif w in ("add", "sin"):
        n = 1 << 26
        x, y = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
        fn = (lambda: ops.add(x, y)) if w == "add" else (lambda: ops.sin(x))
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


def secondary_workloads(torch, ops, gi, peaks, dist, world, rank, a, b, c, sharding):
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
    del xb, yb, xs

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

    # fused attention forward: Z=4, H=32, S=4096, D=128
    Z, H, S, D = 4, 32, 4096, 128
    q = torch.randn(Z, H, S, D, device="cuda").bfloat16()
    k, v = torch.randn_like(q), torch.randn_like(q)
    for causal in (False, True):
        ms = quick_ms(lambda: ops.attention(q, k, v, causal, D ** -0.5), torch, rep=20)
        fl = 4.0 * Z * H * S * S * D * (0.5 if causal else 1.0)
        t = fl / ms / 1e9
        out[f"attention_fwd_{'causal' if causal else 'full'}"] = {"ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf,
                                                                 "frac_of_nominal_2250": t / 2250.0}
    del q, k, v
    # the other head dimensions (same token count): 64 with twice the heads, 256 with half
    for (Hh, Dh) in ((64, 64), (16, 256)):
        q = torch.randn(Z, Hh, S, Dh, device="cuda").bfloat16()
        k, v = torch.randn_like(q), torch.randn_like(q)
        ms = quick_ms(lambda: ops.attention(q, k, v, False, Dh ** -0.5), torch, rep=10)
        t = 4.0 * Z * Hh * S * S * Dh / ms / 1e9
        out[f"attention_fwd_full_d{Dh}"] = {"ms": ms, "TFLOP/s": t, "frac_of_nominal_2250": t / 2250.0}
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
    ms = quick_ms(lambda: ops.matmul(at, bt, "leaky_relu", layout="tile32"), torch, rep=10)
    t = 2.0 * S_ ** 3 / ms / 1e9
    out["matmul_tile32_f16_leaky_8192"] = {"ms": ms, "TFLOP/s": t, "frac_of_burst_peak": t / tf}
    del at, bt

    if world > 1:
        # strong scaling of ONE 8192^3 problem: this rank's M-row shard; and the optional all-gather of C
        r0, r1 = sharding.row_shard(M, world, rank)
        ash, csh = a[r0:r1], c[r0:r1]
        ms = time_region(lambda: ops.matmul_tma(ash, b, True, out=csh), 20, dist, torch)
        out["strong_8192_shard"] = {"rows_per_gpu": r1 - r0, "ms": ms, "TFLOP/s_total": FLOP_PER_STEP / ms / 1e9}
        ms_ag = time_region(lambda: sharding.all_gather_rows(csh), 10, dist, torch)
        out["all_gather_C_nccl"] = {"ms": ms_ag, "bytes_out": M * N * 2, "GB/s_bus": (world - 1) / world * M * N * 2 / ms_ag / 1e6}
        # the same result from ONE kernel per rank: the matmul epilogue stores its rows into every rank's copy of C
        # over NVLink (peer-mapped buffers), followed by a one-element all-reduce as the fence
        if (r1 - r0) * world == M:
            try:   # GatheredRows raises on every rank or on none, so the ranks stay in step
                out.update(fused_gather_workloads(torch, ops, sharding, dist, world, a, b, c, ash, csh, r1 - r0))
            except Exception as e:  # noqa: BLE001
                out["matmul_plus_all_gather"] = {"error": repr(e)}
    return out


def fused_gather_workloads(torch, ops, sharding, dist, world, a, b, c, ash, csh, rows):
    """matmul followed by an NCCL all-gather of C against ONE kernel per rank whose epilogue stores its rows into every
    rank's copy of C over NVLink (peer-mapped buffers) followed by a one-element all-reduce as the fence."""
    out = {}
    gathered = sharding.GatheredRows(rows, N)
    torch.cuda.synchronize()
    dist.barrier()
    sep = lambda: sharding.all_gather_rows(ops.matmul_tma(ash, b, True, out=csh))
    fused = lambda: sharding.matmul_all_gather(ash, b, gathered)
    sep(); fused()
    ms_sep = time_region(sep, 20, dist, torch)
    ms_fused = time_region(fused, 20, dist, torch)
    sent = (world - 1) * rows * N * 2
    out["strong_8192_matmul_plus_all_gather"] = {
        "ms_matmul_then_nccl_all_gather": ms_sep, "ms_fused_epilogue_stores": ms_fused,
        "speedup": ms_sep / ms_fused, "nvlink_bytes_sent_per_gpu": sent,
        "GB/s_sent_per_gpu_fused": sent / ms_fused / 1e6}
    # weak-scaling form: every rank's full 8192-row block gathered into a [world*8192, 8192] matrix
    big = sharding.GatheredRows(M, N)
    torch.cuda.synchronize()
    dist.barrier()
    sep = lambda: sharding.all_gather_rows(ops.matmul_tma(a, b, True, out=c))
    fused = lambda: sharding.matmul_all_gather(a, b, big)
    sep(); fused()
    ms_sep = time_region(sep, 5, dist, torch)
    ms_fused = time_region(fused, 5, dist, torch)
    sent = (world - 1) * M * N * 2
    out["weak_8192_per_gpu_matmul_plus_all_gather"] = {
        "ms_matmul_then_nccl_all_gather": ms_sep, "ms_fused_epilogue_stores": ms_fused,
        "speedup": ms_sep / ms_fused, "nvlink_bytes_sent_per_gpu": sent,
        "GB/s_sent_per_gpu_fused": sent / ms_fused / 1e6,
        "TFLOP/s_total_fused": world * FLOP_PER_STEP / ms_fused / 1e9}
    return out


if __name__ == "__main__":
    main()
