#!/usr/bin/env python
"""Benchmark of the B200 half-precision GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One JSON line on stdout (rank 0).  Metric: TFLOP/s, FLOPs counted as 2*M*N*K per GEMM as the
reference's benchmarks do (benchmark/gemm/bench_float_bf16.cpp:79 of adelj88/rocm_wmma_gemm).

Workloads (synthetic, seeded; the value distributions are the ones the target configs name):
  N = 1   "8192^3 bf16->f32, all 8 layouts": one step = R = 16 passes over the eight row/column-
          major combinations of A, B and C (128 GEMMs), on normal(0, 0.02) inputs cast to bf16.
          With the default 20 steps the timed region lasts about 2 s: `value` is a SUSTAINED
          figure under the power cap.  `burst` holds the best call per layout after an idle
          pause, `per_call` the p10/p50/p90 of the sustained region, `cycles_per_launch` the
          mean call time x the median SM clock sampled during it.
  N > 1   "16384^3 bf16->bf16, A row / B col / C row, C split by column slab": rank r owns
          columns slab(r) of B and C, A is replicated; one step = R slab GEMMs per rank (R
          grows with N so that the region lasts about a second; no collective on the data
          path).  Beside it, outside the timed region: `parity` (the gathered C against the CPU
          reference on sampled rows and columns), `same_workload_base` (the whole 16384^3
          problem on rank 0's GPU alone) with `efficiency_same_workload`, and the step with each
          of the three gathers of C inside it.  The total problem is fixed: scaling is "strong".
Inputs (>= 256 MB) are larger than the 126 MB L2, so no flush is needed between iterations.

`value` is timed with CUDA events on the launching stream with inputs resident in HBM; `e2e`
is the same work through the host-buffer entry points (`b200_gemm_host`; `b200_gemm_slab_host`
for N > 1: pinned host memory, host<->device copies inside the timed region).
`--impl reference` times the reference's own CPU GEMM (test/test.hpp:59-129, compiled unmodified
into oracle/_ref) on all host cores, on a bounded sample of rows of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYOUTS = [(la, lb, lc) for la in (0, 1) for lb in (0, 1) for lc in (0, 1)]  # (A, B, C); 0 row, 1 col
LAYOUT_NAMES = ["".join("rc"[x] for x in l) for l in LAYOUTS]
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes (read + write) of one 8192^3 bf16->f32 launch of gemm_umma_kernel, from the ncu
# capture summarised in profiles/gemm_umma_8192cubed_bf16_f32.md.
NCU_DRAM_BYTES_PER_LAUNCH_8192 = 1.079e9  # 0.841 GB read + 0.237 GB written
REPEATS_N1 = 16  # passes over the 8 layouts per step: 20 steps x 128 GEMMs x ~0.8 ms = 2 s


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    _BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
             0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting"}

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append(mhz)
                for b, name in self._BITS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# --------------------------------------------------------------------------------------------
# CPU arm: the reference's hgemm_cpu on a bounded sample of rows
# --------------------------------------------------------------------------------------------
def make_host_inputs(M, N, K, sigma, seed, bf16=True):
    """Raw 16-bit patterns (numpy uint16) of A (M x K) and B (K x N), normal(0, sigma)."""
    import numpy as np
    import torch
    gen = torch.Generator().manual_seed(seed)
    dt = torch.bfloat16 if bf16 else torch.float16
    A = (torch.randn(M * K, generator=gen) * sigma).to(dt).view(torch.int16).numpy().view(np.uint16)
    B = (torch.randn(K * N, generator=gen) * sigma).to(dt).view(torch.int16).numpy().view(np.uint16)
    return A, B


def cpu_rows_runner(types, M, N, K, lc, la, lb, A, B):
    """Returns (kind, cores, fn) where fn(rows) runs the CPU GEMM on rows [0, rows) and returns
    seconds.  Uses the compiled reference when present, else the C restatement."""
    import numpy as np
    import oracle
    cores = host_cores()
    out_dt = oracle.out_dtype(types)
    ref = oracle.ref_lib()
    if ref is not None:
        def run(rows):
            C = np.empty(rows * N, dtype=out_dt)
            t0 = time.perf_counter()
            ref.ref_hgemm_rows_mt(types, C.ctypes.data, A.ctypes.data, B.ctypes.data, M, N, K, lc, la, lb, 0, rows, cores)
            return time.perf_counter() - t0
        return "reference", cores, run
    lib = oracle.oracle_lib()

    def run(rows):
        C = np.empty(M * N, dtype=out_dt)
        t0 = time.perf_counter()
        lib.oracle_hgemm_rows(types, C.ctypes.data, A.ctypes.data, B.ctypes.data, M, N, K, lc, la, lb, 0, rows, cores)
        return time.perf_counter() - t0
    return "port", cores, run


def calibrate_rows(run, M, cores, target_s):
    """Rows of C that take about target_s: two short runs separate the fixed cost of a call
    (placing B in the reference's matrix class) from the cost per row."""
    r1, r2 = min(M, cores), min(M, 4 * cores)
    t1, t2 = run(r1), run(r2)
    per_row = max((t2 - t1) / max(r2 - r1, 1), 1e-9) if r2 > r1 else t1 / r1
    fixed = max(t1 - r1 * per_row, 0.0)
    want = int(max(cores, min(M, (target_s - fixed) / per_row)))
    return max(cores, (want // cores) * cores)


def cpu_baseline(workload, target_s=12.0):
    types, M, N, K, (la, lb, lc), sigma = workload
    A, B = make_host_inputs(M, N, K, sigma, seed=11, bf16=types >= 2)
    kind, cores, run = cpu_rows_runner(types, M, N, K, lc, la, lb, A, B)
    rows = calibrate_rows(run, M, cores, target_s)
    t = run(rows)
    return {"value": 2.0 * rows * N * K / t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"rows [0,{rows}) of C for {M}x{N}x{K}, A {'rc'[la]} / B {'rc'[lb]} / C {'rc'[lc]} "
                      f"({2.0 * rows * N * K / 1e9:.1f} GFLOP in {t:.1f} s)"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    workload = workload_for(args.gpus)
    types, M, N, K, (la, lb, lc), sigma = workload["cpu"]
    A, B = make_host_inputs(M, N, K, sigma, seed=11, bf16=types >= 2)
    kind, cores, run = cpu_rows_runner(types, M, N, K, lc, la, lb, A, B)
    per_step = max(0.5, min(3.0, 150.0 / max(1, args.steps + args.warmup)))
    rows = calibrate_rows(run, M, cores, per_step)
    for _ in range(args.warmup):
        run(rows)
    times = [run(rows) for _ in range(args.steps)]
    total = sum(times)
    value = 2.0 * rows * N * K * args.steps / total / 1e12
    sample = (f"each step = rows [0,{rows}) of C for {M}x{N}x{K} A {'rc'[la]} / B {'rc'[lb]} / C {'rc'[lc]} "
              f"({2.0 * rows * N * K / 1e9:.1f} GFLOP)")
    line = {
        "impl": "reference", "metric": "TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload["config"],
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_line(line)


# --------------------------------------------------------------------------------------------
# Workloads
# --------------------------------------------------------------------------------------------
def workload_for(n_gpus):
    if n_gpus == 1:
        M = N = K = 8192
        return {"kind": "layouts", "types": 3, "M": M, "N": N, "K": K, "sigma": 0.02, "repeats": REPEATS_N1,
                "cpu": (3, M, N, K, (0, 1, 0), 0.02),
                "config": {"workload": f"8192^3 bf16->f32 GEMM, all 8 row/col-major layouts of A,B,C; one step = {REPEATS_N1} passes "
                                       f"over the 8 layouts ({8 * REPEATS_N1} GEMMs), sustained under the power cap",
                           "M": M, "N": N, "K": K, "layouts": LAYOUT_NAMES, "gemms_per_step": 8 * REPEATS_N1,
                           "inputs": "normal(0,0.02) cast to bf16, seeded",
                           "l2": "inputs (256 MB) larger than L2; no flush"}}
    M = N = K = 16384
    repeats = 8 * n_gpus  # one slab GEMM lasts about 6.3 ms / n_gpus: 20 steps make a region of about a second
    return {"kind": "slab", "types": 2, "M": M, "N": N, "K": K, "sigma": 1.0, "repeats": repeats,
            "cpu": (2, M, N, K, (0, 1, 0), 1.0),
            "config": {"workload": f"16384^3 bf16->bf16 GEMM, A row / B col / C row, C column slabs over {n_gpus} GPUs, A replicated; "
                                   f"one step = {repeats} slab GEMMs per GPU",
                       "M": M, "N": N, "K": K, "layouts": ["rcr"], "gemms_per_step": repeats,
                       "inputs": "normal(0,1) cast to bf16, seeded",
                       "parallelism": f"column-slab x{n_gpus}", "l2": "inputs (>= 576 MB per GPU) larger than L2; no flush"}}


def percentiles(xs):
    xs = sorted(xs)
    pick = lambda q: xs[min(len(xs) - 1, int(q * (len(xs) - 1) + 0.5))]
    return {"p10": pick(0.1), "p50": pick(0.5), "p90": pick(0.9)}


def run_b200(args, rank, world, local_rank):
    import numpy as np
    import torch
    import rocm_wmma_gemm_b200 as g
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = g.loader()
    wl = workload_for(args.gpus)
    M, N, K, types, R = wl["M"], wl["N"], wl["K"], wl["types"], wl["repeats"]
    gen = torch.Generator(device=dev).manual_seed(1234)
    out_dt = torch.float32 if types in (1, 3) else torch.bfloat16
    layouts = wl["kind"] == "layouts"

    def slab_of_b(r, n_cols):
        """Rank r's B slab (K x n_cols, column-major = n_cols rows of K), seeded by r."""
        gen_b = torch.Generator(device=dev).manual_seed(99 + r)
        return (torch.randn(K * max(n_cols, 1), device=dev, generator=gen_b) * wl["sigma"]).to(torch.bfloat16)

    if layouts:
        A = (torch.randn(M * K, device=dev, generator=gen) * wl["sigma"]).to(torch.bfloat16)
        B = (torch.randn(K * N, device=dev, generator=gen) * wl["sigma"]).to(torch.bfloat16)
        C = torch.empty(M * N, device=dev, dtype=out_dt)
        calls = [(C, A, B, M, N, K, lc, la, lb) for (la, lb, lc) in LAYOUTS]
        n_local = N
    else:
        n0, n_local = g.slab(N, world, rank, 256)
        A = (torch.randn(M * K, device=dev, generator=gen) * wl["sigma"]).to(torch.bfloat16)  # same seed: replicated
        B = slab_of_b(rank, n_local)
        C = torch.empty(M * max(n_local, 1), device=dev, dtype=out_dt)
        calls = [(C, A, B, M, n_local, K, 0, 0, 1)] if n_local else []
    ncall = len(calls)
    flops_per_step = 2.0 * M * N * K * R * (len(LAYOUTS) if layouts else 1)

    def step(events=None):
        """R passes over the step's calls; with `events`, one event before each call and one at the end."""
        i = 0
        for _ in range(R):
            for c in calls:
                if events is not None:
                    events[i].record()
                    i += 1
                L.gemm(*c)
        if events is not None:
            events[i].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for c in calls:  # load every kernel this workload uses
        L.gemm(*c)
    barrier()
    g.device_status()

    # ---- burst: the best single call per layout after an idle pause (boost clocks, power budget
    # recovered); N = 1 only, before the sustained region heats the part up ------------------------
    burst = None
    if layouts and world == 1:
        burst = {}
        for i, c in enumerate(calls):
            torch.cuda.synchronize()
            time.sleep(0.25)
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
            for k in range(4):
                evs[k].record()
                L.gemm(*c)
            evs[4].record()
            torch.cuda.synchronize()
            burst[LAYOUT_NAMES[i]] = 2.0 * M * N * K / (min(evs[k].elapsed_time(evs[k + 1]) for k in range(4)) * 1e-3) / 1e12

    for _ in range(args.warmup):
        step()
    barrier()

    sampler = ClockSampler(local_rank)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(R * ncall + 1)] for _ in range(args.steps)]
    launches0 = g.launch_count()
    sampler.start()
    barrier()
    for s in range(args.steps):
        step(ev[s])
    barrier()
    clocks = sampler.stop()
    launches = g.launch_count() - launches0
    g.device_status()

    step_ms = [e[0].elapsed_time(e[-1]) for e in ev] if calls else [0.0] * args.steps
    total_ms = sum(step_ms)
    # per_call_ms[i]: every timed call of calls[i] (R per step)
    per_call_ms = [[e[r * ncall + i].elapsed_time(e[r * ncall + i + 1]) for e in ev for r in range(R)] for i in range(ncall)]
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        lt = torch.tensor([float(launches)], device=dev, dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    total_ms_max = float(t.item())
    value = flops_per_step * args.steps / (total_ms_max * 1e-3) / 1e12

    extra = {}
    # ---- the vendor GEMM on the same GPU in the same run (N = 1): GPUs of this pool settle at
    # different clocks under the 1 kW cap, so a sustained figure only means something next to the
    # vendor library's on the same part ------------------------------------------------------------
    if layouts and world == 1 and not args.no_vendor:
        a2, b2 = A.view(M, K), B.view(N, K)
        o2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        o2f = o2.view(-1)
        runs = {
            "vendor_bf16_out": lambda: torch.matmul(a2, b2.t(), out=o2),
            "this_f32_out": lambda: L.gemm(C, A, B, M, N, K, 0, 0, 1),
            "this_bf16_out": lambda: L.gemm(o2f, A, B, M, N, K, 0, 0, 1),
        }
        for fn in runs.values():
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        time.sleep(0.25)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        for k in range(4):
            evs[k].record()
            runs["vendor_bf16_out"]()
        evs[4].record()
        torch.cuda.synchronize()
        v_burst = 2.0 * M * N * K / (min(evs[k].elapsed_time(evs[k + 1]) for k in range(4)) * 1e-3) / 1e12
        for _ in range(300):  # warm the part up again
            runs["this_f32_out"]()
        block, rounds = 200, 4  # interleaved blocks: every variant sees the same thermal and power state
        times = {k: [] for k in runs}
        vs = ClockSampler(local_rank)
        vs.start()
        v0, v1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(rounds):
            for name, fn in runs.items():
                v0.record()
                for _ in range(block):
                    fn()
                v1.record()
                torch.cuda.synchronize()
                times[name].append(v0.elapsed_time(v1) / block)
        vclk = vs.stop()
        rate = {k: 2.0 * M * N * K / (statistics.median(v) * 1e-3) / 1e12 for k, v in times.items()}
        extra["vendor_same_run"] = {"sustained": rate, "unit": "TFLOP/s", "vendor_burst": v_burst, "sm_mhz": vclk.get("sm_mhz"),
                                    "this_over_vendor_bf16_out": rate["this_bf16_out"] / rate["vendor_bf16_out"],
                                    "note": "8192^3 A row / B col / C row on the same GPU right after the timed region: torch.matmul "
                                            "(vendor GEMM, bf16 out) and this library (f32 out as in the workload, and bf16 out like "
                                            f"the vendor call) in interleaved blocks of {block} calls, {rounds} rounds, median per variant; "
                                            "vendor_burst = best of 4 after 0.25 s idle"}
        del o2, o2f
    if world > 1 and wl["kind"] == "slab":
        try:
            extra.update(multi_gpu_extras(args, g, L, dist, dev, rank, world, wl, A, B, C, n_local, slab_of_b, barrier, value))
        except Exception as ex:  # the compute-only line must survive a failure of what is reported beside it
            extra["multi_gpu_extras_error"] = f"{type(ex).__name__}: {ex}"[:400]

    # ---- end to end through the host-buffer entry points -----------------------------------------
    e2e_steps = max(1, min(args.steps, 3))
    hostA = torch.empty(A.numel(), dtype=torch.bfloat16).pin_memory()
    hostB = torch.empty(B.numel(), dtype=torch.bfloat16).pin_memory()
    hostC = torch.empty(C.numel(), dtype=out_dt).pin_memory()
    hostA.copy_(A)
    hostB.copy_(B)
    if world == 1:
        host_calls = [(hostC, hostA, hostB) + c[3:] for c in calls]
        run_host = lambda: [L.gemm_host(*c, types=types) for c in host_calls]
        api = "b200_gemm_host (pinned host buffers); one e2e step = one pass over the 8 layouts"
        h2d = sum((c[1].numel() + c[2].numel()) * 2 for c in host_calls)
        e2e_flops = 2.0 * M * N * K * len(host_calls)
    else:
        from rocm_wmma_gemm_b200.multi_gpu import SlabDriver
        hdrv = SlabDriver(M, N, K, types, 0, 0, 1, align=256, peer_buffers=False)
        run_host = lambda: hdrv.gemm_host(hostC, hostA, hostB)
        api = ("b200_gemm_slab_host (pinned host buffers; each GPU uploads 1/N of A and its B slab, NCCL all-gather of A over "
               "NVLink, C slab back); one e2e step = one 16384^3 problem")
        h2d = (hostA.numel() // world + hostB.numel()) * 2
        e2e_flops = 2.0 * M * N * K
    run_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        run_host()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    te = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    d2h = hostC.numel() * hostC.element_size() * (len(calls) if world == 1 else 1)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        tb = torch.tensor([float(h2d), float(d2h)], device=dev, dtype=torch.float64)
        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
        h2d, d2h = int(tb[0].item()), int(tb[1].item())
        hdrv.close()
    e2e_value = e2e_flops * e2e_steps / float(te.item()) / 1e12

    if rank == 0:
        peaks = load_peaks()
        n_launch_rank0 = R * ncall * args.steps
        avg_ms = total_ms / max(1, n_launch_rank0)
        flops_per_launch = 2.0 * M * n_local * K
        achieved = flops_per_launch / (avg_ms * 1e-3) / 1e12 if avg_ms > 0 else 0.0
        timed_s = total_ms * 1e-3
        peak_key = "bf16_tflops_sustained" if timed_s >= 1.0 else "bf16_tflops"
        peak = float(peaks[peak_key])
        roofline = {"bound": "tensor", "kernel": "gemm_umma_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak,
                    "peak_source": f"{peaks['_source']} {peak_key} (timed region {timed_s:.2f} s)",
                    "frac_of_nominal_2250": achieved / 2250.0,
                    "frac_of_burst_peak": achieved / float(peaks["bf16_tflops"]),
                    "flops_per_launch": flops_per_launch, "avg_launch_ms": avg_ms,
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH_8192 if layouts else None}
        mhz = clocks.get("sm_mhz")
        line = {
            "metric": "TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms_max / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "timed_region_s": total_ms_max * 1e-3, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": api},
            "gpu_launches": launches, "roofline": roofline,
            "pct_of_nominal_peak": 100.0 * value / (2250.0 * args.gpus),
            "cycles_per_launch": (avg_ms * 1e-3 * mhz * 1e6) if mhz else None,
        }
        line.update(extra)
        names = LAYOUT_NAMES if layouts else ["rcr"]
        line["per_call"] = {names[i]: {k: 2.0 * M * n_local * K / (v * 1e-3) / 1e12
                                       for k, v in zip(("p90", "p50", "p10"), percentiles(per_call_ms[i]).values())}
                            for i in range(ncall)}  # TFLOP/s: the p10 of time is the p90 of rate
        if layouts:
            line["per_layout_tflops"] = {names[i]: line["per_call"][names[i]]["p50"] for i in range(ncall)}
            line["sustained_min_layout"] = min(2.0 * M * N * K / (statistics.mean(per_call_ms[i]) * 1e-3) / 1e12 for i in range(ncall))
        if burst is not None:
            line["burst"] = {"per_layout": burst, "min": min(burst.values()), "max": max(burst.values()),
                             "method": "best of 4 back-to-back calls per layout after 0.25 s idle"}
        if args.gpus == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl["cpu"])
        line["config"] = wl["config"]  # the long object last: a truncated tail keeps the numbers
        emit_line(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def multi_gpu_extras(args, g, L, dist, dev, rank, world, wl, A, B, C, n_local, slab_of_b, barrier, value):
    """What the N > 1 line reports beside the compute-only step (all outside its timed region):
    parity of the gathered C, the same problem on one GPU, and the step with each gather inside."""
    import numpy as np
    import torch
    from rocm_wmma_gemm_b200.multi_gpu import SlabDriver
    M, N, K, types = wl["M"], wl["N"], wl["K"], wl["types"]
    out = {}
    even = n_local * world == N
    drv = SlabDriver(M, N, K, types, 0, 0, 1, align=256)
    full = drv.full_c
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    flops = 2.0 * M * N * K

    def timed(fn, reps):
        for _ in range(2):
            fn()
        barrier()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        barrier()
        tt = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return flops * reps / (float(tt.item()) * 1e-3) / 1e12, float(tt.item()) / reps

    # Every variant is timed the same way and for about half a second (sustained clocks, like the
    # main region), compute-only included, in two interleaved rounds; the better round counts.
    reps = max(20, int(0.5 / (0.0065 / world)))
    # ---- the three gathers, each inside the step ---------------------------------------------
    def plain():
        L.gemm(C, A, B, M, n_local, K, 0, 0, 1)

    def fused():
        drv.gemm_gather(A, B)
        drv.barrier()

    def pushed():
        L.gemm(C, A, B, M, n_local, K, 0, 0, 1)
        drv.push(C)
        drv.barrier()

    staging = torch.empty(M * N, device=dev, dtype=C.dtype)

    def nccl():
        L.gemm(C, A, B, M, n_local, K, 0, 0, 1)
        drv.allgather(full, C, staging)

    if even:
        variants = {"compute_only": plain, "with_fused_gather": fused, "with_push_gather": pushed, "with_allgather": nccl}
        best = {}
        for _ in range(2):
            for name, fn in variants.items():
                v, ms = timed(fn, reps)
                if name not in best or v > best[name][0]:
                    best[name] = (v, ms)
        notes = {"compute_only": "slab GEMM alone, timed like the three below",
                 "with_fused_gather": "b200_gemm_slab_gather + barrier: every tile stored into all GPUs' full C by the GEMM's epilogue",
                 "with_push_gather": "slab GEMM, b200_gemm_slab_push (copy engines, strided peer copies), barrier",
                 "with_allgather": "slab GEMM, b200_gemm_slab_allgather (NCCL all-gather into [G][M][N/G] + re-layout kernel)"}
        base_v = best["compute_only"][0]
        for name, (v, ms) in best.items():
            out[name if name != "compute_only" else "compute_only_same_method"] = {
                "value": v, "unit": "TFLOP/s", "ms": ms, "frac_of_compute_only": v / base_v, "reps": reps, "note": notes[name]}
        # parity of what the fused step leaves on rank 0: sampled rows and columns against the CPU reference
        full.zero_()
        barrier()
        fused()
        torch.cuda.synchronize()
        barrier()
        got = full.view(M, N)
        rng = np.random.default_rng(3)
        rows = sorted(set([0, 255, 256, M - 1] + [int(x) for x in rng.integers(0, M, 4)]))
        cols = sorted(set([0, n_local - 1, n_local, N - 1] + [int(x) for x in rng.integers(0, N, 4)]))
        got_rows = got[rows].float().cpu().numpy()
        got_cols = got[:, cols].float().cpu().numpy()
        bus = (world - 1) / world * M * N * C.element_size()
        e0.record()
        for _ in range(10):
            drv.allgather(full, C, staging)
        e1.record()
        barrier()
        ag_ms = e0.elapsed_time(e1) / 10
        out["allgather_alone"] = {"ms": ag_ms, "bus_GBps": bus / (ag_ms * 1e-3) / 1e9,
                                  "note": "all-gather + re-layout alone; bus bandwidth = (G-1)/G x bytes of C / time; NVLink "
                                          "reference on this pool: 725 GB/s all-reduce bus, 770 GB/s peer copy"}
    # ---- the whole problem on rank 0's GPU while the others idle -----------------------------
    barrier()
    base = torch.zeros(1, device=dev, dtype=torch.float64)
    if rank == 0:
        Bf = torch.cat([slab_of_b(r, g.slab(N, world, r, 256)[1])[: K * g.slab(N, world, r, 256)[1]] for r in range(world)])
        Cf = torch.empty(M * N, device=dev, dtype=C.dtype)
        for _ in range(3):
            L.gemm(Cf, A, Bf, M, N, K, 0, 0, 1)
        torch.cuda.synchronize()
        nb = max(10, int(1.0 / 0.0065))
        e0.record()
        for _ in range(nb):
            L.gemm(Cf, A, Bf, M, N, K, 0, 0, 1)
        e1.record()
        torch.cuda.synchronize()
        base[0] = flops * nb / (e0.elapsed_time(e1) * 1e-3) / 1e12
        if even:
            # CPU reference on the sampled rows and columns (rank 0 holds A and, now, all of B)
            import oracle
            A_bits = A.view(torch.int16).cpu().numpy().view(np.uint16)
            B_bits = Bf.view(torch.int16).cpu().numpy().view(np.uint16)
            ref_r = oracle.bits_to_f32(oracle.hgemm_select(types, A_bits, B_bits, M, N, K, 0, 0, 1, rows=rows), True).reshape(M, N)[rows]
            ref_c = oracle.bits_to_f32(oracle.hgemm_select(types, A_bits, B_bits, M, N, K, 0, 0, 1, cols=cols), True).reshape(M, N)[:, cols]
            d = np.concatenate([(got_rows - ref_r).ravel(), (got_cols - ref_c).ravel()]).astype(np.float64)
            r = np.concatenate([ref_r.ravel(), ref_c.ravel()]).astype(np.float64)
            rel = float(np.sqrt((d ** 2).sum()) / np.sqrt((r ** 2).sum()))
            # bf16 output of a sum of K unit-variance products: |err| <= 2 eps |ref| + eps sqrt(K)
            eps = 2.0 ** -8
            ok = bool((np.abs(d) <= 2 * eps * np.abs(r) + eps * np.sqrt(K)).all())
            out["parity"] = {"rel_fro": rel, "ok": ok, "checked": f"{len(rows)} rows + {len(cols)} columns of the fused-gather C on rank 0 "
                             "against the CPU reference (oracle.hgemm_select)", "tolerance": "per element 2*2^-8*|ref| + 2^-8*sqrt(K)"}
            whole = Cf.view(M, N)
            out["parity"]["bit_equal_to_one_gpu_result"] = bool(torch.equal(whole[rows].float().cpu(), torch.from_numpy(got_rows)))
        del Bf, Cf
    barrier()
    if world > 1:
        dist.all_reduce(base, op=dist.ReduceOp.MAX)
    b = float(base.item())
    out["same_workload_base"] = {"value": b, "unit": "TFLOP/s", "note": "the whole 16384^3 bf16->bf16 problem on rank 0's GPU alone, ~1 s back to back"}
    out["efficiency_same_workload"] = value / (world * b) if b > 0 else None
    for k in ("compute_only_same_method", "with_fused_gather", "with_push_gather", "with_allgather"):
        if k in out and b > 0:
            out[k]["efficiency_same_workload"] = out[k]["value"] / (world * b)
    drv.close()
    return out


class _QuietStdout:
    """Keeps stdout for the one JSON line: while active, file descriptor 1 points at stderr, so
    anything a library prints (NCCL's version banner, for one) cannot precede or follow it."""

    def __enter__(self):
        sys.stdout.flush()
        self._real = os.dup(1)
        os.dup2(2, 1)
        return self

    def emit(self, text: str):
        os.write(self._real, (text + "\n").encode())

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self._real, 1)
        os.close(self._real)
        return False


_OUT = None


def emit_line(obj):
    text = json.dumps(obj)
    if _OUT is not None:
        _OUT.emit(text)
    else:
        print(text, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--no-vendor", action="store_true", help="skip the vendor GEMM yardstick (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    global _OUT
    with _QuietStdout() as out:
        _OUT = out
        try:
            if args.impl == "reference":
                run_reference(args, rank, world)
                return
            if world != args.gpus:
                raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun --nproc-per-node {args.gpus}); "
                                 f"got WORLD_SIZE={world}")
            run_b200(args, rank, world, local_rank)
        finally:
            _OUT = None


if __name__ == "__main__":
    main()
