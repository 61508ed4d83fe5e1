#!/usr/bin/env python
"""Benchmark of the B200 half-precision GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One JSON line on stdout (rank 0).  Metric: TFLOP/s, FLOPs counted as 2*M*N*K per GEMM as the
reference's benchmarks do (benchmark/gemm/bench_float_bf16.cpp:79 of adelj88/rocm_wmma_gemm).

Workloads (synthetic, seeded; the value distributions are the ones the target configs name):
  N = 1   "8192^3 bf16->f32, all 8 layouts": one step = eight GEMMs, one per row/column-major
          combination of A, B and C, on normal(0, 0.02) inputs cast to bf16.
  N > 1   "16384^3 bf16->bf16, A row / B col / C row, C split by column slab": rank r owns
          columns slab(r) of B and C, A is replicated; one step = every rank's slab GEMM (no
          collective on the data path).  `with_allgather` additionally times the optional NCCL
          all-gather of the C slabs.  The total problem is fixed, so scaling is "strong".
Inputs (>= 256 MB) are larger than the 126 MB L2, so no flush is needed between iterations.

`value` is timed with CUDA events on the launching stream with inputs resident in HBM; `e2e`
is the same work through the host-buffer entry point `b200_gemm_host` (pinned host memory,
host<->device copies inside the timed region).  `--impl reference` times the reference's own
CPU GEMM (test/test.hpp:59-129, compiled unmodified into oracle/_ref) on all host cores, on a
bounded sample of rows of the same workload.
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
# capture summarised in profiles/.
NCU_DRAM_BYTES_PER_LAUNCH_8192 = 1.19e9  # mean of the three captured launches: 1.37, 1.10 and 1.10 GB


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
        return {"kind": "layouts", "types": 3, "M": M, "N": N, "K": K, "sigma": 0.02,
                "cpu": (3, M, N, K, (0, 1, 0), 0.02),
                "config": {"workload": "8192^3 bf16->f32 GEMM, all 8 row/col-major layouts of A,B,C (8 GEMMs per step)",
                           "M": M, "N": N, "K": K, "layouts": LAYOUT_NAMES, "inputs": "normal(0,0.02) cast to bf16, seeded",
                           "l2": "inputs (256 MB) larger than L2; no flush"}}
    M = N = K = 16384
    return {"kind": "slab", "types": 2, "M": M, "N": N, "K": K, "sigma": 1.0,
            "cpu": (2, M, N, K, (0, 1, 0), 1.0),
            "config": {"workload": f"16384^3 bf16->bf16 GEMM, A row / B col / C row, C column slabs over {n_gpus} GPUs, A replicated",
                       "M": M, "N": N, "K": K, "layouts": ["rcr"], "inputs": "normal(0,1) cast to bf16, seeded",
                       "parallelism": f"column-slab x{n_gpus}", "l2": "inputs (>= 576 MB per GPU) larger than L2; no flush"}}


def run_b200(args, rank, world, local_rank):
    import torch
    import rocm_wmma_gemm_b200 as g
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = g.loader()
    wl = workload_for(args.gpus)
    M, N, K, types = wl["M"], wl["N"], wl["K"], wl["types"]
    gen = torch.Generator(device=dev).manual_seed(1234)
    out_dt = torch.float32 if types in (1, 3) else torch.bfloat16

    if wl["kind"] == "layouts":
        A = (torch.randn(M * K, device=dev, generator=gen) * wl["sigma"]).to(torch.bfloat16)
        B = (torch.randn(K * N, device=dev, generator=gen) * wl["sigma"]).to(torch.bfloat16)
        C = torch.empty(M * N, device=dev, dtype=out_dt)
        calls = [(C, A, B, M, N, K, lc, la, lb) for (la, lb, lc) in LAYOUTS]
        n_local = N
    else:
        n0, n_local = g.slab(N, world, rank, 256)
        A = (torch.randn(M * K, device=dev, generator=gen) * wl["sigma"]).to(torch.bfloat16)  # same seed: replicated
        gen_b = torch.Generator(device=dev).manual_seed(99 + rank)
        B = (torch.randn(K * max(n_local, 1), device=dev, generator=gen_b) * wl["sigma"]).to(torch.bfloat16)
        C = torch.empty(M * max(n_local, 1), device=dev, dtype=out_dt)
        calls = [(C, A, B, M, n_local, K, 0, 0, 1)] if n_local else []
    flops_per_step = 2.0 * M * N * K * (len(LAYOUTS) if wl["kind"] == "layouts" else 1)

    def step(events=None):
        for i, c in enumerate(calls):
            if events is not None:
                events[i].record()
            L.gemm(*c)
        if events is not None:
            events[len(calls)].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    g.device_status()

    sampler = ClockSampler(local_rank)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(calls) + 1)] for _ in range(args.steps)]
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
    per_call_ms = [[e[i].elapsed_time(e[i + 1]) for e in ev] for i in range(len(calls))]
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        lt = torch.tensor([float(launches)], device=dev, dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    total_ms_max = float(t.item())
    value = flops_per_step * args.steps / (total_ms_max * 1e-3) / 1e12

    extra = {}
    # ---- N = 1 only: the multi-GPU workload on this one GPU, so that the N > 1 lines (16384^3
    # column slabs) have a like-for-like single-GPU number next to the headline ----------------
    if wl["kind"] == "layouts" and world == 1 and not args.no_scaling_base:
        Mb = Nb = Kb = 16384
        Ab = (torch.randn(Mb * Kb, device=dev, generator=gen)).to(torch.bfloat16)
        Bb = (torch.randn(Kb * Nb, device=dev, generator=gen)).to(torch.bfloat16)
        Cb = torch.empty(Mb * Nb, device=dev, dtype=torch.bfloat16)
        for _ in range(3):
            L.gemm(Cb, Ab, Bb, Mb, Nb, Kb, 0, 0, 1)
        torch.cuda.synchronize()
        nb = max(3, min(args.steps, 10))
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(nb):
            L.gemm(Cb, Ab, Bb, Mb, Nb, Kb, 0, 0, 1)
        b1.record()
        torch.cuda.synchronize()
        extra["scaling_base"] = {"workload": "16384^3 bf16->bf16 GEMM, A row / B col / C row, whole problem on 1 GPU",
                                 "value": 2.0 * Mb * Nb * Kb * nb / (b0.elapsed_time(b1) * 1e-3) / 1e12, "unit": "TFLOP/s",
                                 "steps": nb, "note": "single-GPU point of the N>1 workload (N>1 lines shard this problem)"}
        del Ab, Bb, Cb

    # ---- optional all-gather of the C slabs (reported beside the headline, not inside it) ----
    if wl["kind"] == "slab" and world > 1 and n_local * world == N:
        gathered = torch.empty(world * M * n_local, device=dev, dtype=out_dt)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(2):
            step()
            dist.all_gather_into_tensor(gathered, C)
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
            dist.all_gather_into_tensor(gathered, C)
        e1.record()
        barrier()
        tg = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        extra["with_allgather"] = {"value": flops_per_step * args.steps / (float(tg.item()) * 1e-3) / 1e12,
                                   "unit": "TFLOP/s", "note": "slab GEMM + NCCL all_gather of C slabs ([G][M][N/G]) per step"}
        del gathered
        # the same exchange overlapped with the compute, row panel by row panel
        from rocm_wmma_gemm_b200.multi_gpu import ColumnSlabGemm
        plan = ColumnSlabGemm(M, N, K, 0, 0, 1)

        def timed(fn):
            for _ in range(2):
                fn()
            barrier()
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            barrier()
            tt = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return flops_per_step * args.steps / (float(tt.item()) * 1e-3) / 1e12

        def sequential():
            plan.run(C, A, B)
            return plan.gather(C)

        extra["with_full_c_sequential"] = {
            "value": timed(sequential), "unit": "TFLOP/s",
            "note": "ColumnSlabGemm.run then .gather: slab GEMM, all-gather, slabs interleaved into the row-major M x N matrix"}
        extra["with_full_c_overlapped"] = {
            "value": timed(lambda: plan.run_and_gather(C, A, B, panels=4)), "unit": "TFLOP/s",
            "note": "ColumnSlabGemm.run_and_gather: 4 row panels, all-gather of panel p under the GEMM of panel p+1, full C assembled"}

    # ---- end to end through the host-buffer entry point ---------------------------------------
    e2e_steps = max(1, min(args.steps, 3))
    hostA = torch.empty(A.numel(), dtype=torch.bfloat16).pin_memory()
    hostB = torch.empty(B.numel(), dtype=torch.bfloat16).pin_memory()
    hostC = torch.empty(C.numel(), dtype=out_dt).pin_memory()
    hostA.copy_(A)
    hostB.copy_(B)
    host_calls = [(hostC, hostA, hostB) + c[3:] for c in calls]
    for c in host_calls[:1]:
        L.gemm_host(*c, types=types)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for c in host_calls:
            L.gemm_host(*c, types=types)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    te = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = flops_per_step * e2e_steps / float(te.item()) / 1e12
    h2d = sum((c[1].numel() + c[2].numel()) * 2 for c in host_calls)
    d2h = sum(c[0].numel() * c[0].element_size() for c in host_calls)
    if world > 1:
        tb = torch.tensor([float(h2d), float(d2h)], device=dev, dtype=torch.float64)
        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
        h2d, d2h = int(tb[0].item()), int(tb[1].item())

    if rank == 0:
        peaks = load_peaks()
        n_launch_rank0 = len(calls) * args.steps
        avg_ms = total_ms / max(1, n_launch_rank0)
        flops_per_launch = 2.0 * M * n_local * K
        achieved = flops_per_launch / (avg_ms * 1e-3) / 1e12 if avg_ms > 0 else 0.0
        timed_s = total_ms * 1e-3
        peak_key = "bf16_tflops_sustained" if timed_s > 2.0 else "bf16_tflops"
        peak = float(peaks[peak_key])
        roofline = {"bound": "tensor", "kernel": "gemm_umma_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak,
                    "peak_source": f"{peaks['_source']} {peak_key} (timed region {timed_s:.2f} s)",
                    "frac_of_nominal_2250": achieved / 2250.0,
                    "frac_of_sustained": achieved / float(peaks["bf16_tflops_sustained"]),
                    "flops_per_launch": flops_per_launch, "avg_launch_ms": avg_ms,
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH_8192 if wl["kind"] == "layouts" else None}
        line = {
            "metric": "TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms_max / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": wl["config"],
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": "b200_gemm_host (pinned host buffers)"},
            "gpu_launches": launches, "roofline": roofline,
            "pct_of_nominal_peak": 100.0 * value / (2250.0 * args.gpus),
        }
        if wl["kind"] == "layouts":
            line["per_layout_tflops"] = {LAYOUT_NAMES[i]: 2.0 * M * N * K / (statistics.median(per_call_ms[i]) * 1e-3) / 1e12
                                         for i in range(len(calls))}
            line["per_layout_tflops_best"] = {LAYOUT_NAMES[i]: 2.0 * M * N * K / (min(per_call_ms[i]) * 1e-3) / 1e12
                                              for i in range(len(calls))}
        line.update(extra)
        if args.gpus == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl["cpu"])
        emit_line(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    ap.add_argument("--no-scaling-base", action="store_true", help="skip the 16384^3 single-GPU point (profiling runs)")
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
