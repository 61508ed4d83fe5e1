"""Where a GEMM launch spends its time: clock stamps from inside the kernels.

    python -m rocm_wmma_gemm_b200.timeline --type bf16_bf16 --shapes 1024,1024,1024 128,8192,8192

loads the timeline build of the library (`build.py --timeline`: the same sources compiled with
-DB200_GEMM_TIMELINE, whose kernels stamp clock64() at fixed points of the producer, MMA and
epilogue roles of CTA 0 and globaltimer at three points of every CTA; csrc/gemm_kernels.cuh
lists the points), replays each problem from a CUDA graph of back-to-back launches and prints

  * the median stamp of the launches in the middle of the last replay, in SM cycles after the
    point where the kernel before it had completed (the dependency wait of the producer),
  * the time from one launch's first load to the next one's, i.e. the cost of a call,
  * how evenly the CTAs of the last launch ran: first load, end of the main loop and end of each
    CTA relative to the earliest first load.

`B200_GEMM_CONFIG` and the other environment knobs of the library apply as usual.  The timeline
build is a profiling aid: its stamps cost a few global stores per launch, so its absolute times
are a few per cent above the normal build's.
"""
from __future__ import annotations

import argparse
import ctypes
import sys

import numpy as np

from . import build as lib_build

POINTS = ["entry", "set-up done", "dependency wait done", "first TMA load issued", "last TMA load issued",
          "first ring slot full", "last accumulator committed", "MMAs drained", "accumulator seen by epilogue",
          "first store issued", "last store issued", "staging buffers read", "tail barrier", "TMEM freed"]
CLUSTER_POINTS = ["before 1st cluster barrier", "after 1st cluster barrier", "partials sent",
                  "after 2nd cluster barrier", "sums stored", "staging buffers read (cluster)"]
ROWS, SLOTS, CTAS = 64, 24, 1024
TYPES = {"f16_f16": 0, "f32_f16": 1, "bf16_bf16": 2, "f32_bf16": 3}
_ARGS = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 4 + [ctypes.c_int] * 3 + [ctypes.c_void_p]


def load() -> ctypes.CDLL:
    lib = ctypes.CDLL(lib_build.build_timeline(), mode=ctypes.RTLD_LOCAL)
    for name in TYPES:
        out, inp = name.split("_")
        fn = getattr(lib, f"b200_gemm_{out}_{inp}")
        fn.restype, fn.argtypes = ctypes.c_int, _ARGS
    lib.b200_gemm_debug_timeline.restype = ctypes.c_int
    lib.b200_gemm_debug_cta_times.restype = ctypes.c_int
    lib.b200_gemm_debug_reset.restype = ctypes.c_int
    return lib


def run(lib, type_name: str, M: int, N: int, K: int, layouts=(0, 1, 0), launches: int = 20) -> dict:
    import torch
    la, lb, lc = layouts
    out_name, in_name = type_name.split("_")
    dt = torch.float16 if in_name == "f16" else torch.bfloat16
    odt = torch.float32 if out_name == "f32" else dt
    A = (torch.rand(M * K, device="cuda") * 2 - 1).to(dt)
    B = (torch.rand(K * N, device="cuda") * 2 - 1).to(dt)
    C = torch.empty(M * N, device="cuda", dtype=odt)
    fn_c = getattr(lib, f"b200_gemm_{out_name}_{in_name}")

    def call():
        box = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        st = fn_c(C.data_ptr(), A.data_ptr(), B.data_ptr(), M, N, K, 1, lc, la, lb, ctypes.byref(box))
        if st != 0:
            raise RuntimeError(f"b200_gemm_{out_name}_{in_name} returned {st}")
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            call()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    if lib.b200_gemm_debug_reset() != 0:   # only this replay's stamps are read
        raise RuntimeError("b200_gemm_debug_reset failed")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    per_call_us = e0.elapsed_time(e1) / launches * 1e3

    buf = (ctypes.c_ulonglong * (ROWS * SLOTS))()
    count = ctypes.c_uint(0)
    if lib.b200_gemm_debug_timeline(buf, ctypes.byref(count)) != 0:
        raise RuntimeError("b200_gemm_debug_timeline failed")
    t = np.array(buf[:], dtype=np.int64).reshape(ROWS, SLOTS)
    n = count.value
    lo = max(0, n - min(launches, ROWS))
    picked = [i for i in range(lo + min(4, max(0, n - lo - 3)), n - 1)]   # the middle of the last replay
    rel, nxt, ks = [], [], []
    for i in picked:
        a, b = t[i % ROWS].astype(np.float64), t[(i + 1) % ROWS].astype(np.float64)
        stamped = lambda x: np.where(x > 0, x - a[3], np.nan)   # a point this kernel variant does not pass stays 0
        rel.append(stamped(a[1:15]))
        nxt.append(b[0] - a[0])
        ks.append(stamped(a[16:22]))
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)   # a column of points this kernel never passes is all NaN
        rel, ks = np.nanmedian(np.array(rel), axis=0), np.nanmedian(np.array(ks), axis=0)
    cta = (ctypes.c_ulonglong * (3 * CTAS))()
    if lib.b200_gemm_debug_cta_times(cta) != 0:
        raise RuntimeError("b200_gemm_debug_cta_times failed")
    c = np.array(cta[:], dtype=np.int64).reshape(3, CTAS)
    return {"per_call_us": per_call_us, "cycles_after_wait": rel, "cluster_cycles_after_wait": ks,
            "entry_to_next_entry_ns": float(np.median(nxt)), "cta_times": c}


def report(name: str, r: dict, out=sys.stdout) -> None:
    print(f"== {name}: {r['per_call_us']:.2f} us per call (graph replay)", file=out)
    for k, nm in enumerate(POINTS):
        v = r["cycles_after_wait"][k]
        print(f"   {nm:32s} " + (f"{v:9.0f} cycles" if np.isfinite(v) else "        - (not on this kernel's path)"), file=out)
    if np.all(np.isfinite(r["cluster_cycles_after_wait"])):   # stamped only by the kernels with cluster K partitions
        for k, nm in enumerate(CLUSTER_POINTS):
            print(f"   {nm:32s} {r['cluster_cycles_after_wait'][k]:9.0f} cycles", file=out)
    print(f"   entry of one launch to entry of the next: {r['entry_to_next_entry_ns'] / 1e3:.2f} us", file=out)
    c = r["cta_times"]
    live = c[1] > 0
    if live.any():
        first, loop_end, end = c[0][live], c[2][live], c[1][live]
        if len(first):
            t0 = first.min()
            q = lambda x: " ".join(f"{v / 1e3:7.1f}" for v in np.percentile(x, [0, 10, 50, 90, 100]))
            print(f"   {len(first)} CTAs, us after the earliest first load (min p10 p50 p90 max):", file=out)
            print(f"      first load          {q(first - t0)}", file=out)
            print(f"      end of main loop    {q(loop_end - t0)}", file=out)
            print(f"      end of CTA          {q(end - t0)}", file=out)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Clock stamps from inside the GEMM kernels (timeline build).")
    p.add_argument("--type", default="bf16_bf16", choices=list(TYPES))
    p.add_argument("--shapes", nargs="+", default=["1024,1024,1024"], help="M,N,K ...")
    p.add_argument("--layouts", default="r,c,r", help="A,B,C as r/c letters")
    p.add_argument("--launches", type=int, default=20, help="launches per CUDA graph")
    args = p.parse_args(argv)
    lay = tuple({"r": 0, "c": 1}[x] for x in args.layouts.split(","))
    lib = load()
    for s in args.shapes:
        M, N, K = (int(x) for x in s.split(","))
        report(f"{M}x{N}x{K} {args.type} {args.layouts}", run(lib, args.type, M, N, K, lay, args.launches))
    return 0


if __name__ == "__main__":
    sys.exit(main())
