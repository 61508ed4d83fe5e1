"""Builds the sm_100a shared library in-tree with nvcc.

The single library `librocm_wmma_gemm_sm100a.so` takes the place of the reference's
per-architecture `librocm_wmma_gemm_<arch>.so` objects
(rocm_wmma_gemm/CMakeLists.txt:5-93 of the reference): one target architecture, one build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT_DIR = os.path.dirname(PKG_DIR)
LIB_NAME = "librocm_wmma_gemm_sm100a.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
# The same sources with -DB200_GEMM_TIMELINE: kernels that stamp clock values at fixed points of
# every launch (see csrc/gemm_kernels.cuh and timeline.py).  A profiling build, never loaded by
# the package itself.
TIMELINE_LIB_PATH = os.path.join(PKG_DIR, "librocm_wmma_gemm_sm100a_timeline.so")
SOURCES = [os.path.join(PKG_DIR, "csrc", "gemm_lib.cu")]
DEPENDS = SOURCES + [
    os.path.join(PKG_DIR, "csrc", "gemm_kernels.cuh"),
    os.path.join(PKG_DIR, "csrc", "ptx_sm100.cuh"),
    os.path.join(PKG_DIR, "csrc", "config_table.inc"),
    os.path.join(PKG_DIR, "csrc", "slab_driver.inc"),
    os.path.join(ROOT_DIR, "include", "b200_gemm.h"),
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-diag-suppress", "177",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build " + LIB_NAME)
    return exe


def is_stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(d) > t for d in DEPENDS if os.path.exists(d))


def _compile(out: str, extra: list, verbose: bool) -> str:
    cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-o", out] + SOURCES + ["-ldl"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    return _compile(LIB_PATH, [], verbose)


def build_timeline(force: bool = False, verbose: bool = False) -> str:
    """Compile the timeline (profiling) variant of the library; returns its path."""
    if not force and not is_stale(TIMELINE_LIB_PATH):
        return TIMELINE_LIB_PATH
    return _compile(TIMELINE_LIB_PATH, ["-DB200_GEMM_TIMELINE"], verbose)


if __name__ == "__main__":
    if "--timeline" in sys.argv:
        print(build_timeline(force="--force" in sys.argv, verbose="-v" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
