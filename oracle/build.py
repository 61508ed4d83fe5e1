"""Builds the oracle's two libraries (test infrastructure, never loaded by the GEMM library).

  oracle/liboracle_gemm.so      plain-C restatement (cpu_gemm.c), gcc
  oracle/_ref/libref_hgemm.so   the reference's own test/test.hpp compiled unmodified through
                                ref_shim.cpp, g++; only when a reference checkout is present
                                (its sources are used where they lie, nothing is copied)

Both are built without -march flags and with -ffp-contract=off so multiply and add stay
separate binary32 operations, which is what the reference's host build computes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(HERE, "liboracle_gemm.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_LIB = os.path.join(REF_DIR, "libref_hgemm.so")
# The reference checkout: $ROCM_WMMA_GEMM_REFERENCE, else a directory `reference` beside this repository.
REFERENCE_ROOT = os.environ.get("ROCM_WMMA_GEMM_REFERENCE",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
CUDA_INCLUDE = os.environ.get("CUDA_INCLUDE", "/usr/local/cuda/include")


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "cpu_gemm.c")
    if force or _stale(ORACLE_LIB, [src]):
        _run([shutil.which("gcc") or "gcc", "-O2", "-ffp-contract=off", "-std=c11", "-shared", "-fPIC",
              "-o", ORACLE_LIB, src, "-lm", "-lpthread"])
    return ORACLE_LIB


def reference_available() -> bool:
    return os.path.exists(os.path.join(REFERENCE_ROOT, "test", "test.hpp"))


def build_ref(force: bool = False):
    """Compiles the reference's CPU path if its checkout is present; returns the library path,
    the existing prebuilt library when the checkout is absent, or None."""
    src = os.path.join(HERE, "ref_shim.cpp")
    if not reference_available():
        return REF_LIB if os.path.exists(REF_LIB) else None
    deps = [src, os.path.join(REFERENCE_ROOT, "test", "test.hpp"),
            os.path.join(REFERENCE_ROOT, "common", "matrix.hpp")]
    if force or _stale(REF_LIB, deps):
        os.makedirs(REF_DIR, exist_ok=True)
        _run([shutil.which("g++") or "g++", "-std=c++20", "-O2", "-ffp-contract=off", "-shared", "-fPIC",
              "-I" + CUDA_INCLUDE, "-I" + REFERENCE_ROOT, "-I" + os.path.join(REFERENCE_ROOT, "test"),
              "-o", REF_LIB, src, "-lpthread"])
    return REF_LIB


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
