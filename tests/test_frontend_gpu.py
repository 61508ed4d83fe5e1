"""The C++ front end on the GPU: `rocm_wmma_gemm::loader` (dlopen of the library, the four C
symbols) and the header-inline `rocm_wmma_gemm::gemm<>` of include/rocm_wmma_gemm/*.hpp, driven
the way the reference's typed tests drive them (test/gemm/test_float_accum.cpp:80-142):
tests/cpp/test_frontend.cpp is compiled here with g++ against include/ and run."""
import os
import re
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")


def _run(binary):
    pkg = os.path.join(ROOT, "rocm_wmma_gemm_b200")  # the loader dlopen()s librocm_wmma_gemm_sm100a.so by name
    env = dict(os.environ, LD_LIBRARY_PATH=pkg + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
    return subprocess.run([binary], capture_output=True, text=True, timeout=900, env=env)


def test_cpp_front_end(gemm_lib):
    if shutil.which("g++") is None or shutil.which("gcc") is None:
        pytest.skip("no host C++ compiler on this machine")
    built = subprocess.run(["sh", os.path.join(CPP, "build.sh")], capture_output=True, text=True, timeout=600)
    assert built.returncode == 0, built.stdout + built.stderr
    proc = _run(os.path.join(CPP, "test_frontend"))
    assert proc.returncode == 0, proc.stdout[-4000:] + proc.stderr[-2000:]
    m = re.search(r"(\d+) cases, (\d+) failed", proc.stdout)
    # 4 type pairs x 8 layouts x 5 shapes x 2 front ends + 3 batches + 2 behaviour checks
    assert m and int(m.group(1)) == 4 * 8 * 5 * 2 + 3 + 2 and int(m.group(2)) == 0, proc.stdout[-2000:]


@pytest.mark.parametrize("name", ["float_accum", "same_prec"])
def test_reference_typed_tests_compiled_against_this_front_end(name):
    """The reference's own test/gemm/test_float_accum.cpp (f32 outputs, 1e-4 per element) and
    test/gemm/test_same_prec.cpp (f16 / bf16 outputs, cosine similarity), compiled unmodified
    against include/ (tests/cpp/build_reference_test.sh, run where a reference checkout exists;
    the binaries travel with the tree) with a minimal stand-in for the test framework they
    include: 16 type x layout instantiations x 13 sizes each."""
    binary = os.path.join(CPP, f"test_reference_{name}")
    if not os.path.exists(binary):
        pytest.skip(f"tests/cpp/test_reference_{name} has not been built (needs a reference checkout)")
    proc = _run(binary)
    assert proc.returncode == 0, proc.stdout[-4000:] + proc.stderr[-2000:]
    m = re.search(r"(\d+) tests ran, (\d+) failed", proc.stdout)
    assert m and int(m.group(1)) == 16 * 13 and int(m.group(2)) == 0, proc.stdout[-2000:]
