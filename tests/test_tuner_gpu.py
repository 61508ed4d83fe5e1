"""The tuner on the GPU: a two-size, small-budget run of config/tune.py must leave a valid JSON
table in the reference's schema, race.py must be able to time it, and the `tuner` binary (the
reference's process-per-evaluation flow, config/tuner.cpp) must print a time for one config."""
import json
import os
import re
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = os.path.join(ROOT, "rocm_wmma_gemm_b200", "config")


def test_tune_two_sizes_small_budget(tmp_path, gemm_lib):
    out = tmp_path / "table.json"
    proc = subprocess.run([sys.executable, os.path.join(CFG, "tune.py"), "--sizes", "512,512,512", "256,1024,2048",
                           "--layouts", "r,c,r", "c,r,c", "--budget", "6", "--budget-seeded", "4", "--type", "f32_bf16",
                           "--output", str(out)], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    table = json.load(open(out))["configurations"]
    assert len(table) == 4
    from rocm_wmma_gemm_b200.config import tune
    for e in table:
        assert set(e["config"]) == {"tile_m", "tile_n", "stages", "cluster", "split_k", "raster"}
        assert set(e["range"]) == {"M", "N", "K"} and set(e["layout"]) == {"A", "B", "C"}
        assert e["time_ms"] > 0
        c = e["config"]
        assert tune.check_constraints((c["tile_m"], c["tile_n"], c["stages"], c["split_k"], c["raster"]))
    race = subprocess.run([sys.executable, os.path.join(CFG, "race.py"), str(out), "--type", "f32_bf16", "--rounds", "2", "--cross"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert race.returncode == 0, race.stdout[-3000:] + race.stderr[-3000:]


def test_tuner_binary_prints_a_time(tmp_path, gemm_lib):
    if shutil.which("g++") is None:
        pytest.skip("no host C++ compiler on this machine")
    pkg = os.path.join(ROOT, "rocm_wmma_gemm_b200")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    binary = str(tmp_path / "tuner")
    built = subprocess.run(["g++", "-O2", "-std=c++17", f"-I{ROOT}/include", f"-I{cuda}/include", os.path.join(CFG, "tuner.cpp"),
                            "-o", binary, f"-L{pkg}", "-lrocm_wmma_gemm_sm100a", f"-Wl,-rpath,{pkg}", f"-L{cuda}/lib64",
                            "-lcudart", "-ldl", "-lpthread"], capture_output=True, text=True, timeout=300)
    assert built.returncode == 0, built.stdout + built.stderr
    proc = subprocess.run([binary, "1024", "1024", "1024", "128", "128", "4", "1", "1", "0", "0", "1", "0", "sm_100a", "f32_bf16"],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert re.search(r"[0-9.]+", proc.stdout), proc.stdout
