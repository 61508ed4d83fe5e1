"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every symbol
include/b200_gemm.h declares, validates arguments like the header says, and never computes
on the CPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_gemm.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([a-z][a-z0-9_]*)\s*\(", text)
    return sorted({n for n in names if n.startswith(("b200_gemm_", "rocm_wmma_gemm_"))})


def test_header_declares_the_reference_symbols():
    names = declared_functions()
    for suffix in ("f16_f16", "f32_f16", "bf16_bf16", "f32_bf16"):
        assert f"rocm_wmma_gemm_{suffix}" in names
        assert f"b200_gemm_{suffix}" in names


def test_library_exports_every_declared_symbol(gemm_lib):
    lib = gemm_lib.lib()
    names = declared_functions()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200_gemm.h but not exported"
        assert n in gemm_lib.ABI_SYMBOLS, f"{n} has no ctypes signature"
    assert set(gemm_lib.ABI_SYMBOLS) == set(names)


def test_no_oracle_or_cpu_path_in_the_product():
    """The product sources never reference the oracle."""
    pkg = os.path.join(ROOT, "rocm_wmma_gemm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h", ".inc")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)


def _call(g, name, *args):
    return getattr(g.lib(), name)(*args)


def test_argument_validation_needs_no_device(gemm_lib):
    g = gemm_lib
    lib = g.lib()
    p = 0x1000  # never dereferenced: validation fails first
    assert lib.b200_gemm_f32_f16(p, p, p, 128, 128, 128, 1, 2, 0, 0, None) == 1  # bad layout
    assert b"layout" in lib.b200_gemm_last_error()
    assert lib.b200_gemm_f32_f16(p, p, p, 128, 128, 128, 1, 0, -1, 0, None) == 1
    assert lib.b200_gemm_f32_f16(None, p, p, 128, 128, 128, 1, 0, 0, 0, None) == 2  # NULL C
    assert lib.b200_gemm_f16_f16(p, None, p, 128, 128, 128, 1, 0, 0, 0, None) == 2
    assert lib.b200_gemm_f32_f16(p, p, p, 128, 128, 128, 0, 0, 0, 0, None) == 3  # batch 0
    assert lib.b200_gemm_f32_f16(p, p, p, 2 ** 31, 128, 128, 1, 0, 0, 0, None) == 3
    assert lib.b200_gemm_f32_f16(p + 2, p, p, 128, 128, 128, 1, 0, 0, 0, None) == 4  # f32 C at 2 mod 4
    assert lib.b200_gemm_bf16_bf16(p, p + 1, p, 128, 128, 128, 1, 0, 0, 0, None) == 4
    # Empty C: nothing to do, succeeds anywhere.
    assert lib.b200_gemm_f32_f16(None, None, None, 0, 128, 128, 1, 0, 0, 0, None) == 0
    assert lib.b200_gemm_f32_f16(None, None, None, 128, 0, 128, 1, 1, 1, 1, None) == 0
    # The void reference symbols record instead of returning.
    lib.rocm_wmma_gemm_f32_bf16(p, p, p, 128, 128, 128, 1, 7, 0, 0, None)
    assert lib.b200_gemm_last_status() == 1
    lib.rocm_wmma_gemm_f32_bf16(None, None, None, 0, 0, 0, 1, 0, 0, 0, None)
    assert lib.b200_gemm_last_status() == 0
    assert lib.b200_gemm_ex(9, p, p, p, 8, 8, 8, 1, 0, 0, 0, None, None) == 7  # unknown type pair


def test_no_cpu_fallback(gemm_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; this checks the GPU-less behaviour")
    lib = gemm_lib.lib()
    buf = (ctypes.c_float * (128 * 128))()
    p = ctypes.addressof(buf)
    assert lib.b200_gemm_f32_f16(p, p, p, 128, 128, 128, 1, 0, 0, 0, None) == 5  # B200_GEMM_ERR_NO_DEVICE
    assert lib.b200_gemm_host(1, p, p, p, 128, 128, 128, 1, 0, 0, 0) == 5
    with pytest.raises(gemm_lib.GemmError):
        gemm_lib.loader().gemm(p, p, p, 128, 128, 128, types=("f32", "f16"))


def test_slab_partition(gemm_lib):
    g = gemm_lib
    for n in (16384, 32768, 8192, 1000, 255, 1):
        for world in (1, 2, 3, 4, 8):
            for align in (1, 64, 256):
                covered = 0
                for r in range(world):
                    b, c = g.slab(n, world, r, align)
                    assert b == covered or c == 0
                    if r < world - 1 and b + c < n:
                        assert c % align == 0
                    covered = b + c if c else covered
                assert covered == n
    assert g.slab(16384, 8, 3, 256) == (6144, 2048)
    with pytest.raises(g.GemmError):
        g.slab(100, 4, 4)


def test_explicit_config_is_validated(gemm_lib):
    g = gemm_lib
    lib = g.lib()
    p = 0x1000
    bad = [g.GemmConfig(128, 96, 4, 1, 1, 8), g.GemmConfig(256, 256, 4, 1, 1, 8), g.GemmConfig(128, 256, 4, 2, 1, 8),
           g.GemmConfig(256, 64, 4, 2, 1, 8), g.GemmConfig(128, 128, 1, 1, 1, 8), g.GemmConfig(128, 128, 4, 1, 0, 8),
           g.GemmConfig(128, 128, 4, 3, 1, 8)]
    import torch
    if torch.cuda.is_available():
        pytest.skip("explicit-config validation on a GPU is covered by the parity tests")
    for cfg in bad:  # without a device the call stops at NO_DEVICE before config checks
        assert lib.b200_gemm_ex(1, p, p, p, 128, 128, 128, 1, 0, 0, 0, None, ctypes.byref(cfg)) in (5, 7)


def test_version_and_counters(gemm_lib):
    assert b"sm_100a" in gemm_lib.lib().b200_gemm_version()
    assert gemm_lib.launch_count() >= 0


def test_launch_plan_rules():
    """b200_gemm_plan is host code: the launch rules can be checked without a GPU (148 SMs given)."""
    import rocm_wmma_gemm_b200 as g
    # skinny, large operand K-major: operands swapped, 147 slabs of 56 rows, K not partitioned,
    # four k-blocks per ring slot
    p = g.plan(16, 8192, 8192, 0, 0, 1, types=1, sm_count=148)
    assert (p.kernel, p.tile_m, p.tile_n, p.split_k, p.k_blocks_per_slot, p.ctas) == (3, 56, 16, 1, 4, 147)
    assert p.slots >= 3
    # two waves of 104-row slabs
    p = g.plan(16, 28672, 8192, 0, 0, 1, types=1, sm_count=148)
    assert (p.kernel, p.tile_m, p.split_k, p.work_units, p.ctas) == (3, 104, 1, 276, 148)
    # large operand M-major (B row-major): slabs are whole 64-row boxes
    p = g.plan(16, 8192, 8192, 0, 0, 0, types=1, sm_count=148)
    assert p.kernel == 3 and p.tile_m in (64, 128)
    # K not a multiple of 64: one k-block per slot (plain 3-D maps)
    assert g.plan(16, 8192, 8200, 0, 0, 1, types=1, sm_count=148).k_blocks_per_slot == 1
    # column-major C of a skinny problem: the narrow staged-epilogue variant, no operand swap,
    # slabs in whole 32-row store groups (128 slabs of 64 rows, K not partitioned)
    p = g.plan(16, 8192, 8192, 1, 0, 1, types=1, sm_count=148)
    assert (p.kernel, p.tile_m, p.tile_n, p.cluster, p.split_k, p.ctas) == (2, 64, 16, 1, 1, 128)
    # the headline size runs on CTA pairs, one k-block per slot, every SM busy
    p = g.plan(8192, 8192, 8192, 0, 0, 1, types=3, sm_count=148)
    assert (p.kernel, p.cluster, p.tile_m, p.k_blocks_per_slot, p.ctas) == (2, 2, 256, 1, 148) and p.tile_n in (256, 512)
    # a size without a table entry that the nearest entry would under-fill: smaller tile and/or K partitions
    p = g.plan(512, 512, 4096, 0, 0, 1, types=2, sm_count=148)
    assert p.kernel == 2 and p.ctas >= 74
    # leading dimensions TMA cannot address -> the CUDA-core kernel; empty problems launch nothing
    assert g.plan(100, 100, 100, sm_count=148).kernel == 1
    assert g.plan(0, 100, 100, sm_count=148).kernel == 0
    # the workspace query agrees with the plan
    lib = g.lib()
    for (m, n, k, t) in [(16, 8192, 8192, 1), (128, 8192, 8192, 1), (512, 512, 4096, 2), (8192, 8192, 8192, 3)]:
        p = g.plan(m, n, k, 0, 0, 1, types=t)
        if p.split_k == 0:  # balanced schedule: at most two partial tiles per run
            upt = -(-(-(-k // 64)) // p.k_blocks_per_slot)
            workers = min(p.work_units * upt, 148 // p.cluster)
            want = 2 * workers * p.tile_m * p.tile_n * 4
        else:
            want = p.split_k * m * n * 4 if p.split_k > 1 and not p.cluster_k else 0
        assert lib.b200_gemm_workspace_bytes(t, m, n, k, 1, 0, 0, 1, None) == want
    # an explicit balanced configuration (split_k 0): 32 tiles of 128 x 256, 148 runs
    import ctypes
    cfg = g.GemmConfig(128, 256, 4, 1, 0, 0)
    assert lib.b200_gemm_workspace_bytes(1, 128, 8192, 8192, 1, 0, 0, 1, ctypes.byref(cfg)) == 2 * 148 * 128 * 256 * 4
    cfg = g.GemmConfig(256, 512, 4, 2, 0, 0)  # no balanced form of the 512-wide tile
    assert lib.b200_gemm_workspace_bytes(3, 8192, 8192, 8192, 1, 0, 0, 1, ctypes.byref(cfg)) == 0
