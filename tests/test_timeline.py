"""The timeline (profiling) variant of the library: same sources with -DB200_GEMM_TIMELINE."""
import ctypes
import os

import numpy as np
import pytest

from rocm_wmma_gemm_b200 import build as lib_build


def test_timeline_variant_exports_its_readers_and_the_default_build_does_not():
    if not os.path.exists(lib_build.TIMELINE_LIB_PATH):
        pytest.skip("timeline variant not built (python -m rocm_wmma_gemm_b200.build --timeline)")
    tl = ctypes.CDLL(lib_build.TIMELINE_LIB_PATH, mode=ctypes.RTLD_LOCAL)
    for name in ("b200_gemm_debug_timeline", "b200_gemm_debug_cta_times", "b200_gemm_debug_reset", "b200_gemm_ex"):
        assert hasattr(tl, name)
    main = ctypes.CDLL(lib_build.LIB_PATH, mode=ctypes.RTLD_LOCAL)
    assert not hasattr(main, "b200_gemm_debug_timeline")


@pytest.mark.gpu
def test_timeline_stamps_are_in_program_order():
    from rocm_wmma_gemm_b200 import timeline
    lib = timeline.load()
    r = timeline.run(lib, "bf16_bf16", 512, 512, 512, launches=8)
    c = r["cycles_after_wait"]
    # entry, set-up, wait (= 0), first / last TMA, first full, last commit, drained, seen, first / last store, read, tail, freed
    assert c[0] < c[1] and c[2] == 0
    assert 0 < c[3] < c[5] < c[6] < c[8] < c[9] <= c[10] < c[11] < c[13]
    assert c[3] <= c[4] and c[6] <= c[7]
    assert 0 < r["entry_to_next_entry_ns"] < 1e6 and 0 < r["per_call_us"] < 1e3
    t = r["cta_times"]
    live = t[1] > 0
    import rocm_wmma_gemm_b200 as g
    assert live.sum() == g.plan(512, 512, 512, 0, 0, 1, types=2).ctas   # every CTA of the last launch stamped
    assert np.all(t[0][live] <= t[2][live]) and np.all(t[2][live] <= t[1][live])
