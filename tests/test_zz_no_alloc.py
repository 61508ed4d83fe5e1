"""GPU test of `b200_gemm_splitk_static`, the GEMM entry point for callers that are not
allowed to allocate device memory while they run (a server with a fixed memory plan, a
latency-critical thread, a plugin inside a framework that owns the allocator).  Its split-K
partials live in a workspace built into the library instead of an allocated one, so its
results must be identical to the allocating entry point's — on the first call and again on a
second call that finds the first call's leftovers in the workspace.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  Works alone in a fresh process as well as after the rest of the suite."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import rocm_wmma_gemm_b200 as g
from gpu_util import check_parity

pytestmark = pytest.mark.gpu


def _device(bits):
    return torch.from_numpy(bits.view(np.int16)).cuda()


def _both(L, types, A, B, M, N, K, lc, la, lb, cfg):
    out_dt = torch.float32 if types in (1, 3) else torch.int16
    dA, dB = _device(A), _device(B)
    C_ref = torch.full((M * N,), -1, dtype=out_dt, device="cuda")
    C_new = torch.full((M * N,), -1, dtype=out_dt, device="cuda")
    L.gemm(C_ref, dA, dB, M, N, K, lc, la, lb, types=types, config=cfg)       # existing, allocating
    L.gemm_static(C_new, dA, dB, M, N, K, lc, la, lb, types=types, config=cfg)  # new, allocation-free
    torch.cuda.synchronize()
    return C_ref.cpu().numpy(), C_new.cpu().numpy()


@pytest.mark.parametrize("types", range(4), ids=["f16_f16", "f32_f16", "bf16_bf16", "f32_bf16"])
def test_static_workspace_matches_allocating_entry_point_twice(types):
    L = g.loader()
    bf16 = types >= 2
    cfg = g.GemmConfig(128, 128, 4, 1, 4, 0)  # four K partitions -> scratch is used
    # Call 1, then call 2 with a different shape, layout and data: the workspace still holds
    # call 1's partials when call 2 starts.
    cases = [(64, 1024, 4096, 0, 0, 1), (128, 768, 2048 + 64, 1, 1, 0)]
    for call, (M, N, K, lc, la, lb) in enumerate(cases):
        A = oracle.init_matrix(M, K, la, bf16)
        B = oracle.init_matrix(K, N, lb, bf16)
        if call == 1:
            A = A[::-1].copy()
        want, got = _both(L, types, A, B, M, N, K, lc, la, lb, cfg)
        # Same arithmetic, but the two entry points may walk K in a different order, so the
        # comparison uses the parity tests' own per-element tolerance (tests/gpu_util.py).
        as_np = (lambda x: x) if types in (1, 3) else (lambda x: x.view(np.uint16))
        check_parity(types, as_np(got), as_np(want), K, 1.0 / 3.0, M, N, lc)
        ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
        gf = got if types in (1, 3) else oracle.bits_to_f32(got.view(np.uint16), bf16)
        rf = ref if types in (1, 3) else oracle.bits_to_f32(ref, bf16)
        rel = np.sqrt(((gf.astype(np.float64) - rf) ** 2).sum()) / np.sqrt((rf.astype(np.float64) ** 2).sum())
        assert rel <= 1e-3, f"call {call + 1}: relative Frobenius error {rel} against the CPU reference"
    assert g.device_status() == 0


def test_static_entry_point_without_split_and_table_config():
    L = g.loader()
    M, N, K = 256, 512, 256
    A, B = oracle.init_matrix(M, K, 0, True), oracle.init_matrix(K, N, 1, True)
    want, got = _both(L, 3, A, B, M, N, K, 0, 0, 1, None)  # cfg NULL: the tuned table decides
    check_parity(3, got, want, K, 1.0 / 3.0, M, N, 0)


def test_static_entry_point_rejects_what_does_not_fit():
    L = g.loader()
    lib = g.lib()
    a = torch.zeros(4096 * 256, dtype=torch.float16, device="cuda")
    c = torch.zeros(4096 * 4096, dtype=torch.float32, device="cuda")
    cfg = g.GemmConfig(128, 128, 4, 1, 2, 0)
    # 2 partitions x 4096 x 4096 x 4 bytes = 128 MiB of partials: beyond the 16 MiB built in
    with pytest.raises(g.GemmError) as err:
        L.gemm_static(c, a, a, 4096, 4096, 256, 0, 0, 1, config=cfg)
    assert err.value.status == 9 and "workspace" in str(err.value)
    assert (c == 0).all()  # nothing ran
    # a shape the tensor-copy engine cannot address is refused, not sent to another path
    with pytest.raises(g.GemmError) as err:
        L.gemm_static(c, a, a, 17, 33, 9, 0, 0, 1)
    assert err.value.status == 4
    with pytest.raises(g.GemmError) as err:
        L.gemm_static(c, a, a, 16, 16, 0, 0, 0, 1)
    assert err.value.status == 3
    assert lib.b200_gemm_last_status() == 3
