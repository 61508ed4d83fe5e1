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
    cfg = g.GemmConfig(128, 128, 4, 1, 4, 0)  # four K partitions: scratch is used by call 1 (operand swap); call 2 sums them inside clusters
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
    assert g.static_status() == 0  # the entry point's own device status word, not the allocating path's
    assert g.device_status() == 0


@pytest.mark.parametrize("cfg,shape", [
    (g.GemmConfig(256, 128, 4, 2, 4, 2), (512, 384, 2048 + 64, 0, 0, 0)),   # CTA pair + four K partitions
    (g.GemmConfig(256, 512, 4, 2, 2, 0), (512, 1024, 1024, 0, 0, 1)),       # 512-wide pair tile, two partitions
    (None, (16, 4096, 2048, 0, 0, 1)),                                      # skinny: operand swap, transposing epilogue
    (g.GemmConfig(128, 128, 4, 1, 3, 0), (48, 2048, 1024, 0, 0, 0)),        # skinny with K partitions
], ids=["pair-split4", "pair512-split2", "skinny-table", "skinny-split3"])
def test_static_entry_point_shares_the_launch_rules(cfg, shape):
    """The allocation-free entry point plans and launches exactly like the allocating one (CTA
    pairs, 512-wide tiles, the operand swap of skinny problems), so their results are bit-equal."""
    M, N, K, lc, la, lb = shape
    L = g.loader()
    A, B = oracle.init_matrix(M, K, la, True), oracle.init_matrix(K, N, lb, True)
    want, got = _both(L, 3, A, B, M, N, K, lc, la, lb, cfg)
    assert np.array_equal(want.view(np.uint32), got.view(np.uint32))
    ref = oracle.hgemm(3, A, B, M, N, K, lc, la, lb)
    check_parity(3, got, ref, K, 1.0 / 3.0, M, N, lc)
    assert g.static_status() == 0


def test_static_entry_point_allocates_nothing():
    """The defining property: once the first call on the device has done its set-up, free device
    memory is the same before and after any number of calls (the driver reports it per device,
    so any cudaMalloc, stream-ordered allocation or growth of a cached buffer would show)."""
    L = g.loader()
    M, N, K = 128, 1024, 4096
    A, B = _device(oracle.init_matrix(M, K, 0, False)), _device(oracle.init_matrix(K, N, 1, False))
    C = torch.empty(M * N, dtype=torch.float32, device="cuda")

    def calls():
        for split in (8, 2, 5, 1):
            cfg = g.GemmConfig(128, 128, 4, 1, split, 0)
            L.gemm_static(C, A, B, M, N, K, 0, 0, 1, types=1, config=cfg)
            L.gemm_static(C[: 16 * N], A, B, 16, N, K, 0, 0, 1, types=1)
        torch.cuda.synchronize()

    calls()  # first calls: the entry point's set-up, and the driver loads each kernel it meets
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        calls()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free device memory changed by {free0 - free1} bytes"
    assert g.static_status() == 0


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
