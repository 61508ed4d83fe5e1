"""CPU tests of the oracle: the C restatement against (a) the committed golden fixtures the
reference's own code produced, (b) the compiled reference itself when it is present, and
(c) independent float16 / bfloat16 conversions."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ["f16_f16", "f32_f16", "bf16_bf16", "f32_bf16"]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def test_f16_to_f32_all_patterns():
    lib = oracle.oracle_lib()
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([lib.oracle_f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
    assert np.isnan(got[np.isnan(want)]).all()


def test_f32_to_f16_round_to_nearest_even():
    lib = oracle.oracle_lib()
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.uniform(-1, 1, 4000), rng.uniform(-70000, 70000, 2000), rng.normal(0, 1e-5, 2000),
        rng.normal(0, 1e-7, 1000), [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25,
                                    2.0 ** -25 * 1.0001, 2.0 ** -14, 6.1e-5, np.inf, -np.inf],
        # exact ties between neighbouring halves
        (np.arange(1024, 1100, dtype=np.float64) + 0.5) / 1024.0,
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_bf16_conversions():
    torch = pytest.importorskip("torch")
    lib = oracle.oracle_lib()
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.uniform(-1, 1, 3000), rng.normal(0, 100, 1000), [0.0, -0.0, 1.0, 3.3895314e38],
                           # ties: low 16 bits exactly 0x8000
                           np.array([0x3F808000, 0x3F818000, 0xBF808000, 0x40008000], dtype=np.uint32).view(np.float32)
                           ]).astype(np.float32)
    want = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got = np.array([lib.oracle_f32_to_bf16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)
    back = np.array([lib.oracle_bf16_to_f32(int(b)) for b in got], dtype=np.float32)
    assert np.array_equal(back.view(np.uint32), got.astype(np.uint32) << 16)


def test_init_matrix_matches_golden():
    g = np.load(os.path.join(GOLDEN, "init_matrix.npz"))
    for key in g.files:
        r, c, l, bf = [int(x[1:] if x[0] != "b" else x[2:]) for x in key.split("_")]
        got = oracle.init_matrix(r, c, l, bool(bf))
        assert np.array_equal(got, g[key]), key


def test_init_matrix_is_layout_independent_in_logical_order():
    a = oracle.init_matrix(9, 13, 0, False).reshape(9, 13)
    b = oracle.init_matrix(9, 13, 1, False).reshape(13, 9).T
    assert np.array_equal(a, b)
    # A and B start from the same stream (the generator is re-seeded per call).
    assert np.array_equal(oracle.init_matrix(4, 4, 0, False)[:4], oracle.init_matrix(8, 4, 0, False)[:4])


def test_hgemm_small_matches_golden():
    g = np.load(os.path.join(GOLDEN, "hgemm_small.npz"))
    M, N, K = 16, 24, 32
    assert len(g.files) == 32
    for types in range(4):
        bf16 = types >= 2
        for key in range(8):
            lc, la, lb = key >> 2, (key >> 1) & 1, key & 1
            A = oracle.init_matrix(M, K, la, bf16)
            B = oracle.init_matrix(K, N, lb, bf16)
            C = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            want = g[f"t{types}_c{lc}_a{la}_b{lb}"]
            assert C.dtype == want.dtype
            assert np.array_equal(C.view(np.uint8), want.view(np.uint8)), (types, lc, la, lb)


def test_config1_known_answers():
    """fp16 A/B, M=N=K=256, A row / B col / C row: values the reference's hgemm_cpu gives."""
    with open(os.path.join(GOLDEN, "config1.json")) as f:
        kat = json.load(f)
    for types, name in enumerate(NAMES):
        bf16 = types >= 2
        A = oracle.init_matrix(256, 256, 0, bf16)
        B = oracle.init_matrix(256, 256, 1, bf16)
        k = kat["types"][name]
        assert sha(A) == k["sha256_A"] and sha(B) == k["sha256_B"]
        C = oracle.hgemm(types, A, B, 256, 256, 256, 0, 0, 1)
        assert sha(C) == k["sha256_C"], name
    # the fp16 -> f32 headline values, as decimal
    A = oracle.init_matrix(256, 256, 0, False)
    B = oracle.init_matrix(256, 256, 1, False)
    C = oracle.hgemm(1, A, B, 256, 256, 256, 0, 0, 1)
    assert abs(oracle.bits_to_f32(A[:1], False)[0] - (-0.166016)) < 1e-6
    assert abs(C[0] - (-4.48529482)) < 1e-6 and abs(C[-1] - (-0.209937096)) < 1e-7
    assert abs(np.sqrt((C.astype(np.float64) ** 2).sum()) - 1361.53624) < 1e-3


def test_threads_and_row_selection_do_not_change_results():
    M, N, K = 37, 29, 48
    A = oracle.init_matrix(M, K, 1, True)
    B = oracle.init_matrix(K, N, 0, True)
    full = oracle.hgemm(3, A, B, M, N, K, 0, 1, 0, threads=1)
    assert np.array_equal(full, oracle.hgemm(3, A, B, M, N, K, 0, 1, 0, threads=5))
    rows, cols = [0, 5, 36], [1, 28]
    part = oracle.hgemm_select(3, A, B, M, N, K, 0, 1, 0, rows=rows, cols=cols).reshape(M, N)
    assert np.array_equal(part[np.ix_(rows, cols)], full.reshape(M, N)[np.ix_(rows, cols)])
    assert np.isnan(part[1, 1]) and np.isnan(part[0, 0])


def test_cosine_similarity_edge_cases():
    a = np.zeros(12, dtype=np.float32)
    assert oracle.cosine_similarity(a, a, 3, 4, 0, 1) == 1.0
    b = a.copy()
    b[3] = 1.0
    assert oracle.cosine_similarity(a, b, 3, 4, 0, 1) == 0.0
    c = np.arange(1, 13, dtype=np.float32)
    assert abs(oracle.cosine_similarity(c, c, 3, 4, 1, 1) - 1.0) < 1e-6


# ---- against the compiled reference itself (present where a reference checkout is) ----------

needs_ref = pytest.mark.skipif(oracle.ref_lib() is None, reason="compiled reference (oracle/_ref) not available")


@needs_ref
@pytest.mark.parametrize("types", range(4))
def test_restatement_is_bit_exact_against_reference(types):
    bf16 = types >= 2
    for (M, N, K) in [(24, 40, 56), (1, 1, 1), (7, 3, 5), (64, 64, 64)]:
        for key in range(8):
            lc, la, lb = key >> 2, (key >> 1) & 1, key & 1
            A = oracle.init_matrix(M, K, la, bf16)
            B = oracle.init_matrix(K, N, lb, bf16)
            assert np.array_equal(A, oracle.init_matrix(M, K, la, bf16, impl="ref"))
            C = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            R = oracle.hgemm(types, A, B, M, N, K, lc, la, lb, impl="ref")
            assert np.array_equal(C.view(np.uint8), R.view(np.uint8)), (M, N, K, lc, la, lb)
            kind = 1 if types in (1, 3) else (2 if bf16 else 0)
            noisy = C.copy()
            noisy[::3] = noisy[::5][: noisy[::3].size] if noisy[::5].size >= noisy[::3].size else noisy[::3]
            assert oracle.cosine_similarity(noisy, C, M, N, lc, kind) == oracle.cosine_similarity(noisy, C, M, N, lc, kind, impl="ref")


@needs_ref
def test_reference_row_panel_threads_match_whole_gemm():
    M, N, K = 40, 24, 32
    A = oracle.init_matrix(M, K, 0, True)
    B = oracle.init_matrix(K, N, 1, True)
    full = oracle.hgemm(3, A, B, M, N, K, 0, 0, 1, impl="ref").reshape(M, N)
    out = np.zeros(20 * N, dtype=np.float32)
    oracle.ref_lib().ref_hgemm_rows_mt(3, out.ctypes.data, A.ctypes.data, B.ctypes.data, M, N, K, 0, 0, 1, 10, 30, 4)
    assert np.array_equal(out.reshape(20, N), full[10:30])
