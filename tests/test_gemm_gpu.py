"""GPU parity tests: the sm_100a kernels, called through the C ABI, against the CPU oracle on
the same seeded inputs.  Shapes, layouts and tolerances follow the reference's own tests
(test/gemm/test_float_accum.cpp:149-224, test/gemm/test_same_prec.cpp:138-213)."""
import itertools

import numpy as np
import pytest
import torch

import oracle
import rocm_wmma_gemm_b200 as g
from gpu_util import NAMES, as_f32, check_parity, f32_sum_tolerance, gpu_gemm, loader, to_device

pytestmark = pytest.mark.gpu

# The 13 shapes of the reference's typed tests.
REF_SHAPES = [(128, 128, 128), (128, 256, 128), (128, 128, 256), (256, 128, 128), (256, 256, 256),
              (320, 320, 320), (320, 512, 512), (512, 320, 320), (512, 512, 320), (512, 320, 512),
              (512, 512, 512), (1024, 256, 256), (256, 1024, 256)]
LAYOUTS = list(itertools.product((0, 1), repeat=3))  # (layout_a, layout_b, layout_c)
SIGMA_UNIFORM = 1.0 / 3.0  # std of the product of two uniform[-1,1] values


def seeded(M, N, K, la, lb, bf16):
    return oracle.init_matrix(M, K, la, bf16), oracle.init_matrix(K, N, lb, bf16)


@pytest.mark.parametrize("types", range(4), ids=NAMES)
@pytest.mark.parametrize("la,lb,lc", LAYOUTS, ids=["".join("rc"[x] for x in l) for l in LAYOUTS])
def test_reference_shapes(types, la, lb, lc):
    bf16 = types >= 2
    for (M, N, K) in REF_SHAPES:
        A, B = seeded(M, N, K, la, lb, bf16)
        ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
        got = gpu_gemm(types, A, B, M, N, K, lc, la, lb)
        check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)


def test_config1_known_answer():
    """BASELINE config 1: fp16 -> f32, 256^3, A row / B col / C row, through the void
    reference symbol `rocm_wmma_gemm_f32_f16`."""
    A, B = seeded(256, 256, 256, 0, 1, False)
    got = gpu_gemm(1, A, B, 256, 256, 256, 0, 0, 1, checked=False)
    assert g.lib().b200_gemm_last_status() == 0
    ref = oracle.hgemm(1, A, B, 256, 256, 256, 0, 0, 1)
    rel, mx = check_parity(1, got, ref, 256, SIGMA_UNIFORM, 256, 256, 0)
    assert abs(got[0] - (-4.48529482)) < 1e-4 and abs(got[-1] - (-0.209937096)) < 1e-4
    assert abs(np.sqrt((got.astype(np.float64) ** 2).sum()) - 1361.53624) < 1e-2


CONFIGS = [g.GemmConfig(128, 64, 8, 1, 1, 8), g.GemmConfig(128, 128, 6, 1, 1, 4), g.GemmConfig(128, 256, 4, 1, 1, 0),
           g.GemmConfig(256, 128, 8, 2, 1, 2), g.GemmConfig(256, 256, 6, 2, 1, 16), g.GemmConfig(128, 128, 2, 1, 1, 1),
           g.GemmConfig(256, 256, 3, 2, 1, 1), g.GemmConfig(256, 512, 4, 2, 1, 16), g.GemmConfig(256, 512, 2, 2, 1, 3),
           # snake raster (B200_GEMM_RASTER_SNAKE = 128 added to the band height): column sweep, ragged last band, one-row bands
           g.GemmConfig(128, 64, 8, 1, 1, 128), g.GemmConfig(128, 128, 6, 1, 1, 128 + 2), g.GemmConfig(256, 256, 6, 2, 1, 128 + 1),
           g.GemmConfig(256, 512, 4, 2, 1, 128 + 3)]


@pytest.mark.parametrize("cfg", CONFIGS, ids=[f"m{c.tile_m}n{c.tile_n}s{c.stages}c{c.cluster}r{c.raster}" for c in CONFIGS])
def test_every_compiled_variant_every_layout(cfg):
    """Each tile variant, for all 8 layouts and 4 type pairs, on an aligned and a ragged shape."""
    for types in range(4):
        bf16 = types >= 2
        for (la, lb, lc) in LAYOUTS:
            for (M, N, K) in [(384, 1160, 192), (264, 136, 200)] + ([(904, 1160, 72)] if cfg.raster >= 128 else []):
                A, B = seeded(M, N, K, la, lb, bf16)
                ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
                got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)


RAGGED = [(8, 8, 8), (16, 8, 24), (1, 1, 1), (3, 5, 7), (127, 129, 65), (1000, 1000, 1000), (129, 8, 4096),
          (8, 1032, 72), (250, 250, 16), (17, 33, 9)]


@pytest.mark.parametrize("M,N,K", RAGGED)
def test_ragged_and_tiny_shapes(M, N, K):
    """Edge tiles, K tails and sizes whose rows TMA cannot address (odd leading dimensions go
    through the CUDA-core kernel).  The reference's kernel has no K tail and no load bounds
    checks; this library accepts any size."""
    for types in (1, 2):
        bf16 = types >= 2
        for (la, lb, lc) in [(0, 1, 0), (1, 0, 1), (0, 0, 0), (1, 1, 1)]:
            A, B = seeded(M, N, K, la, lb, bf16)
            ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            got = gpu_gemm(types, A, B, M, N, K, lc, la, lb)
            check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)


def test_empty_inputs():
    l = loader()
    c = torch.full((64,), 7.0, device="cuda")
    a = torch.zeros(64, dtype=torch.float16, device="cuda")
    l.gemm(c, a, a, 0, 8, 8)       # M == 0: no-op
    l.gemm(c, a, a, 8, 0, 8)       # N == 0: no-op
    torch.cuda.synchronize()
    assert (c == 7.0).all()
    l.gemm(c, a, a, 8, 8, 0)       # K == 0: the empty sum, C = 0
    torch.cuda.synchronize()
    assert (c == 0.0).all()


@pytest.mark.parametrize("types", range(4), ids=NAMES)
def test_strided_batched(types):
    """batch_count > 1 with the reference's strides M*K, K*N, M*N (kernel/kernel.hpp:165-167);
    the reference ships no batched test."""
    bf16 = types >= 2
    M, N, K, batch = 192, 320, 256, 5
    for (la, lb, lc) in [(0, 1, 0), (1, 0, 0), (0, 0, 1), (1, 1, 1)]:
        # distinct values per batch: rotate the seeded stream
        A = np.concatenate([oracle.init_matrix(M, K, la, bf16)[(np.arange(M * K) + 97 * b) % (M * K)] for b in range(batch)])
        B = np.concatenate([oracle.init_matrix(K, N, lb, bf16)[(np.arange(K * N) + 31 * b) % (K * N)] for b in range(batch)])
        got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, batch=batch)
        for b in range(batch):
            ref = oracle.hgemm(types, A[b * M * K:(b + 1) * M * K], B[b * K * N:(b + 1) * K * N], M, N, K, lc, la, lb)
            check_parity(types, got[b * M * N:(b + 1) * M * N], ref, K, SIGMA_UNIFORM, M, N, lc)
        # an unaligned batched case goes through the CUDA-core kernel
    A = np.concatenate([oracle.init_matrix(9, 7, 0, bf16)] * 3)
    B = np.concatenate([oracle.init_matrix(7, 5, 1, bf16)] * 3)
    got = gpu_gemm(types, A, B, 9, 5, 7, 0, 0, 1, batch=3)
    ref = oracle.hgemm(types, A[:63], B[:35], 9, 5, 7, 0, 0, 1)
    for b in range(3):
        check_parity(types, got[b * 45:(b + 1) * 45], ref, 7, SIGMA_UNIFORM, 9, 5, 0)


@pytest.mark.parametrize("split_k", [2, 3, 8, 64])
def test_split_k(split_k):
    """K partitions through the f32 workspace + deterministic reduction."""
    M, N, K = 128, 384, 2048 + 64
    for types in range(4):
        bf16 = types >= 2
        for (la, lb, lc), cl in [((0, 1, 0), 1), ((1, 0, 1), 1), ((0, 0, 0), 2)]:
            A, B = seeded(M, N, K, la, lb, bf16)
            ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            cfg = g.GemmConfig(128 * cl, 128, 4, cl, split_k, 8)
            got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
            check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)
            again = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
            assert np.array_equal(got.view(np.uint8), again.view(np.uint8)), "split-K must be deterministic"


BALANCED = [
    # tile_m, tile_n, cluster | M, N, K: tiles x K steps that do not divide by the SM count
    (128, 256, 1, 128, 8192, 2048),    # skinny: 32 tiles cut into 148 runs, 4-5 runs per tile
    (128, 128, 1, 384, 1160, 1280 + 64),  # ragged N and K, two k-blocks per ring slot
    (128, 64, 1, 264, 136, 4096),      # narrow one-CTA tile, four k-blocks per slot
    (256, 256, 2, 2048, 2048, 512),    # CTA pairs: 64 tiles on 74 pairs
    (256, 128, 2, 520, 1000, 1024),    # CTA pairs, ragged everywhere
    (256, 192, 2, 640, 1184, 448),     # run-time tile width (K-major B' layouts only)
    (128, 256, 1, 64, 4096, 8192),     # 64 rows without the operand swap
]


@pytest.mark.parametrize("tile_m,tile_n,cluster,M,N,K", BALANCED, ids=[f"{b[0]}x{b[1]}-{b[3]}x{b[4]}x{b[5]}" for b in BALANCED])
def test_balanced_schedule(tile_m, tile_n, cluster, M, N, K):
    """split_k = 0: the tiles' K loops laid end to end and cut into one equal run per SM
    (stream-K); partial tiles meet in the fix-up pass.  All type pairs and layouts, bit-identical
    from run to run, and the same numbers as the plain schedule up to the order of the f32 sum."""
    for types in range(4):
        bf16 = types >= 2
        for (la, lb, lc) in LAYOUTS:
            cfg = g.GemmConfig(tile_m, tile_n, 4, cluster, 0, 2)
            A, B = seeded(M, N, K, la, lb, bf16)
            flex = tile_n not in (64, 128, 256)
            b_n_major = (lb == 0) if lc == 0 else (la == 1)  # kernel view: is B' N-major?
            chunk = 32 if types in (1, 3) else 64
            if flex and (b_n_major or tile_n % chunk):
                with pytest.raises(g.GemmError):
                    gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                continue
            ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
            check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)
            if (la, lb, lc) in ((0, 1, 0), (1, 0, 1)):
                again = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                assert np.array_equal(got.view(np.uint8), again.view(np.uint8)), "the balanced schedule must be deterministic"


def test_balanced_schedule_batched_and_rejected():
    M, N, K, batch = 192, 320, 1024, 3
    A = np.concatenate([oracle.init_matrix(M, K, 0, True)[(np.arange(M * K) + 97 * b) % (M * K)] for b in range(batch)])
    B = np.concatenate([oracle.init_matrix(K, N, 1, True)[(np.arange(K * N) + 31 * b) % (K * N)] for b in range(batch)])
    got = gpu_gemm(3, A, B, M, N, K, 0, 0, 1, batch=batch, config=g.GemmConfig(128, 128, 4, 1, 0, 0))
    for b in range(batch):
        ref = oracle.hgemm(3, A[b * M * K:(b + 1) * M * K], B[b * K * N:(b + 1) * K * N], M, N, K, 0, 0, 1)
        check_parity(3, got[b * M * N:(b + 1) * M * N], ref, K, SIGMA_UNIFORM, M, N, 0)
    # the 512-wide tile has no balanced form
    with pytest.raises(g.GemmError):
        gpu_gemm(3, A[: M * K], B[: K * N], M, N, K, 0, 0, 1, config=g.GemmConfig(256, 512, 4, 2, 0, 0))


CLUSTER_K = [
    # tile_n, split_k | M, N, K
    (256, 4, 128, 2048, 4096),          # 8 tiles x 4 partitions: the skinny streaming case
    (128, 2, 384, 1160, 1280 + 64),     # ragged N and K, two k-blocks per ring slot
    (256, 3, 200, 1000, 3008),          # three partitions (cluster of 3), ragged rows and columns
    (128, 4, 512, 512, 4096),           # 16 tiles x 4
    (256, 2, 136, 520, 192),            # three k-blocks over two partitions (2 + 1)
]


@pytest.mark.parametrize("tile_n,split,M,N,K", CLUSTER_K, ids=[f"{c[0]}-split{c[1]}-{c[2]}x{c[3]}x{c[4]}" for c in CLUSTER_K])
def test_cluster_k_partitions(tile_n, split, M, N, K):
    """K partitions of a one-CTA tile as the CTAs of one thread-block cluster, summed through
    distributed shared memory (no workspace, no reduction pass): all type pairs and layouts
    against the oracle, bit-identical from run to run, and no workspace asked for."""
    lib = g.lib()
    for types in range(4):
        bf16 = types >= 2
        for (la, lb, lc) in LAYOUTS:
            cfg = g.GemmConfig(128, tile_n, 4, 1, split, 0)
            A, B = seeded(M, N, K, la, lb, bf16)
            ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
            check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)
            if (la, lb, lc) in ((0, 1, 0), (1, 0, 1)):
                import ctypes
                assert lib.b200_gemm_workspace_bytes(types, M, N, K, 1, lc, la, lb, ctypes.byref(cfg)) == 0, "expected the cluster path"
                again = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                assert np.array_equal(got.view(np.uint8), again.view(np.uint8))
    assert g.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(64, 2368, 2048 + 64), (48, 4096, 2048), (64, 1000, 4096), (16, 4096, 4096 + 64), (24, 2048, 8192)])
def test_cluster_k_partitions_transposed(M, N, K):
    """Skinny problems: the operand-swapped slab kernel with two or four K partitions per slab
    as the CTAs of a cluster (two: interleaved K steps; partial slabs summed through
    distributed shared memory, transposing stores).  All type pairs and layouts against the
    oracle; the plan reports the form."""
    p = g.plan(M, N, K, 0, 0, 1, types=1, sm_count=148)
    assert p.kernel == 3 and p.cluster_k == 1 and p.split_k in (2, 3, 4) and p.ctas == p.work_units <= 148
    for types in range(4):
        bf16 = types >= 2
        for (la, lb, lc) in LAYOUTS:
            # the skinny dimension is M for a row-major C and N for a column-major one
            m, n = (M, N) if lc == 0 else (N, M)
            A, B = seeded(m, n, K, la, lb, bf16)
            ref = oracle.hgemm(types, A, B, m, n, K, lc, la, lb)
            got = gpu_gemm(types, A, B, m, n, K, lc, la, lb)
            check_parity(types, got, ref, K, SIGMA_UNIFORM, m, n, lc)
            if (la, lb) == (0, 1):
                again = gpu_gemm(types, A, B, m, n, K, lc, la, lb)
                assert np.array_equal(got.view(np.uint8), again.view(np.uint8))
    assert g.device_status() == 0


def test_cluster_k_partitions_batched_and_table():
    M, N, K, batch = 192, 320, 2048, 3
    A = np.concatenate([oracle.init_matrix(M, K, 0, True)[(np.arange(M * K) + 97 * b) % (M * K)] for b in range(batch)])
    B = np.concatenate([oracle.init_matrix(K, N, 1, True)[(np.arange(K * N) + 31 * b) % (K * N)] for b in range(batch)])
    got = gpu_gemm(2, A, B, M, N, K, 0, 0, 1, batch=batch, config=g.GemmConfig(128, 128, 4, 1, 4, 0))
    for b in range(batch):
        ref = oracle.hgemm(2, A[b * M * K:(b + 1) * M * K], B[b * K * N:(b + 1) * K * N], M, N, K, 0, 0, 1)
        check_parity(2, got[b * M * N:(b + 1) * M * N], ref, K, SIGMA_UNIFORM, M, N, 0)
    # more tiles than clusters fit at once: the persistent kernel with its workspace is used
    import ctypes
    cfg = g.GemmConfig(128, 128, 4, 1, 2, 0)
    assert g.lib().b200_gemm_workspace_bytes(2, 4096, 4096, 256, 1, 0, 0, 1, ctypes.byref(cfg)) == 2 * 4096 * 4096 * 4


def test_all_layouts_agree():
    """The same logical product through all 8 layouts gives the same C (tight tolerance: the
    products are identical, only tile shapes and operand roles differ)."""
    M, N, K = 512, 384, 640
    rng = np.random.default_rng(7)
    A = torch.from_numpy(rng.uniform(-1, 1, (M, K)).astype(np.float32)).to(torch.bfloat16)
    B = torch.from_numpy(rng.uniform(-1, 1, (K, N)).astype(np.float32)).to(torch.bfloat16)
    results = []
    for (la, lb, lc) in LAYOUTS:
        Am = (A if la == 0 else A.t()).contiguous().view(torch.int16).numpy().view(np.uint16).ravel()
        Bm = (B if lb == 0 else B.t()).contiguous().view(torch.int16).numpy().view(np.uint16).ravel()
        C = gpu_gemm(3, Am, Bm, M, N, K, lc, la, lb)
        results.append(C.reshape(M, N) if lc == 0 else C.reshape(N, M).T)
    for r in results[1:]:
        assert np.abs(r - results[0]).max() <= 2e-5


def test_host_buffer_entry_point():
    """b200_gemm_host: host pointers in, host pointers out, copies inside the call."""
    M, N, K = 320, 512, 448
    for types in range(4):
        bf16 = types >= 2
        A, B = seeded(M, N, K, 0, 1, bf16)
        ta, tb = torch.from_numpy(A.view(np.int16)).pin_memory(), torch.from_numpy(B.view(np.int16))
        tc = torch.empty(M * N, dtype=torch.float32 if types in (1, 3) else torch.int16)
        loader().gemm_host(tc, ta, tb, M, N, K, 0, 0, 1, types=types)
        got = tc.numpy() if types in (1, 3) else tc.numpy().view(np.uint16)
        ref = oracle.hgemm(types, A, B, M, N, K, 0, 0, 1)
        check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, 0)


def test_linearity():
    """(A1 + A2) * B == A1*B + A2*B within f32 rounding when the sums are exact in f16
    (small integers), at a size the CPU reference cannot cover quickly."""
    M = N = K = 2048
    gen = torch.Generator(device="cuda").manual_seed(3)
    A1 = torch.randint(-4, 5, (M, K), device="cuda", generator=gen).to(torch.float16)
    A2 = torch.randint(-4, 5, (M, K), device="cuda", generator=gen).to(torch.float16)
    B = torch.randint(-4, 5, (K, N), device="cuda", generator=gen).to(torch.float16)
    l = loader()
    outs = []
    for A in (A1, A2, A1 + A2):
        C = torch.empty(M, N, device="cuda", dtype=torch.float32)
        l.gemm(C, A.contiguous(), B.contiguous(), M, N, K, 0, 0, 0)
        outs.append(C)
    g.device_status()
    # integer-valued products and sums below 2^24 are exact in f32: equality is bit-exact
    assert torch.equal(outs[0] + outs[1], outs[2])


N02 = ("normal", 0.02)
UNI = ("uniform", 1.0)
BIG = (
    # (types, M, N, K, la, lb, lc, distribution, sigma): every benchmarked shape under the config the tuned table
    # gives it.  The headline shape (bf16 -> f32 8192^3) and the fp16 -> fp16 squares in all eight layouts:
    [(3, 8192, 8192, 8192, la, lb, lc, N02, 4e-4) for (la, lb, lc) in LAYOUTS]
    + [(0, n, n, n, la, lb, lc, UNI, 1.0 / 3.0) for n in (1024, 2048, 8192) for (la, lb, lc) in LAYOUTS]
    + [
        (0, 4096, 4096, 4096, 1, 0, 1, UNI, 1.0 / 3.0),   # fp16 -> fp16 square, A col / B row / C col
        (0, 4096, 4096, 4096, 0, 1, 0, UNI, 1.0 / 3.0),
        # projection shapes, bf16 -> f32, A row / B col / C row
        (3, 4096, 4096, 2048, 0, 1, 0, N02, 4e-4),
        (3, 4096, 5120, 5120, 0, 1, 0, N02, 4e-4),
        (3, 8192, 28672, 8192, 0, 1, 0, N02, 4e-4),
        (3, 8192, 8192, 28672, 0, 1, 0, N02, 4e-4),
        # skinny fp16 -> f32, B row- and column-major
        (1, 16, 8192, 8192, 0, 0, 0, UNI, 1.0 / 3.0),
        (1, 16, 28672, 8192, 0, 1, 0, UNI, 1.0 / 3.0),
        (1, 64, 8192, 8192, 0, 0, 0, UNI, 1.0 / 3.0),
        (1, 64, 8192, 8192, 0, 1, 0, UNI, 1.0 / 3.0),
        (1, 64, 28672, 8192, 0, 0, 0, UNI, 1.0 / 3.0),
        (1, 64, 28672, 8192, 0, 1, 0, UNI, 1.0 / 3.0),
        (1, 128, 8192, 8192, 0, 0, 0, UNI, 1.0 / 3.0),
        (1, 128, 8192, 8192, 0, 1, 0, UNI, 1.0 / 3.0),
        (1, 128, 28672, 8192, 0, 1, 0, UNI, 1.0 / 3.0),
        # column slabs of the large bf16 -> bf16 problems (8 GPUs: 16384^3 and 32768 x 32768 x 8192)
        (2, 16384, 2048, 16384, 0, 1, 0, ("normal", 1.0), 1.0),
        (2, 8192, 4096, 16384, 0, 1, 0, ("normal", 1.0), 1.0),
        (2, 32768, 4096, 8192, 0, 1, 0, ("normal", 1.0), 1.0),
    ])


@pytest.mark.parametrize("types,M,N,K,la,lb,lc,dist,sigma", BIG,
                         ids=[f"{NAMES[b[0]]}-{b[1]}x{b[2]}x{b[3]}-{'rc'[b[4]]}{'rc'[b[5]]}{'rc'[b[6]]}" for b in BIG])
def test_full_size_sampled_rows_and_columns(types, M, N, K, la, lb, lc, dist, sigma):
    """Full-size shapes: whole rows and whole columns of C (first/last, tile boundaries, random)
    against the CPU oracle, which computes only the sampled elements."""
    bf16 = types >= 2
    dt = torch.bfloat16 if bf16 else torch.float16
    gen = torch.Generator(device="cuda").manual_seed(M + 3 * N + 7 * K)

    def make(rows, cols):
        if dist[0] == "normal":
            x = torch.randn(rows, cols, device="cuda", generator=gen) * dist[1]
        else:
            x = torch.rand(rows, cols, device="cuda", generator=gen) * 2 - 1
        return x.to(dt)

    A, B = make(M, K), make(K, N)
    Am = (A if la == 0 else A.t()).contiguous()
    Bm = (B if lb == 0 else B.t()).contiguous()
    C = torch.full((M * N,), float("nan"), device="cuda").to(torch.float32 if types in (1, 3) else dt)
    loader().gemm(C, Am, Bm, M, N, K, lc, la, lb)
    g.device_status()
    Cl = (C.view(M, N) if lc == 0 else C.view(N, M).t())
    assert not torch.isnan(Cl.float()).any()

    rng = np.random.default_rng(5)
    rows = sorted(set([0, M - 1] + [r for r in (127, 128, 255, 256) if r < M] + list(rng.integers(0, M, 2))))
    cols = sorted(set([0, N - 1] + [c for c in (255, 256, 511, 512) if c < N] + list(rng.integers(0, N, 2))))
    A_bits = Am.view(torch.int16).cpu().numpy().view(np.uint16).ravel()
    B_bits = Bm.view(torch.int16).cpu().numpy().view(np.uint16).ravel()
    eps = 0.0 if types in (1, 3) else (2.0 ** -8 if bf16 else 2.0 ** -11)

    def compare(got, want):
        got, want = got.astype(np.float64), want.astype(np.float64)
        diff = np.abs(got - want)
        rel_fro = np.sqrt((diff ** 2).sum()) / np.sqrt((want ** 2).sum())
        assert rel_fro <= 1e-3, rel_fro
        # 16-bit outputs: output rounding (2 eps |ref| + eps sigma sqrt(K)); all outputs: the
        # order-of-summation noise of an f32 sum of K products.
        bound = 2 * eps * np.abs(want) + eps * sigma * np.sqrt(K) + f32_sum_tolerance(K, sigma)
        assert (diff <= bound).all(), (diff - bound).max()

    ref_rows = oracle.hgemm_select(types, A_bits, B_bits, M, N, K, 0, la, lb, rows=rows, cols=None)
    ref_rows = as_f32(types, ref_rows).reshape(M, N)[rows]
    compare(Cl[rows].float().cpu().numpy(), ref_rows)
    ref_cols = oracle.hgemm_select(types, A_bits, B_bits, M, N, K, 0, la, lb, rows=None, cols=cols)
    ref_cols = as_f32(types, ref_cols).reshape(M, N)[:, cols]
    compare(Cl[:, cols].float().cpu().numpy(), ref_cols)


def test_tuned_table_configs_run():
    """Whatever config the table selects for the benchmark shapes is a compiled variant."""
    for (M, N, K) in [(1024,) * 3, (2048,) * 3, (4096, 4096, 2048), (64, 8192, 8192)]:
        for (la, lb, lc) in LAYOUTS:
            for tg in (0, 1):
                cfg, idx = g.get_gemm_params(M, N, K, lc, la, lb, tg)
                assert idx >= 0 and cfg.tile_m == 128 * cfg.cluster


def test_device_status_is_clean():
    assert g.device_status() == 0
    assert g.launch_count() > 0


SKINNY = [(16, 1024, 512), (8, 256, 2048), (24, 136, 264), (40, 2048, 128), (64, 512, 576), (1, 128, 64), (48, 4096, 1024),
          (1024, 16, 512), (2048, 8, 256), (512, 24, 264), (640, 40, 128), (4096, 64, 192), (256, 32, 1024)]


@pytest.mark.parametrize("M,N,K", SKINNY)
def test_skinny_shapes(M, N, K):
    """One small dimension (<= 64): the narrow tile variants (16 / 32 / 64 columns) and, when the
    small dimension is the kernel's row extent, the operand swap with the transposing epilogue.
    All 8 layouts and 4 type pairs; split-K on top for the deep ones."""
    for types in range(4):
        bf16 = types >= 2
        for (la, lb, lc) in LAYOUTS:
            A, B = seeded(M, N, K, la, lb, bf16)
            ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
            got = gpu_gemm(types, A, B, M, N, K, lc, la, lb)
            check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)
            if K >= 512:
                cfg = g.GemmConfig(128, 128, 4, 1, 3, 0)
                got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)


@pytest.mark.parametrize("M,N,K,batch", [(16, 512, 256, 3), (16, 2048, 256, 3), (24, 4104, 192, 2)])
def test_skinny_batched(M, N, K, batch):
    """Strided-batched skinny problems; the wider ones are cut into row slabs counted over the
    whole batch (48-row slabs x 3 matrices fill one wave)."""
    for types in (1, 2):
        bf16 = types >= 2
        for (la, lb, lc) in [(0, 1, 0), (0, 0, 0), (1, 0, 1)]:
            A = np.concatenate([oracle.init_matrix(M, K, la, bf16)[(np.arange(M * K) + 13 * b) % (M * K)] for b in range(batch)])
            B = np.concatenate([oracle.init_matrix(K, N, lb, bf16)[(np.arange(K * N) + 7 * b) % (K * N)] for b in range(batch)])
            got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, batch=batch)
            for b in range(batch):
                ref = oracle.hgemm(types, A[b * M * K:(b + 1) * M * K], B[b * K * N:(b + 1) * K * N], M, N, K, lc, la, lb)
                check_parity(types, got[b * M * N:(b + 1) * M * N], ref, K, SIGMA_UNIFORM, M, N, lc)


@pytest.mark.parametrize("M,N,K", [(4096, 2560, 1024), (2304, 4352, 1024)])
def test_host_buffer_entry_point_pipelined(M, N, K):
    """Large host-buffer calls are chunked (rows of A or columns of B) and pipelined over
    copy-in / compute / copy-out streams; every layout stores its chunks differently."""
    for types in (2, 3):
        for (la, lb, lc) in LAYOUTS:
            A, B = seeded(M, N, K, la, lb, True)
            want = gpu_gemm(types, A, B, M, N, K, lc, la, lb)  # device-pointer path
            ta = torch.from_numpy(A.view(np.int16)).pin_memory()
            tb = torch.from_numpy(B.view(np.int16)).pin_memory()
            tc = torch.full((M * N,), -1, dtype=torch.float32 if types == 3 else torch.int16).pin_memory()
            loader().gemm_host(tc, ta, tb, M, N, K, lc, la, lb, types=types)
            got = tc.numpy() if types == 3 else tc.numpy().view(np.uint16)
            check_parity(types, got, want, K, SIGMA_UNIFORM, M, N, lc)
    # sampled rows of the last case against the CPU oracle
    rows = [0, 255, 256, M - 1]
    ref = oracle.hgemm_select(types, A, B, M, N, K, 0, la, lb, rows=rows)
    gl = got.reshape(M, N) if lc == 0 else got.reshape(N, M).T
    assert np.abs(gl[rows] - ref.reshape(M, N)[rows]).max() <= 1e-3


def test_concurrent_streams_and_threads():
    """The library keeps no per-call global state: four host threads, each on its own stream,
    run split-K and plain GEMMs at the same time (split-K workspaces are per stream)."""
    import threading
    M, N, K = 256, 768, 2048
    A, B = seeded(M, N, K, 0, 1, True)
    ref = oracle.hgemm(3, A, B, M, N, K, 0, 0, 1)
    dA, dB = to_device(A), to_device(B)
    torch.cuda.synchronize()
    results, errors = {}, []

    def work(i):
        try:
            st = torch.cuda.Stream()
            l = g.loader()
            outs = []
            with torch.cuda.stream(st):
                for rep in range(6):
                    C = torch.full((M * N,), float("nan"), device="cuda")
                    cfg = g.GemmConfig(128, 128, 4, 1, 1 + (i + rep) % 4, 0)
                    l.gemm(C, dA, dB, M, N, K, 0, 0, 1, stream=st, config=cfg, types=3)
                    outs.append(C)
            st.synchronize()
            results[i] = [c.cpu().numpy() for c in outs]
        except Exception as ex:  # surfaced in the main thread
            errors.append(ex)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert g.device_status() == 0
    for i in range(4):
        for out in results[i]:
            check_parity(3, out, ref, K, SIGMA_UNIFORM, M, N, 0)


def test_host_buffer_entry_point_from_two_threads():
    """b200_gemm_host keeps its staging buffers, streams and events per device and serialises
    callers: two host threads with different shapes (the second needs larger buffers, so the
    cached ones are regrown between calls) both get their own result."""
    import threading
    shapes = [(2304, 2560, 512, 0, 0, 1), (3072, 4096, 768, 1, 1, 0)]
    want, got, errors = {}, {}, []
    inputs = {}
    for i, (M, N, K, lc, la, lb) in enumerate(shapes):
        A, B = seeded(M, N, K, la, lb, True)
        inputs[i] = (A, B)
        want[i] = gpu_gemm(3, A, B, M, N, K, lc, la, lb)

    def work(i):
        try:
            M, N, K, lc, la, lb = shapes[i]
            A, B = inputs[i]
            ta, tb = torch.from_numpy(A.view(np.int16)).pin_memory(), torch.from_numpy(B.view(np.int16)).pin_memory()
            outs = []
            for _ in range(3):
                tc = torch.full((M * N,), float("nan"), dtype=torch.float32).pin_memory()
                g.loader().gemm_host(tc, ta, tb, M, N, K, lc, la, lb, types=3)
                outs.append(tc.numpy().copy())
            got[i] = outs
        except Exception as ex:
            errors.append(ex)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i in range(2):
        for out in got[i]:
            # the host path computes C in tiles, whose configurations may partition K differently
            assert np.abs(out - want[i]).max() <= max(1e-4, f32_sum_tolerance(shapes[i][2], SIGMA_UNIFORM))
    assert g.device_status() == 0


SLAB_EDGES = [(16, 8200, 576), (33, 9000, 264), (64, 8192 + 56, 320), (8, 20000, 192), (16, 8192, 4096 + 64),
              # 65..128 rows: too tall for the operand swap, the staged-epilogue kernels with K partitions
              (128, 8192, 576), (96, 9000, 264), (128, 2048, 4096 + 64), (100, 4096, 1024), (72, 1024, 128), (128, 16384 + 8, 64)]


@pytest.mark.parametrize("M,N,K", SLAB_EDGES)
def test_row_slab_edges(M, N, K):
    """Skinny problems wide enough for the row-slab partition (147+ slabs of 8..128 rows of the
    large operand), and their neighbours just above the 64-row limit of the operand swap: ragged last slab, K not a multiple of 64 (one k-block per ring slot, plain
    3-D maps) and long K (four k-blocks per slot through the 4-D maps), both storage orders of
    the large operand (K-major slabs of any height, M-major slabs of 64 rows)."""
    for types, (la, lb, lc) in [(1, (0, 1, 0)), (1, (0, 0, 0)), (2, (0, 1, 0)), (3, (1, 0, 0)), (0, (1, 1, 0)),
                                # column-major C: no operand swap, narrow staged-epilogue tiles on 32..128-row slabs
                                (1, (0, 1, 1)), (2, (1, 0, 1)), (3, (0, 0, 1))]:
        if lb == 0 and N % 8:
            continue
        bf16 = types >= 2
        A, B = seeded(M, N, K, la, lb, bf16)
        ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
        got = gpu_gemm(types, A, B, M, N, K, lc, la, lb)
        check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)


@pytest.mark.parametrize("M,N,K", [(512, 512, 4096), (768, 3072, 768), (1536, 1536, 512), (2048, 512, 2048), (384, 384, 384)])
def test_sizes_without_a_table_entry(M, N, K):
    """Sizes the tuned table does not hold: the borrowed entry is checked against the launch
    path's cost model, which may pick another tile or partition K.  Whatever it picks must
    give the reference's result."""
    for types, (la, lb, lc) in [(3, (0, 1, 0)), (2, (0, 0, 0)), (1, (1, 1, 1)), (0, (1, 0, 0))]:
        bf16 = types >= 2
        A, B = seeded(M, N, K, la, lb, bf16)
        ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
        got = gpu_gemm(types, A, B, M, N, K, lc, la, lb)
        check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)


def test_dependent_calls_back_to_back_and_in_a_graph():
    """Every kernel is launched as a programmatic dependent of the kernel before it (its set-up
    may overlap that kernel's tail).  A chain in which each GEMM reads what the previous one
    wrote - plain, split-K and skinny calls mixed - must give bit-identical results whether the
    calls are separated by synchronisation, issued back to back, or replayed from a CUDA graph."""
    M = 1024
    bf = torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(7)
    X0 = (torch.randn(M, M, device="cuda", generator=gen) * 0.05).to(bf)
    W = [(torch.randn(M, M, device="cuda", generator=gen) * 0.05).to(bf) for _ in range(4)]
    V = (torch.randn(16, M, device="cuda", generator=gen) * 0.05).to(bf)
    l = loader()
    split = g.GemmConfig(128, 128, 4, 1, 4, 0)

    def chain(bufs, sync):
        x = X0
        for i, w in enumerate(W):
            l.gemm(bufs[i], x, w, M, M, M, 0, 0, 1, types=2, config=split if i % 2 else None)
            if sync:
                torch.cuda.synchronize()
            x = bufs[i]
        l.gemm(bufs[4], V, x, 16, M, M, 0, 0, 1, types=2)  # skinny call reading the chain's end

    def fresh():
        return [torch.zeros(M, M, device="cuda", dtype=bf) for _ in range(4)] + [torch.zeros(16, M, device="cuda", dtype=bf)]

    ref = fresh()
    chain(ref, sync=True)
    torch.cuda.synchronize()
    b2b = fresh()
    for _ in range(3):
        chain(b2b, sync=False)
    torch.cuda.synchronize()
    for r, o in zip(ref, b2b):
        assert torch.equal(r.view(torch.int16), o.view(torch.int16))
    gb = fresh()
    chain(gb, sync=False)  # warm the per-stream state before capture
    torch.cuda.synchronize()
    for t in gb:
        t.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain(gb, sync=False)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert g.device_status() == 0
    for r, o in zip(ref, gb):
        assert torch.equal(r.view(torch.int16), o.view(torch.int16))
    assert float(ref[4].float().abs().max()) > 0


@pytest.mark.parametrize("tile_n", [160, 192, 224])
def test_pair_tile_widths_between_the_compiled_ones(tile_n):
    """The 256-column CTA-pair kernel takes its tile width at run time (multiples of 32 columns
    between 128 and 256; whole 128-byte output chunks, so 16-bit outputs need multiples of 64;
    the kernel view's B' must be K-major).  Ragged N, split-K and raster bands on top."""
    M, N, K = 640, 1000 if tile_n != 192 else 1184, 448
    for types in range(4):
        bf16 = types >= 2
        chunk = 32 if types in (1, 3) else 64
        for (la, lb, lc) in [(0, 1, 0), (1, 1, 0), (0, 0, 1), (0, 1, 1)]:
            A, B = seeded(M, N, K, la, lb, bf16)
            for split_k, raster in [(1, 0), (2, 2)]:
                cfg = g.GemmConfig(256, tile_n, 6, 2, split_k, raster)
                if tile_n % chunk:
                    with pytest.raises(g.GemmError):
                        gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                    continue
                ref = oracle.hgemm(types, A, B, M, N, K, lc, la, lb)
                got = gpu_gemm(types, A, B, M, N, K, lc, la, lb, config=cfg)
                check_parity(types, got, ref, K, SIGMA_UNIFORM, M, N, lc)
    # an N-major B' (row-major B with a row-major C) cannot use an in-between width
    A, B = seeded(M, N, K, 0, 0, True)
    with pytest.raises(g.GemmError):
        gpu_gemm(3, A, B, M, N, K, 0, 0, 0, config=g.GemmConfig(256, tile_n, 6, 2, 1, 0))
    # ... and one CTA cannot either
    with pytest.raises(g.GemmError):
        gpu_gemm(3, A, B, M, N, K, 0, 0, 1, config=g.GemmConfig(128, tile_n, 4, 1, 1, 0))
