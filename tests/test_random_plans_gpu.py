"""Randomised sweep of the launch rules: shapes the tuned table has no entry for, every type
pair and layout, batched now and then, each through whatever `b200_gemm_plan` chooses for it
(narrow tiles, slabs with and without K partitions in clusters, run-time pair widths, the
CUDA-core kernel, ...).  The reference here is an f32 matrix product of the same half-precision
inputs on the GPU (torch): the shapes are too large for the CPU oracle, which the other tests
use; the tolerance is theirs (tests/gpu_util.py: one output rounding plus sqrt(K) growth)."""
import random

import pytest
import torch

import rocm_wmma_gemm_b200 as g

pytestmark = pytest.mark.gpu


def _cases(seed: int, n: int):
    rnd = random.Random(seed)
    out = []
    for i in range(n):
        family = i % 3
        if family == 0:    # skinny, either orientation
            a, b = rnd.choice([1, 8, 16, 24, 40, 48, 64]), rnd.choice([1000, 2048, 2368, 4096, 8192])
            M, N = (a, b) if rnd.random() < 0.7 else (b, a)
            K = rnd.choice([1024, 2112, 4096, 4160, 8192])
        elif family == 1:  # a few tile-rows, long K
            a, b = rnd.choice([96, 128, 136, 192, 256, 320, 384]), rnd.choice([1024, 2048, 4096, 5000, 8192])
            M, N = (a, b) if rnd.random() < 0.7 else (b, a)
            K = rnd.choice([1024, 2048, 3008, 4096, 8192])
        else:              # mid-size rectangles
            M, N = rnd.randrange(256, 3200, 8), rnd.randrange(256, 3200, 8)
            K = rnd.choice([64, 128, 256, 512, 1000, 1536, 2304, 3000])
        types = rnd.randrange(4)
        la, lb, lc = rnd.randrange(2), rnd.randrange(2), rnd.randrange(2)
        batch = 1 if rnd.random() < 0.85 or M * N > 2_000_000 else rnd.choice([2, 3])
        out.append((M, N, K, types, la, lb, lc, batch))
    return out


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_through_the_default_plans(seed):
    L = g.loader()
    kinds = set()
    for (M, N, K, types, la, lb, lc, batch) in _cases(seed, 24):
        bf16 = types >= 2
        dt = torch.bfloat16 if bf16 else torch.float16
        odt = torch.float32 if types in (1, 3) else dt
        gen = torch.Generator(device="cuda").manual_seed(seed * 1000 + M + N + K)
        A = (torch.rand(batch, M, K, device="cuda", generator=gen) * 2 - 1).to(dt)
        B = (torch.rand(batch, K, N, device="cuda", generator=gen) * 2 - 1).to(dt)
        Am = A if la == 0 else A.transpose(1, 2).contiguous()
        Bm = B if lb == 0 else B.transpose(1, 2).contiguous()
        C = torch.full((batch, M, N) if lc == 0 else (batch, N, M), float("nan"), device="cuda", dtype=odt)
        L.gemm(C, Am, Bm, M, N, K, layout_c=lc, layout_a=la, layout_b=lb, batch_count=batch, types=types)
        torch.cuda.synchronize()
        got = (C if lc == 0 else C.transpose(1, 2)).float()
        ref = torch.bmm(A.float(), B.float())
        if types in (1, 3):   # f32 output: relative Frobenius error as in the parity tests
            rel = ((got - ref).norm() / ref.norm()).item()
            assert rel <= 1e-3, (M, N, K, types, la, lb, lc, batch, rel)
        else:                 # 16-bit output: one rounding of the f32 sum (+ the order of the f32 additions)
            ulp = 2.0 ** -8 if bf16 else 2.0 ** -11
            lim = 2 * ulp * ref.abs() + ulp * (K ** 0.5) / 3.0
            worst = ((got - ref).abs() - lim).max().item()
            assert worst <= 0, (M, N, K, types, la, lb, lc, batch, worst)
        p = g.plan(M, N, K, lc, la, lb, types=types, batch_count=batch)
        kinds.add((p.kernel, p.cluster, p.cluster_k, min(p.split_k, 2)))
    assert g.device_status() == 0
    assert len(kinds) >= 4, kinds   # the sweep really went through several kernel families
