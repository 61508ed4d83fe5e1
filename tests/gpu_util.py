"""Helpers shared by the GPU parity tests: move raw 16-bit patterns to the device, call the
library through its C ABI, bring C back as numpy."""
import numpy as np
import torch

import oracle
import rocm_wmma_gemm_b200 as g

NAMES = ["f16_f16", "f32_f16", "bf16_bf16", "f32_bf16"]
EPS_OUT = {0: 2.0 ** -11, 2: 2.0 ** -8}  # half-ulp relative step of f16 / bf16 outputs
LOADER = None


def loader():
    global LOADER
    if LOADER is None:
        LOADER = g.loader()
    return LOADER


def to_device(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16)).cuda()


def out_tensor(types: int, n: int, guard: int = 0) -> torch.Tensor:
    """Output buffer of n elements (+ guard elements either side), poisoned so that any
    element the kernel fails to write shows up (NaN for f32, 0xFFFF for 16-bit)."""
    if types in (1, 3):
        return torch.full((n + 2 * guard,), float("nan"), dtype=torch.float32, device="cuda")
    return torch.full((n + 2 * guard,), -1, dtype=torch.int16, device="cuda")


def gpu_gemm(types, A_bits, B_bits, M, N, K, lc, la, lb, batch=1, config=None, checked=True, guard=64):
    """Runs C = A*B on the GPU through the C ABI; returns flat numpy C (float32 or uint16)."""
    dA, dB = to_device(A_bits), to_device(B_bits)
    n = M * N * batch
    dC = out_tensor(types, n, guard)
    esz = dC.element_size()
    ptr = dC.data_ptr() + guard * esz
    loader().gemm(ptr, dA, dB, M, N, K, lc, la, lb, batch_count=batch, types=types, config=config, checked=checked)
    g.device_status()  # synchronises; raises if a kernel gave up on a bounded wait
    out = dC.cpu().numpy()
    if guard:
        poison = out[:guard]
        ok = np.isnan(poison).all() if types in (1, 3) else (poison == -1).all()
        tail = out[guard + n:]
        ok = ok and (np.isnan(tail).all() if types in (1, 3) else (tail == -1).all())
        assert ok, "the kernel wrote outside C"
    out = out[guard:guard + n]
    return out if types in (1, 3) else out.view(np.uint16)


def as_f32(types, C):
    return C if types in (1, 3) else oracle.bits_to_f32(C, types == 2)


def f32_sum_tolerance(K, sigma):
    """Order-of-summation noise between two f32 sums of K products of standard deviation sigma:
    the CPU reference adds sequentially (error ~ 2^-24 * sqrt(K) * |partial sum| per element,
    |partial sum| ~ sigma * sqrt(K)); 16x that covers the tail over millions of elements."""
    return 2.0 ** -20 * K * sigma


def check_parity(types, gpu, ref, K, sigma, M, N, lc, abs_tol_f32=None):
    """The acceptance bar for one result.

    f32 outputs: relative Frobenius error <= 1e-3, and every element within abs_tol_f32 of the
    CPU reference: 1e-4 (the reference test's own tolerance, test/gemm/test_float_accum.cpp:128,
    which its shapes with K <= 512 meet) or, for longer sums, f32_sum_tolerance(K, sigma).
    f16 / bf16 outputs: |gpu - ref| <= 2*eps*|ref| + eps*sigma*sqrt(K) per element, where eps is
    2^-11 (f16) or 2^-8 (bf16) and sigma the standard deviation of one product, and the
    reference's cosine-similarity thresholds (0.995 / 0.97, test/test.hpp:204-211)."""
    gf, rf = as_f32(types, gpu).astype(np.float64), as_f32(types, ref).astype(np.float64)
    assert not np.isnan(gf).any(), "unwritten or NaN elements in C"
    diff = np.abs(gf - rf)
    rel_fro = np.sqrt((diff ** 2).sum()) / max(np.sqrt((rf ** 2).sum()), 1e-30)
    assert rel_fro <= 1e-3, f"relative Frobenius error {rel_fro}"
    if types in (1, 3):
        if abs_tol_f32 is None:
            abs_tol_f32 = 1e-4 if K <= 512 else f32_sum_tolerance(K, sigma)
        assert diff.max() <= abs_tol_f32, f"max abs error {diff.max()} > {abs_tol_f32}"
    else:
        eps = EPS_OUT[types]
        bound = 2 * eps * np.abs(rf) + eps * sigma * np.sqrt(K)
        worst = (diff - bound).max()
        assert worst <= 0, f"element exceeds K-scaled tolerance by {worst}"
        kind = 2 if types == 2 else 0
        cos = oracle.cosine_similarity(gpu, ref, M, N, lc, kind)
        assert cos > (0.97 if types == 2 else 0.995), f"cosine similarity {cos}"
    return rel_fro, diff.max()
