"""Generates the golden fixtures in this directory from the reference's own CPU code.

Run where a checkout of adelj88/rocm_wmma_gemm is available (oracle/build.py compiles its
test/test.hpp unmodified into oracle/_ref/libref_hgemm.so):

    python tests/golden/make_golden.py

Fixtures (inputs come from the reference's seeded init_matrix, outputs from its hgemm_cpu):
  init_matrix.npz   raw 16-bit patterns of small matrices, both layouts, f16 and bf16
  hgemm_small.npz   C for M,N,K = 16,24,32, all 4 type pairs x 8 layout triples
  config1.json      known answers for fp16->f32 M=N=K=256, A row / B col / C row, plus a
                    SHA-256 of A, B and C for all four type pairs at that shape
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SMALL = (16, 24, 32)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def main():
    if oracle.ref_lib() is None:
        raise SystemExit("the compiled reference (oracle/_ref) is not available here")
    init = {}
    for rows, cols in [(5, 7), (16, 16), (3, 64)]:
        for layout in (0, 1):
            for bf16 in (0, 1):
                init[f"r{rows}_c{cols}_l{layout}_bf{bf16}"] = oracle.init_matrix(rows, cols, layout, bool(bf16), impl="ref")
    np.savez_compressed(os.path.join(HERE, "init_matrix.npz"), **init)

    M, N, K = SMALL
    small = {}
    for types in range(4):
        bf16 = types >= 2
        for key in range(8):
            lc, la, lb = key >> 2, (key >> 1) & 1, key & 1
            A = oracle.init_matrix(M, K, la, bf16, impl="ref")
            B = oracle.init_matrix(K, N, lb, bf16, impl="ref")
            small[f"t{types}_c{lc}_a{la}_b{lb}"] = oracle.hgemm(types, A, B, M, N, K, lc, la, lb, impl="ref")
    np.savez_compressed(os.path.join(HERE, "hgemm_small.npz"), **small)

    kat = {"shape": [256, 256, 256], "layout": {"A": "row_major", "B": "col_major", "C": "row_major"}, "types": {}}
    for types, name in enumerate(["f16_f16", "f32_f16", "bf16_bf16", "f32_bf16"]):
        bf16 = types >= 2
        A = oracle.init_matrix(256, 256, 0, bf16, impl="ref")
        B = oracle.init_matrix(256, 256, 1, bf16, impl="ref")
        C = oracle.hgemm(types, A, B, 256, 256, 256, 0, 0, 1, impl="ref")
        Cf = C if C.dtype == np.float32 else oracle.bits_to_f32(C, bf16)
        kat["types"][name] = {
            "sha256_A": sha(A), "sha256_B": sha(B), "sha256_C": sha(C),
            "A00": float(oracle.bits_to_f32(A[:1], bf16)[0]), "A01": float(oracle.bits_to_f32(A[1:2], bf16)[0]),
            "C00": float(Cf[0]), "C_last": float(Cf[-1]),
            "frobenius": float(np.sqrt((Cf.astype(np.float64) ** 2).sum())),
        }
    with open(os.path.join(HERE, "config1.json"), "w") as f:
        json.dump(kat, f, indent=1, sort_keys=True)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
