"""TEST INFRASTRUCTURE — NOT PRODUCT CODE.

ctypes view of the CPU oracle for the half-precision GEMM path:

* `liboracle_gemm.so` — plain-C restatement (cpu_gemm.c) of the reference's input generator,
  CPU reference GEMM and cosine-similarity check (test/test.hpp:33-196 of
  adelj88/rocm_wmma_gemm).
* `_ref/libref_hgemm.so` — the reference's own test/test.hpp compiled unmodified through
  ref_shim.cpp (present when oracle/build.py could see a reference checkout, or prebuilt).

Only tests/, the smoke check and the benchmark's CPU-baseline / reference legs import this
package.  The GEMM library never does.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))
TYPE_PAIRS = {("f16", "f16"): 0, ("f32", "f16"): 1, ("bf16", "bf16"): 2, ("f32", "bf16"): 3}

_c = ctypes
_sz = _c.c_size_t
_vp = _c.c_void_p


def _load(path, sigs):
    lib = _c.CDLL(path)
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


_ORACLE_SIGS = {
    "oracle_f16_to_f32": (_c.c_float, [_c.c_uint16]),
    "oracle_f32_to_f16": (_c.c_uint16, [_c.c_float]),
    "oracle_bf16_to_f32": (_c.c_float, [_c.c_uint16]),
    "oracle_f32_to_bf16": (_c.c_uint16, [_c.c_float]),
    "oracle_init_matrix": (None, [_vp, _sz, _sz, _c.c_int, _c.c_int]),
    "oracle_init_matrix_cyclic": (None, [_vp, _sz, _sz, _c.c_int, _c.c_int]),
    "oracle_hgemm": (_c.c_int, [_c.c_int, _vp, _vp, _vp, _sz, _sz, _sz, _c.c_int, _c.c_int, _c.c_int, _c.c_int]),
    "oracle_hgemm_rows": (_c.c_int, [_c.c_int, _vp, _vp, _vp, _sz, _sz, _sz, _c.c_int, _c.c_int, _c.c_int,
                                     _sz, _sz, _c.c_int]),
    "oracle_hgemm_select": (_c.c_int, [_c.c_int, _vp, _vp, _vp, _sz, _sz, _sz, _c.c_int, _c.c_int, _c.c_int,
                                       _vp, _sz, _sz, _sz, _vp, _sz, _c.c_int]),
    "oracle_cosine_similarity": (_c.c_float, [_vp, _vp, _sz, _sz, _c.c_int, _c.c_int]),
}
_REF_SIGS = {
    "ref_init_matrix": (None, [_vp, _sz, _sz, _c.c_int, _c.c_int]),
    "ref_hgemm": (None, [_c.c_int, _vp, _vp, _vp, _sz, _sz, _sz, _c.c_int, _c.c_int, _c.c_int]),
    "ref_hgemm_rows_mt": (None, [_c.c_int, _vp, _vp, _vp, _sz, _sz, _sz, _c.c_int, _c.c_int, _c.c_int,
                                 _sz, _sz, _c.c_int]),
    "ref_cosine_similarity": (_c.c_float, [_vp, _vp, _sz, _sz, _c.c_int, _c.c_int]),
    "ref_hardware_threads": (_c.c_uint, []),
}

_oracle = None
_ref = None
_ref_tried = False


def oracle_lib():
    """The C restatement; built on first use (needs gcc)."""
    global _oracle
    if _oracle is None:
        _oracle = _load(_build.build_oracle(), _ORACLE_SIGS)
    return _oracle


def ref_lib():
    """The compiled reference CPU path, or None when neither a reference checkout nor a
    prebuilt oracle/_ref library is available."""
    global _ref, _ref_tried
    if not _ref_tried:
        _ref_tried = True
        path = _build.build_ref()
        if path and os.path.exists(path):
            _ref = _load(path, _REF_SIGS)
    return _ref


def host_threads() -> int:
    return os.cpu_count() or 1


def _p(a: np.ndarray):
    return a.ctypes.data_as(_vp)


def out_dtype(types: int):
    return np.float32 if types in (1, 3) else np.uint16


def init_matrix(rows: int, cols: int, layout: int, bf16: bool, impl: str = "oracle", cyclic: bool = False) -> np.ndarray:
    """Flat uint16 array (raw f16 / bf16 bits) of a rows x cols matrix stored in `layout`."""
    data = np.empty(rows * cols, dtype=np.uint16)
    if impl == "ref":
        assert not cyclic
        ref_lib().ref_init_matrix(_p(data), rows, cols, layout, int(bf16))
    elif cyclic:
        oracle_lib().oracle_init_matrix_cyclic(_p(data), rows, cols, layout, int(bf16))
    else:
        oracle_lib().oracle_init_matrix(_p(data), rows, cols, layout, int(bf16))
    return data


def hgemm(types: int, A: np.ndarray, B: np.ndarray, M: int, N: int, K: int, lc: int, la: int, lb: int,
          impl: str = "oracle", threads: int = 0) -> np.ndarray:
    """C = A * B on the CPU.  A, B: flat uint16 arrays of raw bits; returns flat C (float32 or
    raw uint16 bits) in layout lc."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    assert A.size == M * K and B.size == K * N
    C = np.zeros(M * N, dtype=out_dtype(types))
    if impl == "ref":
        ref_lib().ref_hgemm(types, _p(C), _p(A), _p(B), M, N, K, lc, la, lb)
    else:
        rc = oracle_lib().oracle_hgemm(types, _p(C), _p(A), _p(B), M, N, K, lc, la, lb, threads or host_threads())
        if rc != 0:
            raise RuntimeError("oracle_hgemm failed")
    return C


def hgemm_select(types: int, A: np.ndarray, B: np.ndarray, M: int, N: int, K: int, lc: int, la: int, lb: int,
                 rows=None, cols=None, threads: int = 0) -> np.ndarray:
    """Computes only C(i, j) for i in rows and j in cols (None = all); other elements stay NaN
    (f32) / 0xFFFF (16-bit)."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    dt = out_dtype(types)
    C = np.full(M * N, np.nan if dt == np.float32 else 0xFFFF, dtype=dt)
    r = None if rows is None else np.ascontiguousarray(rows, dtype=np.uint32)
    c = None if cols is None else np.ascontiguousarray(cols, dtype=np.uint32)
    rc = oracle_lib().oracle_hgemm_select(
        types, _p(C), _p(A), _p(B), M, N, K, lc, la, lb,
        _p(r) if r is not None else None, 0 if r is None else r.size, 0, M,
        _p(c) if c is not None else None, 0 if c is None else c.size, threads or host_threads())
    if rc != 0:
        raise RuntimeError("oracle_hgemm_select failed")
    return C


def cosine_similarity(gpu: np.ndarray, cpu: np.ndarray, M: int, N: int, layout: int, kind: int, impl: str = "oracle") -> float:
    """kind: 0 f16 bits, 1 float32, 2 bf16 bits."""
    gpu = np.ascontiguousarray(gpu)
    cpu = np.ascontiguousarray(cpu)
    if impl == "ref":
        return float(ref_lib().ref_cosine_similarity(_p(gpu), _p(cpu), M, N, layout, kind))
    return float(oracle_lib().oracle_cosine_similarity(_p(gpu), _p(cpu), M, N, layout, kind))


def bits_to_f32(bits: np.ndarray, bf16: bool) -> np.ndarray:
    bits = np.asarray(bits, dtype=np.uint16)
    if bf16:
        return (bits.astype(np.uint32) << 16).view(np.float32)
    return bits.view(np.float16).astype(np.float32)
