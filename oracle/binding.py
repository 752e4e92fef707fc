"""ctypes binding of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the shipped
package never does.  `oracle()` loads liboracle.so (the plain-C restatement, built by `make -C oracle`);
`ref_oracle()` loads _ref/libref_oracle.so (the reference project's own oracle kernels compiled for the
host, built by `make -C oracle ref` on a machine that has the reference tree) or returns None.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import ml_dtypes  # numpy's bfloat16
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

DTYPE_CODE = {"f16": 0, "f32": 1, "f64": 2, "tf32": 3, "bf16": 4}
NP_DTYPE = {"f16": np.float16, "f32": np.float32, "f64": np.float64, "tf32": np.float32, "bf16": ml_dtypes.bfloat16}


def build(ref: bool = True) -> None:
    subprocess.run(["make", "-s", "-C", _HERE], check=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    if ref:
        subprocess.run(["make", "-s", "-C", _HERE, "ref"], check=False, stdout=subprocess.DEVNULL,
                       stderr=subprocess.DEVNULL)


_vp, _i, _d = C.c_void_p, C.c_int, C.c_double
_lib = None
_ref = None


def oracle() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(ref=False)
        _lib = C.CDLL(path)
        _lib.orc_gemm.argtypes = [_i, _i, _i, _i, _d, _vp, _i, _vp, _i, _d, _vp, _vp, _i, _i, _vp]
        _lib.orc_sw_gemm.argtypes = [_i, _i, _i, _i, _i, _d, _vp, _i, _vp, _i, _d, _vp, _vp, _i, _i, _vp, _i]
        _lib.orc_sw_presums.argtypes = [_i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp]
        _lib.orc_truth_rows.argtypes = [_i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _i, _vp]
    return _lib


def ref_oracle():
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref_oracle.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
        _ref.ref_sw_gemm.argtypes = [_i, _i, _i, _i, _i, _d, _vp, _i, _vp, _i, _d, _vp, _i]
        _ref.ref_sw_presums.argtypes = [_i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _vp]
    return _ref


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _rows(rows):
    if rows is None:
        return 0, None, None
    r = np.ascontiguousarray(rows, dtype=np.int32)
    return int(r.size), r, r.ctypes.data_as(_vp)


def sw_gemm(dtype: str, level: int, A: np.ndarray, B: np.ndarray, rows=None, alpha=1.0, beta=0.0, Cin=None,
            interim_round: bool = False) -> np.ndarray:
    """D = alpha * (A @ B by Strassen-Winograd at `level`) + beta * Cin in the type set `dtype`.

    With `rows` (level 0: C rows; level 1: quadrant rows r, producing C rows r and r + M/2; level 2: rows r of the
    innermost quadrants, producing C rows r, r + M/4, r + M/2 and r + 3M/4) only those rows of the returned matrix
    are meaningful; the rest are zero.
    """
    npd = NP_DTYPE[dtype]
    A = np.ascontiguousarray(A, dtype=npd)
    B = np.ascontiguousarray(B, dtype=npd)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    out = np.zeros((M, N), dtype=npd)
    cin = None if Cin is None else np.ascontiguousarray(Cin, dtype=npd)
    n, keep, rp = _rows(rows)
    rc = oracle().orc_sw_gemm(DTYPE_CODE[dtype], level, M, N, K, alpha, _ptr(A), K, _ptr(B), N, beta, _ptr(cin),
                              _ptr(out), N, n, rp, int(interim_round))
    if rc != 0:
        raise ValueError(f"orc_sw_gemm rejected the arguments (rc={rc})")
    return out


def sw_presums(dtype: str, A: np.ndarray, B: np.ndarray):
    """(pa[4, M/2, K/2] = S1,S2,A02,A1S2 ; pb[4, K/2, N/2] = B10,B31,S3,S3B2) in the operand type."""
    npd = NP_DTYPE[dtype]
    A = np.ascontiguousarray(A, dtype=npd)
    B = np.ascontiguousarray(B, dtype=npd)
    M, K = A.shape
    _, N = B.shape
    pa = np.zeros((4, M // 2, K // 2), dtype=npd)
    pb = np.zeros((4, K // 2, N // 2), dtype=npd)
    rc = oracle().orc_sw_presums(DTYPE_CODE[dtype], M, N, K, _ptr(A), K, _ptr(B), N, _ptr(pa), _ptr(pb))
    if rc != 0:
        raise ValueError("orc_sw_presums rejected the arguments")
    return pa, pb


def truth_rows(dtype: str, A: np.ndarray, B: np.ndarray, rows) -> np.ndarray:
    """Rows `rows` of A @ B accumulated in double from the stored operand values."""
    npd = NP_DTYPE[dtype]
    A = np.ascontiguousarray(A, dtype=npd)
    B = np.ascontiguousarray(B, dtype=npd)
    M, K = A.shape
    _, N = B.shape
    n, keep, rp = _rows(rows)
    out = np.zeros((n, N), dtype=np.float64)
    rc = oracle().orc_truth_rows(DTYPE_CODE[dtype], M, N, K, _ptr(A), K, _ptr(B), N, _ptr(out), n, rp)
    if rc != 0:
        raise ValueError("orc_truth_rows rejected the arguments")
    return out


def ref_sw_gemm(dtype: str, level: int, A: np.ndarray, B: np.ndarray, alpha=1.0, beta=0.0, Cin=None):
    """The reference project's own oracle kernels (host build).  Returns None when that build is absent."""
    lib = ref_oracle()
    if lib is None:
        return None
    npd = NP_DTYPE[dtype]
    A = np.ascontiguousarray(A, dtype=npd)
    B = np.ascontiguousarray(B, dtype=npd)
    M, K = A.shape
    _, N = B.shape
    out = np.zeros((M, N), dtype=npd) if Cin is None else np.array(Cin, dtype=npd, order="C", copy=True)
    rc = lib.ref_sw_gemm(DTYPE_CODE[dtype], level, M, N, K, alpha, _ptr(A), K, _ptr(B), N, beta, _ptr(out), N)
    if rc != 0:
        raise ValueError("ref_sw_gemm rejected the arguments")
    return out


def ref_sw_presums(dtype: str, A: np.ndarray, B: np.ndarray):
    lib = ref_oracle()
    if lib is None:
        return None
    npd = NP_DTYPE[dtype]
    A = np.ascontiguousarray(A, dtype=npd)
    B = np.ascontiguousarray(B, dtype=npd)
    M, K = A.shape
    _, N = B.shape
    pa = np.zeros((4, M // 2, K // 2), dtype=npd)
    pb = np.zeros((4, K // 2, N // 2), dtype=npd)
    rc = lib.ref_sw_presums(DTYPE_CODE[dtype], M, N, K, _ptr(A), K, _ptr(B), N, _ptr(pa), _ptr(pb))
    if rc != 0:
        raise ValueError("ref_sw_presums rejected the arguments")
    return pa, pb
