"""Seeded synthetic operands (the C generator in csrc/fill.cu, bound through the C ABI).

These stand in for the reference driver's run-time fills (src/cuda/kernel_runner.cpp:263-275 and
tests/base_test.cuh:248-262 in the reference project): element i of a matrix is a pure function of
(seed, subsequence, i), identical on host and device for the "uniform1" and "harness" distributions.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

DTYPE_CODE = {"f16": 0, "f32": 1, "f64": 2, "bf16": 3}
DIST_CODE = {"uniform1": 0, "normal": 1, "harness": 2}
NP_DTYPE = {"f16": np.float16, "f32": np.float32, "f64": np.float64}


def np_dtype(dtype: str):
    """numpy element type of `dtype`; bfloat16 comes from the ml_dtypes package (imported only when asked for)."""
    if dtype == "bf16":
        import ml_dtypes

        return ml_dtypes.bfloat16
    return NP_DTYPE[dtype]


def fill_host(dtype: str, dist: str, shape, seed: int = 1, subsequence: int = 0) -> np.ndarray:
    """Matrix of `shape` filled on the host."""
    out = np.empty(shape, dtype=np_dtype(dtype))
    rc = _lib.load().sb200_fill_host(DTYPE_CODE[dtype], DIST_CODE[dist], seed, subsequence,
                                     out.ctypes.data_as(C.c_void_p), out.size)
    if rc != 0:
        raise ValueError(f"sb200_fill_host failed with {rc}")
    return out


def fill_device(dtype: str, dist: str, shape, seed: int = 1, subsequence: int = 0, device="cuda:0"):
    """torch CUDA tensor of `shape` filled on the device (same values as fill_host)."""
    import torch

    tdt = {"f16": torch.float16, "f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16}[dtype]
    out = torch.empty(shape, dtype=tdt, device=device)
    with torch.cuda.device(out.device):
        s = torch.cuda.current_stream(out.device).cuda_stream
        rc = _lib.load().sb200_fill_device(DTYPE_CODE[dtype], DIST_CODE[dist], seed, subsequence, out.data_ptr(),
                                           out.numel(), s)
    if rc != 0:
        raise RuntimeError(f"sb200_fill_device failed with {rc}")
    return out


def operands(dtype: str, dist: str, m: int, n: int, k: int, seed: int = 1, device=None):
    """(A, B) with the convention A = subsequence 0, B = subsequence 1.  Host arrays when device is None."""
    if device is None:
        return fill_host(dtype, dist, (m, k), seed, 0), fill_host(dtype, dist, (k, n), seed, 1)
    return fill_device(dtype, dist, (m, k), seed, 0, device), fill_device(dtype, dist, (k, n), seed, 1, device)
