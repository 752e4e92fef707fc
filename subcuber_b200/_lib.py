"""ctypes loader for libsubcuber_b200.so (the C ABI declared in include/subcuber_b200.h).

The library is the product: there is no Python or CPU fallback.  If the shared object is missing it is
built with nvcc; if that is impossible the import fails with an error that says so.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

LIB_PATH = _build.LIB


class KernelRunnerBuffers(C.Structure):
    """Mirror of `struct KernelRunnerBuffers` (reference: src/cuda/kernel_runner_support.cuh:16-21)."""

    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("d", C.c_void_p)]


RUN_ARGTYPES = [KernelRunnerBuffers, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_int,
                C.c_int, C.POINTER(C.c_float)]
RUN_FN = C.CFUNCTYPE(C.c_int, *RUN_ARGTYPES)


class KernelEntry(C.Structure):
    """Mirror of `sb200_kernel_entry` (reference: `struct KernelEntry`, src/cuda/kernel_runner.cpp:99-105)."""

    _fields_ = [("name", C.c_char_p), ("arch", C.c_char_p), ("dtype", C.c_char_p), ("strassen_level", C.c_int),
                ("run", RUN_FN)]


class WorkspaceLayout(C.Structure):
    """Mirror of `sb200_workspace_layout`."""

    _fields_ = [("status", C.c_size_t), ("presum_a", C.c_size_t), ("presum_b", C.c_size_t),
                ("handoff", C.c_size_t * 4), ("total", C.c_size_t), ("mq", C.c_int), ("nq", C.c_int),
                ("kq", C.c_int), ("tiles_m", C.c_int), ("tiles_n", C.c_int), ("bn", C.c_int)]


class GemmOptions(C.Structure):
    """Mirror of `sb200_gemm_options`."""

    _fields_ = [("sm_limit", C.c_int), ("no_split", C.c_int), ("wait_limit_us", C.c_int),
                ("drop_split_flags", C.c_int)]


_lib = None


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load the CUDA library, building it first when the .so is absent.  Raises if neither works."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m subcuber_b200.build`")
        _build.build()
    elif not _build.up_to_date():
        # a library older than its sources may no longer match the struct mirrors below
        if build_if_missing and _build.have_nvcc():
            _build.build()
        else:
            raise RuntimeError(f"{LIB_PATH} is older than its sources: run `python -m subcuber_b200.build`")
    lib = C.CDLL(LIB_PATH)
    lib.sb200_num_kernels.restype = C.c_int
    lib.sb200_kernel.restype = C.POINTER(KernelEntry)
    lib.sb200_kernel.argtypes = [C.c_int]
    lib.sb200_gemm_can_implement.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int]
    lib.sb200_gemm_workspace_bytes.restype = C.c_size_t
    lib.sb200_gemm_workspace_bytes.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int]
    lib.sb200_gemm.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                               C.c_size_t, C.c_void_p]
    lib.sb200_gemm_workspace_bytes_opt.restype = C.c_size_t
    lib.sb200_gemm_workspace_bytes_opt.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(GemmOptions)]
    lib.sb200_gemm_opt.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                   C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(GemmOptions)]
    lib.sb200_gemm_deal.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(GemmOptions), C.c_int,
                                    C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int)]
    lib.sb200_gemm_ex.argtypes = [C.c_char_p, C.c_double, C.c_void_p, C.c_void_p, C.c_double, C.c_void_p, C.c_void_p,
                                  C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.sb200_gemm_colmajor.argtypes = lib.sb200_gemm.argtypes
    lib.sb200_gemm_status.argtypes = [C.c_void_p, C.c_void_p]
    lib.sb200_gemm_launches.argtypes = [C.c_char_p]
    lib.sb200_gemm_host.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
    lib.sb200_gemm_workspace_layout.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(WorkspaceLayout)]
    lib.sb200_gemm_timed.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)]
    lib.sb200_tile_program.argtypes = [C.c_char_p, C.c_void_p, C.c_size_t]
    lib.sb200_tile_program_bytes.restype = C.c_size_t
    lib.sb200_fill_device.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_uint, C.c_void_p, C.c_ulonglong, C.c_void_p]
    lib.sb200_fill_host.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_uint, C.c_void_p, C.c_ulonglong]
    lib.sb200_events_create.restype = C.c_void_p
    lib.sb200_events_create.argtypes = [C.c_int]
    lib.sb200_events_destroy.restype = None
    lib.sb200_events_destroy.argtypes = [C.c_void_p]
    lib.sb200_events_elapsed_ms.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float)]
    lib.sb200_gemm_events.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                      C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(GemmOptions)]
    lib.sb200_peer_signal.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]
    lib.sb200_peer_wait.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_uint, C.c_void_p, C.c_void_p]
    lib.sb200_gemm_f16_sw_static_scratch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                                     C.c_void_p, C.c_int]
    _lib = lib
    return lib
