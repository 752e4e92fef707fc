"""Python mirror of the reference benchmark driver's kernel interface.

`kernels()` lists the registry rows (reference: `kKernels[]`, src/cuda/kernel_runner.cpp:107-181);
`run_kernel` calls one row through its `run_<kernel>` C entry point exactly as the reference driver does
(src/cuda/kernel_runner.cpp:319); `gemm` is the operator call (one asynchronous GEMM on the current stream).
All compute happens in the CUDA library; tensors are torch CUDA tensors used as device buffers only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib

ERROR_NAMES = {
    0: "ok",
    1: "misaligned operand",
    4: "invalid problem",
    5: "not supported",
    6: "workspace null / too small / misaligned",
    7: "internal error",
    8: "no such kernel",
    101: "device: producer wait timed out",
    102: "device: mma wait timed out",
    103: "device: epilogue wait timed out",
    104: "device: presum wait timed out",
    105: "device: split-tile wait timed out",
    201: "device: a flag from another GPU did not arrive in time",
}

TORCH_DTYPE = {"f16": torch.float16, "f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16}


class KernelError(RuntimeError):
    def __init__(self, kernel: str, code: int):
        self.kernel, self.code = kernel, code
        super().__init__(f"{kernel}: error {code} ({ERROR_NAMES.get(code, 'CUDA/cuBLAS error')})")


@dataclass(frozen=True)
class KernelInfo:
    name: str
    arch: str
    dtype: str
    strassen_level: int
    index: int


def normalize_arch(arch: str) -> str:
    """Reference aliases (src/cuda/kernel_runner.cpp:190-196) plus the Blackwell ones."""
    arch = arch.lower()
    if arch in ("sm70", "70", "compute_70"):
        return "volta"
    if arch in ("sm80", "80", "compute_80"):
        return "ampere"
    if arch in ("sm90", "sm90a", "90", "90a", "compute_90a"):
        return "hopper"
    if arch in ("sm100", "sm100a", "100", "100a", "compute_100a", "b200"):
        return "blackwell"
    return arch


def to_torch(x, device) -> torch.Tensor:
    """Host array -> tensor on `device` (bfloat16 arrays of the ml_dtypes package go through their bit pattern)."""
    import numpy as np

    if x.dtype.name == "bfloat16":
        return torch.from_numpy(np.ascontiguousarray(x).view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(x).to(device)


def to_numpy(t: torch.Tensor):
    """Tensor -> host array (bfloat16 as the ml_dtypes type)."""
    if t.dtype == torch.bfloat16:
        import ml_dtypes

        return t.contiguous().view(torch.int16).cpu().numpy().view(ml_dtypes.bfloat16)
    return t.cpu().numpy()


def normalize_dtype(dtype: str) -> str:
    """Reference aliases (src/cuda/kernel_runner.cpp:198-204)."""
    dtype = dtype.lower()
    if dtype in ("float", "fp32", "s"):
        return "f32"
    if dtype in ("half", "fp16", "h"):
        return "f16"
    if dtype in ("bfloat16", "bf"):
        return "bf16"
    if dtype in ("double", "fp64", "d"):
        return "f64"
    return dtype


def kernels(dtype: Optional[str] = None, level: Optional[int] = None, regex: Optional[str] = None) -> List[KernelInfo]:
    import re

    lib = _lib.load()
    out = []
    for i in range(lib.sb200_num_kernels()):
        e = lib.sb200_kernel(i).contents
        info = KernelInfo(e.name.decode(), e.arch.decode(), e.dtype.decode(), int(e.strassen_level), i)
        if dtype is not None and info.dtype != normalize_dtype(dtype):
            continue
        if level is not None and info.strassen_level != level:
            continue
        if regex is not None and not re.search(regex, info.name):
            continue
        out.append(info)
    return out


def _check_inputs(a: torch.Tensor, b: torch.Tensor):
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("operands must be CUDA tensors: this backend has no CPU path")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("expected A (m x k) and B (k x n)")
    if not (a.is_contiguous() and b.is_contiguous()):
        raise ValueError("operands must be packed row-major")
    if a.dtype != b.dtype:
        raise ValueError("A and B must have the same dtype")


def run_kernel(name: str, a: torch.Tensor, b: torch.Tensor, d: Optional[torch.Tensor] = None, warmup: int = 1,
               iterations: int = 1, split_k: int = 1, stream: Optional[torch.cuda.Stream] = None):
    """Call `run_<name>` through the C ABI.  Returns (d, avg_ms).  Raises KernelError on a nonzero return."""
    lib = _lib.load()
    _check_inputs(a, b)
    m, k = a.shape
    n = b.shape[1]
    if d is None:
        d = torch.zeros((m, n), dtype=a.dtype, device=a.device)
    fn = getattr(lib, "run_" + name, None)
    if fn is None:
        raise KernelError(name, 8)
    fn.argtypes = _lib.RUN_ARGTYPES
    fn.restype = C.c_int
    s = stream if stream is not None else torch.cuda.current_stream(a.device)
    streams = (C.c_void_p * 1)(C.c_void_p(s.cuda_stream))
    avg = C.c_float(0.0)
    buf = _lib.KernelRunnerBuffers(a.data_ptr(), b.data_ptr(), None, d.data_ptr())
    with torch.cuda.device(a.device):
        rc = fn(buf, m, n, k, warmup, iterations, streams, 1, split_k, C.byref(avg))
    if rc != 0:
        raise KernelError(name, rc)
    return d, float(avg.value)


def options(sm_limit: int = 0, no_split: bool = False, wait_limit_us: int = 0,
            drop_split_flags: bool = False) -> "_lib.GemmOptions":
    """Per-call options of the tensor-core kernels (`sb200_gemm_options`): SMs the kernels may occupy, no K-split of a
    partial last wave, the bound of the device-side waits, and the test aid that makes a split wait run out."""
    return _lib.GemmOptions(int(sm_limit), int(bool(no_split)), int(wait_limit_us), int(bool(drop_split_flags)))


def _options_key(opts) -> tuple:
    return (0, 0) if opts is None else (int(opts.sm_limit), int(opts.no_split))


class Workspace:
    """Device workspace for `gemm`, sized for one (kernel, m, n, k, options); reusable across calls of that shape."""

    def __init__(self, kernel: str, m: int, n: int, k: int, device, opts=None):
        lib = _lib.load()
        rc = lib.sb200_gemm_can_implement(kernel.encode(), m, n, k)
        if rc != 0:
            raise KernelError(kernel, rc)
        with torch.cuda.device(device):  # the layout depends on the SM count of the device that will run the call
            self.nbytes = int(lib.sb200_gemm_workspace_bytes_opt(kernel.encode(), m, n, k,
                                                                 C.byref(opts) if opts is not None else None))
        self.buf = torch.empty(self.nbytes + 256, dtype=torch.uint8, device=device)
        off = (-self.buf.data_ptr()) % 256
        self.ptr = self.buf.data_ptr() + off
        self.key = (kernel, m, n, k) + _options_key(opts)


def gemm(kernel: str, a: torch.Tensor, b: torch.Tensor, d: Optional[torch.Tensor] = None,
         workspace: Optional[Workspace] = None, check: bool = True, alpha: float = 1.0, beta: float = 0.0,
         c: Optional[torch.Tensor] = None, opts=None) -> torch.Tensor:
    """D = A @ B, or D = alpha * (A @ B) + beta * C when alpha / beta / c are given, with the named kernel;
    asynchronous on the current stream (synchronises only if `check`).  C may be D itself.  `opts` (see `options`)
    applies to the plain form only."""
    lib = _lib.load()
    _check_inputs(a, b)
    m, k = a.shape
    n = b.shape[1]
    if d is None:
        d = torch.empty((m, n), dtype=a.dtype, device=a.device)
    if workspace is None or workspace.key != (kernel, m, n, k) + _options_key(opts):
        workspace = Workspace(kernel, m, n, k, a.device, opts)
    s = torch.cuda.current_stream(a.device).cuda_stream
    scaled = alpha != 1.0 or beta != 0.0
    if scaled and opts is not None:
        raise ValueError("options are not supported together with alpha / beta")
    if scaled and beta != 0.0:
        if c is None or not c.is_cuda or not c.is_contiguous() or c.shape != d.shape or c.dtype != d.dtype:
            raise ValueError("beta != 0 needs a contiguous CUDA tensor C with the shape and dtype of D")
    with torch.cuda.device(a.device):
        if scaled:
            rc = lib.sb200_gemm_ex(kernel.encode(), alpha, a.data_ptr(), b.data_ptr(), beta,
                                   c.data_ptr() if c is not None else None, d.data_ptr(), m, n, k, workspace.ptr,
                                   workspace.nbytes, s)
        else:
            rc = lib.sb200_gemm_opt(kernel.encode(), a.data_ptr(), b.data_ptr(), d.data_ptr(), m, n, k, workspace.ptr,
                                    workspace.nbytes, s, C.byref(opts) if opts is not None else None)
        if rc != 0:
            raise KernelError(kernel, rc)
        if check:
            rc = lib.sb200_gemm_status(workspace.ptr, s)
            if rc != 0:
                raise KernelError(kernel, rc)
    return d


class HostPipeline:
    """GEMMs on operands that live in pinned host memory, with the copies overlapped with the compute: while step i
    runs its kernels, step i + 1's operands travel to the device and step i - 1's result travels back (three streams,
    two sets of device buffers, PCIe used in both directions at once).  Every step still moves all of its bytes.

        pipe = HostPipeline(kernel, m, n, k, torch.float16, device)
        for a_host, b_host, d_host in work: pipe.submit(a_host, b_host, d_host)
        pipe.finish()
    """

    def __init__(self, kernel: str, m: int, n: int, k: int, dtype: torch.dtype, device, opts=None):
        self.kernel, self.m, self.n, self.k, self.device = kernel, m, n, k, torch.device(device)
        self.opts = opts
        self.ws = Workspace(kernel, m, n, k, device, opts)
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        self.slots = [{"a": torch.empty((m, k), dtype=dtype, device=device),
                       "b": torch.empty((k, n), dtype=dtype, device=device),
                       "d": torch.empty((m, n), dtype=dtype, device=device),
                       "in": torch.cuda.Event(), "mm": torch.cuda.Event(), "out": torch.cuda.Event(), "used": False}
                      for _ in range(2)]
        self.steps = 0

    def submit(self, a_host: torch.Tensor, b_host: torch.Tensor, d_host: torch.Tensor) -> None:
        """Enqueue D = A @ B for one set of pinned host tensors; returns at once."""
        for t in (a_host, b_host, d_host):
            if t.is_cuda or not t.is_pinned() or not t.is_contiguous():
                raise ValueError("HostPipeline takes contiguous tensors in pinned host memory")
        lib = _lib.load()
        slot = self.slots[self.steps % 2]
        self.steps += 1
        if slot["used"]:
            self.s_in.wait_event(slot["mm"])    # the kernels that read this slot's operands have finished
        with torch.cuda.stream(self.s_in):
            slot["a"].copy_(a_host, non_blocking=True)
            slot["b"].copy_(b_host, non_blocking=True)
            slot["in"].record(self.s_in)
        self.s_mm.wait_event(slot["in"])
        if slot["used"]:
            self.s_mm.wait_event(slot["out"])   # the slot's previous result has left
        with torch.cuda.device(self.device):
            rc = lib.sb200_gemm_opt(self.kernel.encode(), slot["a"].data_ptr(), slot["b"].data_ptr(),
                                    slot["d"].data_ptr(), self.m, self.n, self.k, self.ws.ptr, self.ws.nbytes,
                                    self.s_mm.cuda_stream, C.byref(self.opts) if self.opts is not None else None)
        if rc != 0:
            raise KernelError(self.kernel, rc)
        slot["mm"].record(self.s_mm)
        self.s_out.wait_event(slot["mm"])
        with torch.cuda.stream(self.s_out):
            d_host.copy_(slot["d"], non_blocking=True)
            slot["out"].record(self.s_out)
        slot["used"] = True

    def join(self, stream: torch.cuda.Stream) -> None:
        """Make `stream` wait for everything submitted so far (no host synchronisation)."""
        for slot in self.slots:
            if slot["used"]:
                stream.wait_event(slot["out"])

    def finish(self) -> None:
        """Wait for everything submitted so far and check the device status word."""
        for s in (self.s_in, self.s_mm, self.s_out):
            s.synchronize()
        rc = _lib.load().sb200_gemm_status(self.ws.ptr, self.s_mm.cuda_stream)
        if rc != 0:
            raise KernelError(self.kernel, rc)


def gemm_colmajor(kernel: str, a_cm: torch.Tensor, b_cm: torch.Tensor, m: int, n: int, k: int) -> torch.Tensor:
    """Column-major problem: `a_cm` holds A (m x k) column-major, i.e. it is the contiguous (k x m) tensor A^T; `b_cm`
    likewise is the contiguous (n x k) tensor B^T.  Returns the contiguous (n x m) tensor D^T = column-major D."""
    lib = _lib.load()
    if tuple(a_cm.shape) != (k, m) or tuple(b_cm.shape) != (n, k):
        raise ValueError("column-major operands are passed as their contiguous transposes")
    _check_inputs(b_cm, a_cm)
    d = torch.empty((n, m), dtype=a_cm.dtype, device=a_cm.device)
    workspace = Workspace(kernel, n, m, k, a_cm.device)
    s = torch.cuda.current_stream(a_cm.device).cuda_stream
    with torch.cuda.device(a_cm.device):
        rc = lib.sb200_gemm_colmajor(kernel.encode(), a_cm.data_ptr(), b_cm.data_ptr(), d.data_ptr(), m, n, k,
                                     workspace.ptr, workspace.nbytes, s)
        if rc == 0:
            rc = lib.sb200_gemm_status(workspace.ptr, s)
    if rc != 0:
        raise KernelError(kernel, rc)
    return d


def gemm_host(kernel: str, a, b):
    """End-to-end call on HOST arrays (numpy): copies in, runs on the GPU, copies D back."""
    import numpy as np

    lib = _lib.load()
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[1]
    d = np.empty((m, n), dtype=a.dtype)
    rc = lib.sb200_gemm_host(kernel.encode(), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p),
                             d.ctypes.data_as(C.c_void_p), m, n, k)
    if rc != 0:
        raise KernelError(kernel, rc)
    return d
