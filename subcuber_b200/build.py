"""In-tree build of the CUDA library (sm_100a only).

    python -m subcuber_b200.build            # build libsubcuber_b200.so and the kernel_runner binary
    python -m subcuber_b200.build --force    # rebuild even if up to date

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is installed.  The outputs are
written next to this file (they are git-ignored build artefacts).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsubcuber_b200.so")
RUNNER = os.path.join(HERE, "kernel_runner")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]

LIB_SOURCES = ["sw_host.cu", "any_size.cu", "dgemm_sw.cu", "abi.cu", "fill.cu", "static_scratch.cu"]
RUNNER_SOURCES = ["kernel_runner.cpp"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build subcuber_b200")
    return nvcc


def _cuda_lib_dir(nvcc: str) -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "lib64")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _all_deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h", ".cpp", ".inc"))]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "subcuber_b200.h"))
    deps.append(os.path.abspath(__file__))
    return deps


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the shared library (and the driver binary); return the library path."""
    nvcc = _nvcc()
    libdir = _cuda_lib_dir(nvcc)
    deps = _all_deps()
    sources = [s for s in LIB_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if force or not _newer(LIB, deps):
        objs = []
        for src in sources:
            obj = os.path.join(CSRC, src.rsplit(".", 1)[0] + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
            # tuning aid: compile in-kernel cycle counters in (SB200_PROFILE=1, or KSTEP / EPILOGUE / TRACE for more)
            prof = os.environ.get("SB200_PROFILE")
            if prof:
                cmd.insert(1, "-DSB200_PROFILE" + ("" if prof == "1" else "_" + prof.upper()))
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            subprocess.run(cmd, check=True)
            objs.append(obj)
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs, "-L" + libdir, "-lcublas", "-lcublasLt", "-lcudart",
               "-Xlinker", "-rpath=" + libdir]
        subprocess.run(cmd, check=True)
    runner_srcs = [os.path.join(CSRC, s) for s in RUNNER_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if runner_srcs and (force or not _newer(RUNNER, deps + [LIB])):
        cmd = [nvcc, "-O2", "-std=c++17", *runner_srcs, "-o", RUNNER, "-L" + HERE, "-lsubcuber_b200",
               "-L" + libdir, "-lcudart", "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", "-rpath=" + libdir]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
