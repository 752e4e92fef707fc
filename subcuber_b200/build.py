"""In-tree build of the CUDA library (sm_100a only).

    python -m subcuber_b200.build            # build libsubcuber_b200.so and the kernel_runner binary
    python -m subcuber_b200.build --force    # rebuild even if up to date

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is installed.  The outputs are
written next to this file (they are git-ignored build artefacts).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
# builds with the in-kernel measurement aids (SB200_PROFILE in the environment) go to a library of their own, so that
# the product library never carries them
_PROFILE = os.environ.get("SB200_PROFILE", "")
LIB = os.path.join(HERE, "libsubcuber_b200_prof.so" if _PROFILE else "libsubcuber_b200.so")
RUNNER = os.path.join(HERE, "kernel_runner_prof" if _PROFILE else "kernel_runner")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]

LIB_SOURCES = ["sw_host.cu", "any_size.cu", "dgemm_sw.cu", "abi.cu", "fill.cu", "static_scratch.cu", "peer_flags.cu"]
RUNNER_SOURCES = ["kernel_runner.cpp"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build subcuber_b200")
    return nvcc


def _cuda_lib_dir(nvcc: str) -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "lib64")


STAMP = LIB + ".srchash"


def _source_hash() -> str:
    """Digest of everything the binaries are made from (file times do not survive every copy of the tree)."""
    h = hashlib.sha256()
    for d in sorted(_all_deps()):
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(os.environ.get("SB200_PROFILE", "").encode())
    return h.hexdigest()


def _all_deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h", ".cpp", ".inc"))]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "subcuber_b200.h"))
    deps.append(os.path.abspath(__file__))
    return deps


def have_nvcc() -> bool:
    return bool(shutil.which("nvcc")) or os.path.exists("/usr/local/cuda/bin/nvcc")


def up_to_date() -> bool:
    """True when the shared library and the driver exist and were built from the present sources."""
    if not (os.path.exists(LIB) and os.path.exists(RUNNER) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the shared library (and the driver binary); return the library path."""
    nvcc = _nvcc()
    libdir = _cuda_lib_dir(nvcc)
    sources = [s for s in LIB_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    stale = force or not up_to_date()
    if stale:
        objs, cmds = [], []
        for src in sources:
            obj = os.path.join(CSRC, src.rsplit(".", 1)[0] + ("_prof.o" if _PROFILE else ".o"))
            cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
            # tuning aid: compile in-kernel cycle counters in (SB200_PROFILE=1, or KSTEP / EPILOGUE / TRACE for more)
            prof = os.environ.get("SB200_PROFILE")
            if prof:
                cmd.insert(1, "-DSB200_PROFILE" + ("" if prof == "1" else "_" + prof.upper()))
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            cmds.append(cmd)
            objs.append(obj)
        # the translation units are independent: compile them side by side
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=len(cmds)) as pool:
            list(pool.map(lambda c: subprocess.run(c, check=True), cmds))
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs, "-L" + libdir, "-lcublas", "-lcublasLt", "-lcudart",
               "-Xlinker", "-rpath=" + libdir]
        subprocess.run(cmd, check=True)
    runner_srcs = [os.path.join(CSRC, s) for s in RUNNER_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if runner_srcs and stale:
        cmd = [nvcc, "-O2", "-std=c++17", *runner_srcs, "-o", RUNNER, "-L" + HERE, "-l" + os.path.basename(LIB)[3:-3],
               "-L" + libdir, "-lcudart", "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", "-rpath=" + libdir]
        subprocess.run(cmd, check=True)
    if stale:
        with open(STAMP, "w") as f:
            f.write(_source_hash() + "\n")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
