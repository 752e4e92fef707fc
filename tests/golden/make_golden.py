"""Generate tests/golden/ref_oracle_vectors.npz from the reference project's own oracle kernels.

Run on a machine that has the reference tree (it is read where it lies; `make -C oracle ref` compiles its
oracle kernel templates for the host into oracle/_ref/libref_oracle.so):

    python tests/golden/make_golden.py

Every case stores the inputs (from the seeded generator of the library, host side) and the output of
ReferenceStrassenWinogradGemm / ReferenceGemm (reference: src/cuda/strassen_reference_l1.cuh:216-251,
src/cuda/cubic_reference.cuh:42-72) at the type sets the reference harness instantiates
(tests/base_test.cuh:290).  The committed .npz lets the oracle tests run where the reference tree is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as ob  # noqa: E402
from subcuber_b200 import inputs  # noqa: E402

CASES = [
    # (dtype, level, m, n, k, dist, alpha, beta)
    ("f16", 1, 64, 48, 32, "uniform1", 1.0, 0.0),
    ("f16", 1, 96, 64, 80, "harness", 1.0, 0.0),
    ("f16", 0, 40, 24, 56, "uniform1", 1.0, 0.0),
    ("f16", 1, 33, 20, 16, "uniform1", 1.0, 0.0),   # odd M: the reference falls back to the naive kernel
    ("f32", 1, 64, 48, 32, "uniform1", 1.0, 0.0),
    ("f32", 1, 128, 32, 64, "normal", 1.0, 0.0),
    ("f32", 1, 48, 80, 24, "harness", 0.5, 2.0),    # alpha / beta with a C input
    ("f32", 0, 24, 40, 72, "normal", 1.0, 0.0),
    ("f64", 1, 64, 48, 32, "uniform1", 1.0, 0.0),
    ("f64", 1, 32, 96, 48, "normal", -1.0, 1.0),
    ("f64", 0, 16, 16, 16, "harness", 1.0, 0.0),
    # the same kernel templates instantiated for bfloat16 storage (stored as their 16-bit patterns)
    ("bf16", 1, 64, 48, 32, "uniform1", 1.0, 0.0),
    ("bf16", 1, 48, 80, 24, "harness", 0.5, 2.0),
    ("bf16", 0, 40, 24, 56, "uniform1", 1.0, 0.0),
]


def _stored(x):
    return x.view(np.uint16) if x.dtype.name == "bfloat16" else x


def main():
    ob.build(ref=True)
    if ob.ref_oracle() is None:
        raise SystemExit("oracle/_ref/libref_oracle.so is missing: the reference tree is needed to make goldens")
    out = {}
    names = []
    for idx, (dt, level, m, n, k, dist, alpha, beta) in enumerate(CASES):
        a, b = inputs.operands(dt, dist, m, n, k, seed=100 + idx)
        cin = inputs.fill_host(dt, "uniform1", (m, n), seed=100 + idx, subsequence=2) if beta != 0.0 else None
        d = ob.ref_sw_gemm(dt, level, a, b, alpha=alpha, beta=beta, Cin=cin)
        name = f"case{idx:02d}"
        names.append(name)
        out[name + "_meta"] = np.array([ob.DTYPE_CODE[dt], level, m, n, k, inputs.DIST_CODE[dist]], dtype=np.int64)
        out[name + "_ab"] = np.array([alpha, beta], dtype=np.float64)
        out[name + "_a"] = _stored(a)
        out[name + "_b"] = _stored(b)
        if cin is not None:
            out[name + "_c"] = _stored(cin)
        out[name + "_d"] = _stored(d)
    # presum dump kernel (strassen_reference_l1.cuh:119-183) for the types where it rounds like the GEMM kernel
    for dt in ("f32", "f64"):
        a, b = inputs.operands(dt, "uniform1", 32, 48, 24, seed=7)
        pa, pb = ob.ref_sw_presums(dt, a, b)
        out[f"presum_{dt}_a"] = a
        out[f"presum_{dt}_b"] = b
        out[f"presum_{dt}_pa"] = pa
        out[f"presum_{dt}_pb"] = pb
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_oracle_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(names)} gemm cases, 2 presum cases, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
