"""Sweep of the GEMM kernels against cuBLAS over shapes, element types and Strassen levels, one JSON line per cell.

    python -m subcuber_b200.sweep --out sweep.jsonl [--sizes 2048,4096,8192,16384] [--dtypes f16,f32,f64]
                                  [--levels 0,1,2] [--seconds 0.5] [--shapes 16384x8192x32768,...]

The reference project evaluates its kernels the same way - every kernel beside a cuBLAS-class baseline on the same
shapes, best configuration per shape (example/ampere/strassen_gemm/eval.py:41-75 there) - with a script that starts
over when interrupted.  This one is resumable: a cell whose line is already in the output file is skipped, so an
interrupted sweep continues where it stopped.

A cell is (m, n, k, dtype, level).  Both arms run through the driver ABI (`run_<kernel>`: its own CUDA events on the
stream) on the same device buffers, for about `--seconds` each after one untimed call, so the figures are steady
state under the GPU's power cap rather than the first milliseconds after an idle period.  Lines carry effective
TFLOPS = 2MNK / t for the kernel and for cuBLAS (f32 cells: the TF32 tensor-op row, which is what the kernels
compute in), their ratio, and the fraction of the nominal dense tensor peak of the type.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

KERNELS = {
    ("f16", 0): "blackwell_f16_cubic_2sm_256x256", ("f16", 1): "blackwell_f16_sw_interleaved_presum_2sm",
    ("f16", 2): "blackwell_f16_sw_level2_2sm",
    ("bf16", 0): "blackwell_bf16_cubic_2sm_256x256", ("bf16", 1): "blackwell_bf16_sw_interleaved_presum_2sm",
    ("bf16", 2): "blackwell_bf16_sw_level2_2sm",
    ("f32", 0): "blackwell_f32_cubic_2sm_256x256", ("f32", 1): "blackwell_f32_sw_interleaved_presum_2sm",
    ("f32", 2): "blackwell_f32_sw_level2_2sm",
    ("f64", 0): "blackwell_f64_cubic_dmma", ("f64", 1): "blackwell_f64_sw_level1", ("f64", 2): "blackwell_f64_sw_level2",
}
CUBLAS = {"f16": "cublas_f16", "bf16": "cublas_bf16", "f32": "cublas_tf32", "f64": "cublas_f64"}
DENSE_PEAK = {"f16": 2250.0, "bf16": 2250.0, "f32": 1125.0, "f64": 40.0}   # nominal dense TFLOP/s per B200


def cell_key(m, n, k, dtype, level) -> str:
    return f"{m}x{n}x{k}:{dtype}:L{level}"


def done_cells(path: str) -> set:
    done = set()
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                try:
                    done.add(json.loads(line)["cell"])
                except (ValueError, KeyError):
                    continue   # a line cut short by an interruption: the cell runs again
    return done


def plan_cells(sizes, shapes, dtypes, levels):
    cells = []
    for dtype in dtypes:
        for m, n, k in [(s, s, s) for s in sizes] + shapes:
            for level in levels:
                if (dtype, level) in KERNELS:
                    cells.append((m, n, k, dtype, level))
    return cells


def timed(runner, kernel, a, b, d, seconds):
    """Mean ms per call over about `seconds` of back-to-back calls, after one untimed call."""
    _, probe = runner.run_kernel(kernel, a, b, d, warmup=1, iterations=2)
    iters = max(3, int(seconds * 1e3 / max(probe, 1e-3)))
    _, ms = runner.run_kernel(kernel, a, b, d, warmup=0, iterations=iters)
    return ms, iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--sizes", default="2048,4096,8192,16384")
    ap.add_argument("--shapes", default="", help="extra MxNxK shapes, comma separated")
    ap.add_argument("--dtypes", default="f16,f32,f64")
    ap.add_argument("--levels", default="0,1,2")
    ap.add_argument("--seconds", type=float, default=0.5)
    ap.add_argument("--max-f64", type=int, default=16384, help="largest extent run in fp64 (a step takes seconds beyond)")
    args = ap.parse_args(argv)

    import torch

    from . import inputs, runner

    if not torch.cuda.is_available():
        print("the sweep needs a CUDA device: this backend has no CPU path", file=sys.stderr)
        return 2
    device = torch.device("cuda", torch.cuda.current_device())
    sizes = [int(s) for s in args.sizes.split(",") if s]
    shapes = [tuple(int(x) for x in s.lower().split("x")) for s in args.shapes.split(",") if s]
    dtypes = [runner.normalize_dtype(d) for d in args.dtypes.split(",") if d]
    levels = [int(x) for x in args.levels.split(",") if x != ""]
    done = done_cells(args.out)
    gpu = torch.cuda.get_device_name(device)
    buffers = {}
    with open(args.out, "a") as out:
        for m, n, k, dtype, level in plan_cells(sizes, shapes, dtypes, levels):
            key = cell_key(m, n, k, dtype, level)
            if key in done:
                continue
            if dtype == "f64" and max(m, n, k) > args.max_f64:
                continue
            if (m, n, k, dtype) not in buffers:
                buffers.clear()
                torch.cuda.empty_cache()
                a, b = inputs.operands(dtype, "uniform1", m, n, k, seed=1, device=device)
                buffers[(m, n, k, dtype)] = (a, b, torch.empty((m, n), dtype=a.dtype, device=device))
            a, b, d = buffers[(m, n, k, dtype)]
            kernel = KERNELS[(dtype, level)]
            line = {"cell": key, "m": m, "n": n, "k": k, "dtype": dtype, "level": level, "kernel": kernel, "gpu": gpu}
            try:
                ms, iters = timed(runner, kernel, a, b, d, args.seconds)
                blas_ms, _ = timed(runner, CUBLAS[dtype], a, b, d, args.seconds)
                flops = 2.0 * m * n * k
                tf, blas_tf = flops / (ms * 1e-3) / 1e12, flops / (blas_ms * 1e-3) / 1e12
                line.update({"ms": ms, "tflops": tf, "cublas": CUBLAS[dtype], "cublas_ms": blas_ms,
                             "cublas_tflops": blas_tf, "ratio": tf / blas_tf, "frac_of_dense_peak": tf / DENSE_PEAK[dtype],
                             "iterations": iters})
            except runner.KernelError as exc:
                line.update({"error": exc.code, "message": str(exc)})
            out.write(json.dumps(line) + "\n")
            out.flush()
            print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
