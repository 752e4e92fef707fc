"""The benchmark driver binary (csrc/kernel_runner.cpp): the command line of the reference's
src/cuda/kernel_runner.cpp (:190-220 flag forms and aliases, :240-242 usage, :297-303,335-338,377-379 table)."""
import os
import subprocess

import pytest

from subcuber_b200 import build as _build

BIN = os.path.join(os.path.dirname(_build.__file__), "kernel_runner")


@pytest.fixture(scope="module")
def binary():
    _build.build(force=False)
    assert os.path.exists(BIN)
    return BIN


def _run(binary, *args):
    return subprocess.run([binary, *args], capture_output=True, text=True, timeout=300)


def test_help_and_usage(binary):
    r = _run(binary, "--help")
    assert r.returncode == 0
    for flag in ("--m=<M>", "--dtype=f32|f16|f64", "--gpu_arch=blackwell", "--strassen_level=0|1|2|all", "--kernel_regex"):
        assert flag in r.stderr
    # missing arguments: usage again, non-zero exit
    r = _run(binary, "--m=128")
    assert r.returncode != 0 and "Usage:" in r.stderr


def test_rejects_other_architectures_and_levels(binary):
    base = ["--m=256", "--n=256", "--k=256", "--dtype=f16", "--iterations=1", "--warmup=0", "--streams=1"]
    assert _run(binary, *base, "--gpu_arch=hopper", "--strassen_level=1").returncode != 0
    assert _run(binary, *base, "--gpu_arch=blackwell", "--strassen_level=3").returncode != 0
    # a regex that matches nothing is reported, exit code 1 (kernel_runner.cpp:300-310 in the reference)
    r = _run(binary, *base, "--gpu_arch=blackwell", "--strassen_level=1", "--kernel_regex=no_such_kernel")
    assert r.returncode == 1 and "No kernels registered" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,level,expect", [
    ("f16", "1", ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_sw_fused_presum"]),
    ("half", "2", ["blackwell_f16_sw_level2_2sm"]),
    ("f32", "all", ["blackwell_f32_cubic_2sm_256x256", "blackwell_f32_sw_level2", "cublas_tf32"]),
    ("fp64", "all", ["blackwell_f64_cubic_dmma", "blackwell_f64_sw_level1", "blackwell_f64_sw_level2", "cublas_f64"]),
    ("bf16", "all", ["blackwell_bf16_cubic_2sm_256x256", "blackwell_bf16_sw_interleaved_presum_2sm",
                     "blackwell_bf16_sw_level2_2sm", "cublas_bf16"]),
    ("f16", "1", ["blackwell_f16_strassen_fused_presum_2sm"]),
])
def test_table_on_gpu(binary, dtype, level, expect):
    # both flag forms: "--flag=value" and "--flag value"; "--level" is an alias of "--strassen_level"
    r = _run(binary, "--m", "1024", "--n=1024", "--k", "1024", f"--dtype={dtype}", "--gpu_arch", "sm100",
             f"--level={level}", "--iterations=2", "--warmup=1", "--streams=1", "--json")
    assert r.returncode == 0, r.stderr
    assert r.stdout.startswith("Running ")
    assert "kernel" in r.stdout and "split_k" in r.stdout and "avg_ms" in r.stdout and "gflops" in r.stdout
    for name in expect:
        rows = [ln for ln in r.stdout.splitlines() if ln.startswith(name + " ")]
        assert rows and "skipped" not in rows[0], name
    assert "Best kernel" in r.stdout or "best" in r.stdout.lower()


@pytest.mark.gpu
def test_sizes_off_the_tile_grid_on_gpu(binary):
    """Every positive size runs: short last blocks, and rows off the 16-byte grid through padded copies."""
    r = _run(binary, "--m=1001", "--n=1037", "--k=523", "--dtype=f16", "--gpu_arch=blackwell", "--level=all",
             "--iterations=2", "--warmup=1", "--streams=1", "--kernel_regex=blackwell")
    assert r.returncode == 0, r.stderr
    rows = [ln for ln in r.stdout.splitlines() if ln.startswith("blackwell_f16_")]
    assert len(rows) >= 10 and not any("skipped" in ln for ln in rows)
