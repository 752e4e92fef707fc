"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Tolerances follow the reference harness (tests/base_test.cuh:85-117 in the reference project): an element
passes if abs <= tol_abs OR rel <= tol_rel; f32: 1e-4 / 1e-4, f16: abs 4 (level 1), rel 1e-2.  On the harness'
own value set (multiples of 0.25) every partial sum is exactly representable, so the comparison there is
BIT-EXACT.  On uniform[-1,1) inputs the gate is the one the path's specification states: relative Frobenius
error against an fp64 product no worse than 1.5x the error of the reference's own level-1 routine (the CPU
oracle at the harness' types) on the same inputs.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

L1_F16 = ["blackwell_f16_sw_interleaved_presum", "blackwell_f16_sw_fused_presum",
          "blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_sw_fused_presum_2sm",
          "blackwell_f16_sw_merged_presum_2sm"]
L1_F32 = ["blackwell_f32_sw_interleaved_presum", "blackwell_f32_sw_fused_presum",
          "blackwell_f32_sw_interleaved_presum_2sm", "blackwell_f32_sw_fused_presum_2sm",
          "blackwell_f32_sw_merged_presum_2sm"]
L2_F16 = ["blackwell_f16_sw_level2", "blackwell_f16_sw_level2_2sm"]
L2_F32 = ["blackwell_f32_sw_level2", "blackwell_f32_sw_level2_2sm"]
# Strassen's original algorithm: the same products of blocks summed another way, checked against the same oracle
STRASSEN_F16 = ["blackwell_f16_strassen_fused_presum", "blackwell_f16_strassen_fused_presum_2sm",
                "blackwell_f16_strassen_presum_2sm"]
STRASSEN_F32 = ["blackwell_f32_strassen_fused_presum", "blackwell_f32_strassen_fused_presum_2sm",
                "blackwell_f32_strassen_presum_2sm"]
# bfloat16 storage: the f16 kernels with the other 16-bit format
BF16 = ["blackwell_bf16_cubic_128x256", "blackwell_bf16_cubic_2sm_256x256", "blackwell_bf16_sw_fused_presum_2sm",
        "blackwell_bf16_sw_interleaved_presum", "blackwell_bf16_sw_interleaved_presum_2sm",
        "blackwell_bf16_sw_merged_presum_2sm"]
L2_BF16 = ["blackwell_bf16_sw_level2", "blackwell_bf16_sw_level2_2sm"]
L0_F16 = ["blackwell_f16_cubic_128x256", "blackwell_f16_cubic_128x128", "blackwell_f16_cubic_2sm_256x256"]
L0_F32 = ["blackwell_f32_cubic_128x256", "blackwell_f32_cubic_128x128", "blackwell_f32_cubic_2sm_256x256"]


def _dt(kernel):
    if "_bf16_" in kernel:
        return "bf16"
    return "f16" if "_f16_" in kernel else ("f64" if "_f64_" in kernel else "f32")


def _level(kernel):
    return 0 if "cubic" in kernel else (2 if "level2" in kernel else 1)


def _run(kernel, a_np, b_np, device, opts=None):
    import torch

    from subcuber_b200 import runner

    a = runner.to_torch(a_np, device)
    b = runner.to_torch(b_np, device)
    d = torch.full((a.shape[0], b.shape[1]), float("nan"), dtype=a.dtype, device=device)
    runner.gemm(kernel, a, b, d, opts=opts)
    torch.cuda.synchronize()
    return runner.to_numpy(d)


def _rel_fro(x, truth):
    return float(np.linalg.norm(x.astype(np.float64) - truth) / np.linalg.norm(truth))


# --------------------------------------------------------------------------------------------- bit-exact
SMALL_SHAPES = [(256, 512, 128), (384, 768, 320), (272, 528, 144), (2, 16, 16), (130, 48, 80), (1024, 1024, 1024)]


@pytest.mark.parametrize("kernel", L0_F16 + L0_F32 + L1_F16 + L1_F32 + STRASSEN_F16 + STRASSEN_F32 + BF16)
@pytest.mark.parametrize("shape", SMALL_SHAPES)
def test_bit_exact_on_harness_values(kernel, shape, oracle, cuda_device):
    from subcuber_b200 import inputs

    m, n, k = shape
    dt = _dt(kernel)
    a, b = inputs.operands(dt, "harness", m, n, k, seed=m + n + k)
    got = _run(kernel, a, b, cuda_device)
    want = oracle.sw_gemm(dt, _level(kernel), a, b)
    assert not np.isnan(got.astype(np.float32)).any()
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} elements differ from the oracle"
    truth = a.astype(np.float64) @ b.astype(np.float64)
    if dt == "f32":
        assert np.array_equal(got.astype(np.float64), truth)


@pytest.mark.parametrize("kernel", L2_F16 + L2_F32 + L2_BF16)
@pytest.mark.parametrize("shape", [(512, 1024, 256), (544, 1056, 288), (4, 32, 32), (260, 96, 160), (1024, 1024, 512),
                                   (2048, 1536, 512)])
def test_level2_bit_exact_on_harness_values(kernel, shape, oracle, cuda_device):
    """49 products as seven chained level-1 groups.  On the harness' value set every presum of both recursion steps
    (at most 16 terms of magnitude <= 4 in steps of 0.25) and every partial sum is exact, so the result equals the
    oracle's level-2 recursion bit for bit, whatever the order of the additions."""
    from subcuber_b200 import inputs

    m, n, k = shape
    dt = _dt(kernel)
    a, b = inputs.operands(dt, "harness", m, n, k, seed=m + n + k)
    got = _run(kernel, a, b, cuda_device)
    want = oracle.sw_gemm(dt, 2, a, b)
    assert not np.isnan(got.astype(np.float32)).any()
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} elements differ from the oracle"
    if dt == "f32":
        assert np.array_equal(got.astype(np.float64), a.astype(np.float64) @ b.astype(np.float64))


# ------------------------------------------------------------------------- alpha / beta / C, column-major
SCALED_KERNELS = ["blackwell_f16_cubic_2sm_256x256", "blackwell_f16_sw_interleaved_presum_2sm",
                  "blackwell_f16_sw_interleaved_presum", "blackwell_f32_sw_interleaved_presum_2sm",
                  "blackwell_f16_sw_level2_2sm", "blackwell_f32_sw_level2", "blackwell_f64_cubic_dmma",
                  "blackwell_f64_sw_level1", "blackwell_f64_sw_level2"]


@pytest.mark.parametrize("kernel", SCALED_KERNELS)
@pytest.mark.parametrize("alpha,beta", [(2.0, -0.5), (-1.0, 0.0), (0.5, 1.0)])
def test_alpha_beta_bit_exact_on_harness_values(kernel, alpha, beta, oracle, cuda_device):
    """D = alpha * A B + beta * C, the reference operators' general form (strassen_gemm.h:365-451): on the harness'
    value set and with power-of-two scales every sum stays exact, so the result equals the oracle's bit for bit."""
    import torch

    from subcuber_b200 import inputs, runner

    m, n, k = (528, 1056, 288) if _level(kernel) == 2 else (272, 528, 144)
    dt = _dt(kernel)
    a_np, b_np = inputs.operands(dt, "harness", m, n, k, seed=17)
    c_np = inputs.operands(dt, "harness", m, n, n, seed=18)[0]   # an m x n matrix of the same value set
    a, b, c = (torch.from_numpy(x).to(cuda_device) for x in (a_np, b_np, c_np))
    d = runner.gemm(kernel, a, b, alpha=alpha, beta=beta, c=c)
    torch.cuda.synchronize()
    want = oracle.sw_gemm(dt, _level(kernel), a_np, b_np, alpha=alpha, beta=beta, Cin=c_np)
    assert np.array_equal(d.cpu().numpy(), want)
    if beta != 0.0:  # in place: C and D the same buffer
        d2 = runner.gemm(kernel, a, b, d=c, alpha=alpha, beta=beta, c=c)
        torch.cuda.synchronize()
        assert np.array_equal(d2.cpu().numpy(), want)


# ----------------------------------------------------------------- extents that do not divide into blocks
def _padded_oracle(oracle, dt, level, a, b, alpha=1.0, beta=0.0, cin=None):
    """The oracle on the zero-padded problem the kernels compute: rows are padded to 16 bytes (fp64: extents to a
    multiple of the block count, 16-byte aligned block rows), then the matrices are cut at multiples of the block
    extents (m: ceil(m / blocks); n, k: the same rounded up to 16 bytes) and the short last blocks read as zeros."""
    m, k = a.shape
    n = b.shape[1]
    div = 1 << level
    vec = 16 // a.dtype.itemsize
    up = lambda x, g: -(-x // g) * g
    if dt == "f64":
        mp, np_, kp = up(m, div), up(n, div * vec), up(k, div * vec)
    else:
        mp, np_, kp = div * (-(-m // div)), div * up(-(-up(n, vec) // div), vec), div * up(-(-up(k, vec) // div), vec)
    ap = np.zeros((mp, kp), dtype=a.dtype); ap[:m, :k] = a
    bp = np.zeros((kp, np_), dtype=b.dtype); bp[:k, :n] = b
    cp = None
    if cin is not None:
        cp = np.zeros((mp, np_), dtype=cin.dtype); cp[:m, :n] = cin
    return oracle.sw_gemm(dt, level, ap, bp, alpha=alpha, beta=beta, Cin=cp)[:m, :n]


RAGGED_KERNELS = ["blackwell_f16_sw_interleaved_presum", "blackwell_f16_sw_interleaved_presum_2sm",
                  "blackwell_f16_sw_fused_presum_2sm", "blackwell_f32_sw_interleaved_presum_2sm",
                  "blackwell_f32_sw_fused_presum", "blackwell_f16_sw_level2", "blackwell_f16_sw_level2_2sm",
                  "blackwell_f32_sw_level2_2sm", "blackwell_f16_cubic_2sm_256x256", "blackwell_f64_cubic_dmma",
                  "blackwell_f64_sw_level1", "blackwell_f64_sw_level2", "blackwell_f16_strassen_fused_presum_2sm",
                  "blackwell_f32_strassen_fused_presum"]
# rows on the 16-byte grid (short last blocks only), and rows off it (zero-padded copies, then short blocks)
RAGGED_SHAPES = [(255, 520, 136), (1001, 776, 264), (131, 264, 200), (257, 517, 129), (1023, 1030, 515)]


@pytest.mark.parametrize("kernel", RAGGED_KERNELS)
@pytest.mark.parametrize("shape", RAGGED_SHAPES)
def test_any_extents_bit_exact_on_harness_values(kernel, shape, oracle, cuda_device):
    """Extents that do not divide into 2 (4) blocks per dimension, and rows that do not start on 16 bytes: the
    kernels compute the zero-padded problem, whose product is the product.  Exact on the harness' value set."""
    from subcuber_b200 import inputs

    m, n, k = shape
    dt = _dt(kernel)
    a, b = inputs.operands(dt, "harness", m, n, k, seed=m + n + k)
    got = _run(kernel, a, b, cuda_device)
    assert not np.isnan(got).any()
    want = _padded_oracle(oracle, dt, _level(kernel), a, b)
    assert np.array_equal(got, want), f"{np.count_nonzero(got != want)} elements differ from the oracle"
    assert np.array_equal(got, oracle.sw_gemm(dt, 0, a, b))  # and equals the plain product of the unpadded operands


@pytest.mark.parametrize("kernel", ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_sw_level2_2sm",
                                    "blackwell_f32_sw_interleaved_presum", "blackwell_f64_sw_level1"])
@pytest.mark.parametrize("shape", [(1001, 776, 264), (517, 1030, 259)])
def test_any_extents_alpha_beta(kernel, shape, oracle, cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    m, n, k = shape
    dt = _dt(kernel)
    a_np, b_np = inputs.operands(dt, "harness", m, n, k, seed=21)
    c_np = np.ascontiguousarray(inputs.operands(dt, "harness", m, n + 8, n + 8, seed=22)[0][:, :n])
    a, b, c = (torch.from_numpy(x).to(cuda_device) for x in (a_np, b_np, c_np))
    d = runner.gemm(kernel, a, b, alpha=2.0, beta=-0.5, c=c)
    torch.cuda.synchronize()
    want = _padded_oracle(oracle, dt, _level(kernel), a_np, b_np, alpha=2.0, beta=-0.5, cin=c_np)
    assert np.array_equal(d.cpu().numpy(), want)


@pytest.mark.parametrize("kernel", ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_sw_level2_2sm",
                                    "blackwell_f16_sw_interleaved_presum"])
@pytest.mark.parametrize("shape", [(1537, 1288, 1032), (1025, 2051, 1283)])
def test_any_extents_uniform_inputs_f16(kernel, shape, oracle, cuda_device):
    """Inexact inputs: the error gate against the reference routine on the padded problem."""
    from subcuber_b200 import inputs

    m, n, k = shape
    a, b = inputs.operands("f16", "uniform1", m, n, k, seed=9)
    got = _run(kernel, a, b, cuda_device)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    ref = _padded_oracle(oracle, "f16", _level(kernel), a, b)
    assert _rel_fro(got, truth) <= 1.5 * _rel_fro(ref, truth)


def test_any_extents_column_major_and_auto(oracle, cuda_device):
    """The column-major entry point and the size-based kernel choice take the same sizes."""
    import torch

    from subcuber_b200 import inputs, runner

    m, n, k = 515, 1001, 264
    a, b = inputs.operands("f16", "harness", m, n, k, seed=12)
    want = oracle.sw_gemm("f16", 0, a, b)
    a_cm = torch.from_numpy(np.ascontiguousarray(a.T)).to(cuda_device)   # k x m: A stored column-major
    b_cm = torch.from_numpy(np.ascontiguousarray(b.T)).to(cuda_device)
    d_cm = runner.gemm_colmajor("blackwell_f16_sw_interleaved_presum_2sm", a_cm, b_cm, m, n, k)
    torch.cuda.synchronize()
    assert np.array_equal(d_cm.cpu().numpy().T, want)
    got = _run("blackwell_f16_sw_auto", a, b, cuda_device)
    assert np.array_equal(got, want)


def test_any_extents_split_last_wave(oracle, cuda_device):
    from subcuber_b200 import inputs, runner

    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    m, n, k = 1001, 2568, 1160
    a, b = inputs.operands("f16", "harness", m, n, k, seed=4)
    got = _run(kernel, a, b, cuda_device, runner.options(sm_limit=16))
    assert np.array_equal(got, oracle.sw_gemm("f16", 0, a, b))


def test_scaled_form_is_refused_where_it_is_not_built(cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    a_np, b_np = inputs.operands("f16", "harness", 256, 256, 128, seed=1)
    a, b = torch.from_numpy(a_np).to(cuda_device), torch.from_numpy(b_np).to(cuda_device)
    with pytest.raises(runner.KernelError):
        runner.gemm("blackwell_f16_sw_fused_presum", a, b, alpha=2.0)   # fused-presum plan: D = A B only
    with pytest.raises(ValueError):
        runner.gemm("blackwell_f16_cubic_2sm_256x256", a, b, beta=1.0)  # beta without C


@pytest.mark.parametrize("kernel", ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f64_sw_level1",
                                    "blackwell_f32_cubic_2sm_256x256"])
def test_column_major_operands(kernel, cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    m, n, k = 384, 272, 528
    dt = _dt(kernel)
    a_np, b_np = inputs.operands(dt, "harness", m, n, k, seed=23)
    a_cm = torch.from_numpy(np.ascontiguousarray(a_np.T)).to(cuda_device)   # column-major A = contiguous A^T
    b_cm = torch.from_numpy(np.ascontiguousarray(b_np.T)).to(cuda_device)
    d_cm = runner.gemm_colmajor(kernel, a_cm, b_cm, m, n, k)
    torch.cuda.synchronize()
    want = a_np.astype(np.float64) @ b_np.astype(np.float64)
    assert np.array_equal(d_cm.cpu().numpy().T.astype(np.float64), want.astype(a_np.dtype).astype(np.float64))


def test_auto_kernel_runs_the_kernel_it_names(lib, cuda_device):
    import ctypes as C

    import torch

    from subcuber_b200 import inputs, runner

    lib.sb200_auto_kernel.restype = C.c_char_p
    lib.sb200_auto_kernel.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int]
    for dt, (m, n, k) in (("f16", (512, 768, 256)), ("f64", (256, 384, 128))):
        a_np, b_np = inputs.operands(dt, "harness", m, n, k, seed=31)
        a, b = torch.from_numpy(a_np).to(cuda_device), torch.from_numpy(b_np).to(cuda_device)
        d = runner.gemm(f"blackwell_{dt}_sw_auto", a, b)
        named = lib.sb200_auto_kernel(dt.encode(), m, n, k).decode()
        ref = runner.gemm(named, a, b)
        torch.cuda.synchronize()
        assert torch.equal(d, ref)


# ------------------------------------------------------------------------------------------ fp64 (DMMA)
F64 = ["blackwell_f64_cubic_dmma", "blackwell_f64_sw_level1", "blackwell_f64_sw_level2"]


@pytest.mark.parametrize("kernel", F64)
@pytest.mark.parametrize("shape", [(256, 512, 128), (384, 768, 320), (264, 520, 136), (4, 16, 16), (132, 48, 80),
                                   (1024, 1024, 512)])
def test_f64_bit_exact_on_harness_values(kernel, shape, oracle, cuda_device):
    from subcuber_b200 import inputs

    m, n, k = shape
    level = {"cubic": 0, "level1": 1, "level2": 2}[kernel.rsplit("_", 1)[-1].replace("dmma", "cubic")]
    a, b = inputs.operands("f64", "harness", m, n, k, seed=m + n + k)
    got = _run(kernel, a, b, cuda_device)
    assert not np.isnan(got).any()
    assert np.array_equal(got, a @ b)                      # every sum is exact on this value set
    assert np.array_equal(got, oracle.sw_gemm("f64", level, a, b))


@pytest.mark.parametrize("kernel", F64)
@pytest.mark.parametrize("dist", ["uniform1", "normal"])
def test_f64_uniform_inputs(kernel, dist, oracle, cuda_device):
    """fp64 throughout: the result differs from the reference routine only by the order of fp64 additions, and its
    error against a higher-precision product stays within 1.5x the routine's."""
    from subcuber_b200 import inputs

    m, n, k = 768, 1280, 1024
    level = {"cubic": 0, "level1": 1, "level2": 2}[kernel.rsplit("_", 1)[-1].replace("dmma", "cubic")]
    a, b = inputs.operands("f64", dist, m, n, k, seed=12)
    got = _run(kernel, a, b, cuda_device)
    truth = (a.astype(np.longdouble) @ b.astype(np.longdouble)).astype(np.float64)
    ref = oracle.sw_gemm("f64", level, a, b)
    err, ref_err = _rel_fro(got, truth), _rel_fro(ref, truth)
    assert err <= 1.5 * ref_err + 1e-17, f"{err:.3e} vs reference routine {ref_err:.3e}"
    assert np.allclose(got, ref, rtol=1e-11, atol=1e-11)


def test_f64_agrees_with_cublas(cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    a = inputs.fill_device("f64", "uniform1", (1024, 768), 3, 0, cuda_device)
    b = inputs.fill_device("f64", "uniform1", (768, 1536), 3, 1, cuda_device)
    d = runner.gemm("blackwell_f64_sw_level2", a, b)
    ref, _ = runner.run_kernel("cublas_f64", a, b, warmup=0, iterations=1)
    torch.cuda.synchronize()
    assert torch.allclose(d, ref, rtol=1e-11, atol=1e-11)


# ------------------------------------------------------------------------------- K-split of the last wave
SPLIT_CASES = [
    # CTA pairs draw whole tiles (nothing is cut): these check that their drawn order gives the same bits
    ("blackwell_f16_sw_interleaved_presum_2sm", 8, (512, 2560, 2048)),  # quadrant 1 x 5 pair tiles drawn by 4 pairs
    ("blackwell_f16_cubic_2sm_256x256", 16, (1024, 768, 1024)),          # 4 x 3 pair tiles drawn by 8 pairs
    ("blackwell_f16_sw_merged_presum_2sm", 8, (1536, 2560, 2048)),       # quadrant 3 x 5 pair tiles drawn by 4 pairs
    ("blackwell_f32_sw_merged_presum_2sm", 0, (4608, 5120, 1024)),       # quadrant 9 x 10 = 90 pair tiles on 74 pairs
    ("blackwell_f16_sw_level2_2sm", 8, (1024, 5120, 4096)),              # every group: 1 x 5 pair tiles drawn by 4 pairs
    # kernel, SMs, shape: the tile count leaves a last wave at most half full, whose tiles are split in two K-halves
    ("blackwell_f16_cubic_128x256", 8, (384, 768, 1024)),              # 3 x 3 = 9 tiles on 8 CTAs
    ("blackwell_f16_cubic_2sm_256x256", 8, (512, 640, 1024)),          # 2 x 3 = 6 pair tiles on 4 pairs... 2 left
    ("blackwell_f32_cubic_2sm_256x256", 8, (1280, 256, 512)),          # 5 tiles on 4 pairs
    ("blackwell_f16_sw_interleaved_presum", 8, (768, 1536, 2048)),     # quadrant 3 x 3 tiles on 8 CTAs
    ("blackwell_f16_sw_interleaved_presum_2sm", 8, (512, 2560, 1024)),  # quadrant 1 x 5 pair tiles on 4 pairs
    ("blackwell_f32_sw_interleaved_presum_2sm", 12, (3584, 512, 1024)),  # quadrant 7 x 1 on 6 pairs
    ("blackwell_f16_sw_level2_2sm", 8, (1024, 5120, 2048)),            # every group: 1 x 5 pair tiles on 4 pairs
    ("blackwell_f32_sw_level2", 8, (1536, 3072, 1024)),                # every group: 3 x 3 tiles on 8 CTAs
    ("blackwell_f16_sw_level2", 0, (5120, 15360, 2048)),               # all SMs: 10 x 15 = 150 tiles on 148 CTAs
]


@pytest.mark.parametrize("kernel,sms,shape", SPLIT_CASES)
def test_split_last_wave_bit_exact_on_harness_values(kernel, sms, shape, oracle, cuda_device):
    from subcuber_b200 import inputs, runner

    m, n, k = shape
    dt = _dt(kernel)
    level = _level(kernel)
    a, b = inputs.operands(dt, "harness", m, n, k, seed=4)
    got = _run(kernel, a, b, cuda_device, runner.options(sm_limit=sms))
    unsplit = _run(kernel, a, b, cuda_device, runner.options(sm_limit=sms, no_split=True))
    assert not np.isnan(got).any()
    assert np.array_equal(got, unsplit)
    if m * n * k <= 2 ** 34:
        assert np.array_equal(got, oracle.sw_gemm(dt, level, a, b))
    else:
        rows = np.arange(0, m, 97, dtype=np.int32)
        assert np.array_equal(got[rows], oracle.sw_gemm(dt, 0, a, b, rows=rows)[rows])


@pytest.mark.parametrize("kernel", ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_sw_level2_2sm"])
def test_split_last_wave_uniform_inputs(kernel, oracle, cuda_device):
    """On inexact inputs the split changes only the order of fp32 additions: the result stays within the error gate."""
    from subcuber_b200 import inputs, runner

    m, n, k = (512, 2560, 1024) if _level(kernel) == 1 else (1024, 5120, 2048)
    a, b = inputs.operands("f16", "uniform1", m, n, k, seed=6)
    got = _run(kernel, a, b, cuda_device, runner.options(sm_limit=8))
    truth = a.astype(np.float64) @ b.astype(np.float64)
    ref = oracle.sw_gemm("f16", _level(kernel), a, b)
    assert _rel_fro(got, truth) <= 1.5 * _rel_fro(ref, truth)


@pytest.mark.parametrize("kernel", L2_F16)
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (1536, 1280, 2304)])
def test_level2_uniform_inputs_f16(kernel, shape, oracle, cuda_device):
    """Error gate at level 2: no worse than 1.5x the level-1 routine applied recursively with interim results rounded
    to the output type at every hop, which is what the reference's level-2 operator does
    (include/cutlass/gemm/device/strassen_gemm.h:1807-1914); this path keeps the interim sums in fp32."""
    from subcuber_b200 import inputs

    m, n, k = shape
    a, b = inputs.operands("f16", "uniform1", m, n, k, seed=9)
    got = _run(kernel, a, b, cuda_device)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    ref = oracle.sw_gemm("f16", 2, a, b, interim_round=True)
    ref32 = oracle.sw_gemm("f16", 2, a, b)
    err, ref_err, ref32_err = _rel_fro(got, truth), _rel_fro(ref, truth), _rel_fro(ref32, truth)
    assert err <= 1.5 * ref_err, f"rel. Frobenius error {err:.3e} vs reference routine {ref_err:.3e}"
    assert err <= 1.5 * ref32_err, f"rel. Frobenius error {err:.3e} vs fp32-interim recursion {ref32_err:.3e}"
    diff = np.abs(got.astype(np.float64) - ref32.astype(np.float64))
    assert ((diff <= 7.0) | (diff <= 1e-2 * np.abs(ref32.astype(np.float64)))).all()


@pytest.mark.parametrize("kernel", L2_F32)
def test_level2_uniform_inputs_tf32(kernel, oracle, cuda_device):
    from subcuber_b200 import inputs

    m, n, k = 1024, 768, 1280
    a, b = inputs.operands("f32", "normal", m, n, k, seed=8)
    got = _run(kernel, a, b, cuda_device)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    model = oracle.sw_gemm("tf32", 2, a, b)
    err, model_err = _rel_fro(got, truth), _rel_fro(model, truth)
    assert err <= 4.0 * model_err + 1e-6, f"{err:.3e} vs TF32 model {model_err:.3e}"
    assert err < 6e-3


@pytest.mark.parametrize("kernel", L1_F16 + L1_F32)
@pytest.mark.parametrize("shape", [(2048, 2048, 2048), (6144, 2560, 2048), (2048, 4096, 6144)])
def test_bit_exact_on_harness_values_reference_shapes(kernel, shape, oracle, cuda_device):
    """Shapes of the reference's own gtest lists (tests/f32_strassen_winograd_tile.cu:22-34), row-sampled."""
    from subcuber_b200 import inputs

    m, n, k = shape
    dt = _dt(kernel)
    a, b = inputs.operands(dt, "harness", m, n, k, seed=3)
    got = _run(kernel, a, b, cuda_device)
    rows = np.array([0, 1, 127, 128, m // 4 + 5, m // 2 - 1], dtype=np.int32)
    want = oracle.sw_gemm(dt, 1, a, b, rows=rows)
    for r in rows:
        assert np.array_equal(got[r], want[r]) and np.array_equal(got[r + m // 2], want[r + m // 2])
    # whole-matrix check that does not depend on the size: sum of all elements = colsum(A) . rowsum(B)
    if dt == "f32":
        total = float(a.astype(np.float64).sum(axis=0) @ b.astype(np.float64).sum(axis=1))
        assert float(got.astype(np.float64).sum()) == total


# ------------------------------------------------------------------------------------- presum workspace
@pytest.mark.parametrize("kernel", ["blackwell_f16_sw_interleaved_presum", "blackwell_f32_sw_interleaved_presum",
                                    "blackwell_f16_sw_interleaved_presum_2sm"])
@pytest.mark.parametrize("shape", [(256, 512, 128), (272, 528, 144), (1024, 768, 512)])
def test_presum_workspace_bit_exact(kernel, shape, oracle, lib, cuda_device):
    """The eight presums the first launch materialises equal the oracle's, bit for bit, on uniform inputs."""
    import torch

    from subcuber_b200 import _lib as L
    from subcuber_b200 import inputs, runner

    m, n, k = shape
    dt = _dt(kernel)
    a_np, b_np = inputs.operands(dt, "uniform1", m, n, k, seed=21)
    a = torch.from_numpy(a_np).to(cuda_device)
    b = torch.from_numpy(b_np).to(cuda_device)
    ws = runner.Workspace(kernel, m, n, k, cuda_device)
    runner.gemm(kernel, a, b, workspace=ws)
    torch.cuda.synchronize()
    lay = L.WorkspaceLayout()
    assert lib.sb200_gemm_workspace_layout(kernel.encode(), m, n, k, C.byref(lay)) == 0
    off = ws.ptr - ws.buf.data_ptr()
    raw = ws.buf.cpu().numpy()
    npd = oracle.NP_DTYPE[dt]
    es = np.dtype(npd).itemsize
    pa = raw[off + lay.presum_a: off + lay.presum_a + 4 * lay.mq * lay.kq * es].view(npd).reshape(4, lay.mq, lay.kq)
    pb = raw[off + lay.presum_b: off + lay.presum_b + 4 * lay.kq * lay.nq * es].view(npd).reshape(4, lay.kq, lay.nq)
    want_a, want_b = oracle.sw_presums(dt, a_np, b_np)
    assert np.array_equal(pa, want_a)
    assert np.array_equal(pb, want_b)


# ------------------------------------------------------------------------------------------ tolerances
def _harness_tol(dt, level):
    if dt == "f16":
        return (4.0 if level == 1 else 7.0), 1e-2
    return 1e-4, 1e-4


@pytest.mark.parametrize("kernel", L1_F16 + L0_F16 + STRASSEN_F16)
@pytest.mark.parametrize("shape", [(512, 512, 512), (1024, 1024, 1024), (1536, 640, 1152)])
def test_uniform_inputs_f16(kernel, shape, oracle, cuda_device):
    from subcuber_b200 import inputs

    m, n, k = shape
    a, b = inputs.operands("f16", "uniform1", m, n, k, seed=5)
    got = _run(kernel, a, b, cuda_device)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    level = _level(kernel)
    ref = oracle.sw_gemm("f16", level, a, b)
    err, ref_err = _rel_fro(got, truth), _rel_fro(ref, truth)
    assert err <= 1.5 * ref_err, f"rel. Frobenius error {err:.3e} vs reference routine {ref_err:.3e}"
    tol_abs, tol_rel = _harness_tol("f16", max(level, 1))
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    ok = (diff <= tol_abs) | (diff <= tol_rel * np.abs(ref.astype(np.float64)))
    assert ok.all()
    if level == 0:
        assert np.allclose(got.astype(np.float64), truth, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("kernel", L1_F32 + L0_F32 + STRASSEN_F32)
@pytest.mark.parametrize("dist", ["uniform1", "normal"])
def test_uniform_inputs_tf32(kernel, dist, oracle, cuda_device):
    """fp32 storage with TF32 tensor-core math: the reference has no TF32 oracle; the CPU model rounds every
    multiplicand to TF32 (error ~ 2^-11 per operand, zero mean).  The tensor core reads the upper 19 bits,
    i.e. truncates (error up to 2^-10 per operand, one sign), so the bound is 4x that model's error, and the
    result must also sit within TF32 distance of the fp64 product."""
    from subcuber_b200 import inputs

    m, n, k = 1024, 768, 1280
    a, b = inputs.operands("f32", dist, m, n, k, seed=8)
    got = _run(kernel, a, b, cuda_device)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    model = oracle.sw_gemm("tf32", _level(kernel), a, b)
    err, model_err = _rel_fro(got, truth), _rel_fro(model, truth)
    assert err <= 4.0 * model_err + 1e-6, f"{err:.3e} vs TF32 model {model_err:.3e}"
    assert err < 3e-3


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("shape", [(2048, 2048, 2048), (1001, 2568, 1160), (4096, 1536, 3072)])
def test_strassen_presum_plan_equals_the_fused_plan(dtype, shape, cuda_device):
    """Strassen's original algorithm on materialised presums (a launch that only forms the ten presums, then the seven
    products) runs the tile program of the fused plan on operand values that are the same bit for bit (fp32 sum of two
    raw values, one rounding), so the two plans agree exactly on any input."""
    from subcuber_b200 import inputs

    m, n, k = shape
    a, b = inputs.operands(dtype, "uniform1", m, n, k, seed=21)
    fused = _run(f"blackwell_{dtype}_strassen_fused_presum_2sm", a, b, cuda_device)
    fast = _run(f"blackwell_{dtype}_strassen_presum_2sm", a, b, cuda_device)
    assert np.array_equal(fused, fast), f"{np.count_nonzero(fused != fast)} elements differ"
    again = _run(f"blackwell_{dtype}_strassen_presum_2sm", a, b, cuda_device)
    assert np.array_equal(fast, again)


# ----------------------------------------------------------------------------------------- full size
@pytest.mark.parametrize("kernel,size", [("blackwell_f16_sw_interleaved_presum", 8192),
                                         ("blackwell_f16_sw_interleaved_presum_2sm", 8192),
                                         ("blackwell_f16_sw_merged_presum_2sm", 8192),
                                         ("blackwell_f16_cubic_128x256", 8192),
                                         ("blackwell_f32_sw_interleaved_presum", 4096)])
def test_full_size_properties(kernel, size, oracle, cuda_device):
    """The benchmark workload itself (f16, level 1, 8192^3): sampled rows against fp64 and against the
    reference routine, plus the checksum identity sum(C) = colsum(A) . rowsum(B) over the whole matrix."""
    import torch

    from subcuber_b200 import inputs, runner

    dt = _dt(kernel)
    a = inputs.fill_device(dt, "uniform1", (size, size), 1, 0, cuda_device)
    b = inputs.fill_device(dt, "uniform1", (size, size), 1, 1, cuda_device)
    d = runner.gemm(kernel, a, b)
    torch.cuda.synchronize()
    total_dev = float(d.double().sum())
    total = float(a.double().sum(dim=0) @ b.double().sum(dim=1))
    scale = float((a.double().abs().sum(dim=0) @ b.double().abs().sum(dim=1)))
    assert abs(total_dev - total) <= 2e-5 * scale
    a_np, b_np = a.cpu().numpy(), b.cpu().numpy()
    rows = np.array([0, 77, size // 4, size // 2 - 1], dtype=np.int32)
    all_rows = np.concatenate([rows, rows + size // 2])
    truth = oracle.truth_rows(dt, a_np, b_np, all_rows)
    got = d[torch.from_numpy(all_rows).long().to(cuda_device)].cpu().numpy()
    if dt == "f16":
        level = _level(kernel)
        ref = oracle.sw_gemm("f16", level, a_np, b_np, rows=(rows if level else all_rows))[all_rows]
        err, ref_err = _rel_fro(got, truth), _rel_fro(ref, truth)
        assert err <= 1.5 * ref_err, f"{err:.3e} vs reference routine {ref_err:.3e}"
    else:
        assert _rel_fro(got, truth) < 3e-3


def _checksum_ok(a, b, d, tol):
    """sum(D) = colsum(A) . rowsum(B) over the whole matrix, in double on the device."""
    total_dev = float(d.double().sum())
    total = float(a.double().sum(dim=0) @ b.double().sum(dim=1))
    scale = float(a.double().abs().sum(dim=0) @ b.double().abs().sum(dim=1))
    return abs(total_dev - total) <= tol * scale, (total_dev, total, scale)


# The configurations the headline metric is quoted on, at their full sizes.  The CPU oracle cannot form whole
# matrices of this size in test time, so: sampled rows against the fp64 product and against the reference routine (or
# the TF32 model), and the checksum identity over every element.
def test_target_config_f16_level1_16384(oracle, cuda_device):
    """f16 Strassen-Winograd level 1 at M = N = K = 16384 (the reference's own test lists reach 16384:
    tests/hopper_f16_tensorop_strassen_winograd_presum.cu:10-35)."""
    import torch

    from subcuber_b200 import inputs, runner

    size = 16384
    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    a = inputs.fill_device("f16", "uniform1", (size, size), 1, 0, cuda_device)
    b = inputs.fill_device("f16", "uniform1", (size, size), 1, 1, cuda_device)
    d = runner.gemm(kernel, a, b)
    torch.cuda.synchronize()
    ok, info = _checksum_ok(a, b, d, 2e-5)
    assert ok, info
    a_np, b_np = a.cpu().numpy(), b.cpu().numpy()
    rows = np.array([0, 131, size // 4 + 5, size // 2 - 1], dtype=np.int32)   # quadrant rows
    all_rows = np.concatenate([rows, rows + size // 2])
    truth = oracle.truth_rows("f16", a_np, b_np, all_rows)
    got = d[torch.from_numpy(all_rows).long().to(cuda_device)].cpu().numpy()
    ref = oracle.sw_gemm("f16", 1, a_np, b_np, rows=rows)[all_rows]
    err, ref_err = _rel_fro(got, truth), _rel_fro(ref, truth)
    assert err <= 1.5 * ref_err, f"{err:.3e} vs reference routine {ref_err:.3e}"
    # harness tolerance element by element against the reference routine (tests/base_test.cuh:92-93 in the reference)
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    assert ((diff <= 4.0) | (diff <= 1e-2 * np.abs(ref.astype(np.float64)))).all()


def test_config_f16_level2_16384(oracle, cuda_device):
    """f16 level 2 (49 products) at 16384^3 (the reference's level-2 shapes:
    tests/ampere_f16_tensorop_strassen_winograd_presum_level_2.cu:8-11).  Sampled rows against the fp64 product: no
    worse than 1.5x the two-level recursion of the reference routine, with interim sums rounded to the output type
    at every hop as the reference's level-2 operator does (include/cutlass/gemm/device/strassen_gemm.h:1807-1914) and
    with interim sums kept in fp32; the whole matrix by checksum."""
    import torch

    from subcuber_b200 import inputs, runner

    size = 16384
    a = inputs.fill_device("f16", "uniform1", (size, size), 1, 0, cuda_device)
    b = inputs.fill_device("f16", "uniform1", (size, size), 1, 1, cuda_device)
    d = runner.gemm("blackwell_f16_sw_level2_2sm", a, b)
    torch.cuda.synchronize()
    ok, info = _checksum_ok(a, b, d, 2e-5)
    assert ok, info
    a_np, b_np = a.cpu().numpy(), b.cpu().numpy()
    rows = np.array([3, size // 16 + 1, size // 8 + 77, size // 4 - 2], dtype=np.int32)   # rows of the innermost quadrants
    all_rows = np.concatenate([rows + i * (size // 4) for i in range(4)])
    truth = oracle.truth_rows("f16", a_np, b_np, all_rows)
    got = d[torch.from_numpy(all_rows).long().to(cuda_device)].cpu().numpy()
    ref = oracle.sw_gemm("f16", 2, a_np, b_np, rows=rows, interim_round=True)[all_rows]
    ref32 = oracle.sw_gemm("f16", 2, a_np, b_np, rows=rows)[all_rows]
    err, ref_err, ref32_err = _rel_fro(got, truth), _rel_fro(ref, truth), _rel_fro(ref32, truth)
    assert err <= 1.5 * ref_err, f"{err:.3e} vs reference routine (two levels, rounded hops) {ref_err:.3e}"
    assert err <= 1.5 * ref32_err, f"{err:.3e} vs two-level recursion with fp32 hops {ref32_err:.3e}"


@pytest.mark.parametrize("kernel", ["blackwell_f32_sw_interleaved_presum_2sm", "blackwell_f32_sw_level2_2sm"])
def test_config_tf32_rectangular_k_heavy(kernel, oracle, cuda_device):
    """f32 storage, TF32 math, M = 16384, N = 8192, K = 32768, normal(0, 1) inputs, levels 1 and 2 (the reference's
    only TF32 tensor-op instantiation: example/strassen_gemm_ampere_tf32_tensorop/
    strassen_ampere_tf32_tensorop_gemm.cu:185-237).  Sampled rows against the fp64 product within 4x the error of the
    round-to-nearest TF32 level-1 model (the tensor core truncates), whole matrix by checksum."""
    import torch

    from subcuber_b200 import inputs, runner

    m, n, k = 16384, 8192, 32768
    a = inputs.fill_device("f32", "normal", (m, k), 1, 0, cuda_device)
    b = inputs.fill_device("f32", "normal", (k, n), 1, 1, cuda_device)
    d = runner.gemm(kernel, a, b)
    torch.cuda.synchronize()
    ok, info = _checksum_ok(a, b, d, 2e-4)
    assert ok, info
    a_np, b_np = a.cpu().numpy(), b.cpu().numpy()
    level = _level(kernel)
    rows = np.array([1, m // 8 + 9, m // 4 - 1], dtype=np.int32)   # rows of the innermost quadrants of either level
    nblk = 1 << level
    all_rows = np.concatenate([rows + i * (m // nblk) for i in range(nblk)])
    truth = oracle.truth_rows("f32", a_np, b_np, all_rows)
    got = d[torch.from_numpy(all_rows).long().to(cuda_device)].cpu().numpy()
    model = oracle.sw_gemm("tf32", level, a_np, b_np, rows=rows)[all_rows]
    err, model_err = _rel_fro(got, truth), _rel_fro(model, truth)
    assert err <= 4.0 * model_err + 1e-6, f"{err:.3e} vs TF32 model at level {level} {model_err:.3e}"
    assert err < (3e-3 if level == 1 else 6e-3)


def test_config_f32_level1_2048_against_fp64(oracle, cuda_device):
    """f32 level 1 at M = N = K = 2048, uniform[-1, 1) inputs, the whole matrix against the fp64 product (the
    reference's f32 gtest shape, tests/base_test.cuh:290-302 with its host fp64 check)."""
    from subcuber_b200 import inputs

    m = n = k = 2048
    a, b = inputs.operands("f32", "uniform1", m, n, k, seed=1)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    model = oracle.sw_gemm("tf32", 1, a, b)
    for kernel in ("blackwell_f32_sw_interleaved_presum_2sm", "blackwell_f32_sw_interleaved_presum"):
        got = _run(kernel, a, b, cuda_device)
        err, model_err = _rel_fro(got, truth), _rel_fro(model, truth)
        assert err <= 4.0 * model_err + 1e-6, f"{kernel}: {err:.3e} vs TF32 model {model_err:.3e}"
        assert err < 3e-3


# ------------------------------------------------------------------------------------- bounded waits
def test_bounded_wait_gives_up_and_the_device_stays_usable(oracle, cuda_device):
    """Every device-side wait is bounded (the reference's PostsumSemaphore spins without a bound,
    include/cutlass/postsum_semaphore.h:102-110).  Here one such wait is made to run out: the first K-halves of the
    split tiles do not publish their flags, the second halves give up after the (shortened) limit, unwind their CTAs
    and report status 105.  Nothing faults and nothing spins past its limit; the same GEMM then runs normally on the
    same device and is bit-exact."""
    import torch

    from subcuber_b200 import inputs, runner

    kernel = "blackwell_f16_sw_interleaved_presum"
    m, n, k = 768, 1536, 2048          # quadrant 3 x 3 tiles on 8 CTAs: the ninth tile is cut into two K-halves
    a_np, b_np = inputs.operands("f16", "harness", m, n, k, seed=4)
    a, b = runner.to_torch(a_np, cuda_device), runner.to_torch(b_np, cuda_device)
    d = torch.zeros((m, n), dtype=torch.float16, device=cuda_device)
    with pytest.raises(runner.KernelError) as exc:
        runner.gemm(kernel, a, b, d, opts=runner.options(sm_limit=8, wait_limit_us=1000, drop_split_flags=True))
    assert exc.value.code == 105
    torch.cuda.synchronize()
    got = _run(kernel, a_np, b_np, cuda_device, runner.options(sm_limit=8))
    assert np.array_equal(got, oracle.sw_gemm("f16", 1, a_np, b_np))


def test_level0_agrees_with_cublas(cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    a = inputs.fill_device("f16", "uniform1", (2048, 1024), 2, 0, cuda_device)
    b = inputs.fill_device("f16", "uniform1", (1024, 3072), 2, 1, cuda_device)
    d_blas, ms_blas = runner.run_kernel("cublas_f16", a, b, warmup=1, iterations=2)
    d_ours, ms_ours = runner.run_kernel("blackwell_f16_cubic_128x256", a, b, warmup=1, iterations=2)
    assert ms_blas > 0 and ms_ours > 0
    torch.cuda.synchronize()
    diff = (d_blas.double() - d_ours.double()).abs().max().item()
    assert diff <= 0.07  # both round an fp32 sum of 1024 products to fp16 (values up to ~64: ulp 0.03)


# ------------------------------------------------------------------------------------------- bfloat16
@pytest.mark.parametrize("kernel", BF16 + L2_BF16)
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (1536, 640, 1152), (1001, 776, 264)])
def test_uniform_inputs_bf16(kernel, shape, oracle, cuda_device):
    """Inexact inputs: error against the fp64 product no worse than 1.5x that of the reference routine with bfloat16
    storage (its templates instantiated for the type; the zero-padded problem where extents do not divide)."""
    from subcuber_b200 import inputs

    m, n, k = shape
    a, b = inputs.operands("bf16", "uniform1", m, n, k, seed=5)
    got = _run(kernel, a, b, cuda_device)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    ref = _padded_oracle(oracle, "bf16", _level(kernel), a, b)
    err, ref_err = _rel_fro(got, truth), _rel_fro(ref, truth)
    assert err <= 1.5 * ref_err, f"rel. Frobenius error {err:.3e} vs reference routine {ref_err:.3e}"
    assert err < 2e-2  # bfloat16 keeps 8 significant bits; level-1 presums are rounded to it once


@pytest.mark.parametrize("kernel", ["blackwell_bf16_sw_interleaved_presum_2sm", "blackwell_bf16_sw_level2_2sm"])
def test_alpha_beta_bf16(kernel, oracle, cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    m, n, k = (528, 1056, 288) if _level(kernel) == 2 else (272, 528, 144)
    a_np, b_np = inputs.operands("bf16", "harness", m, n, k, seed=17)
    c_np = inputs.operands("bf16", "harness", m, n, n, seed=18)[0]
    a, b, c = (runner.to_torch(x, cuda_device) for x in (a_np, b_np, c_np))
    d = runner.gemm(kernel, a, b, alpha=2.0, beta=-0.5, c=c)
    torch.cuda.synchronize()
    want = oracle.sw_gemm("bf16", _level(kernel), a_np, b_np, alpha=2.0, beta=-0.5, Cin=c_np)
    assert np.array_equal(runner.to_numpy(d), want)


def test_bf16_agrees_with_cublas(cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    a = inputs.fill_device("bf16", "uniform1", (1024, 1024), seed=3, device=cuda_device)
    b = inputs.fill_device("bf16", "uniform1", (1024, 1024), seed=3, subsequence=1, device=cuda_device)
    d_ours = runner.gemm("blackwell_bf16_cubic_2sm_256x256", a, b)
    d_blas, _ = runner.run_kernel("cublas_bf16", a, b)
    torch.cuda.synchronize()
    diff = (d_blas.double() - d_ours.double()).abs().max().item()
    assert diff <= 0.26  # both round an fp32 sum of 1024 products to bfloat16 (values up to ~32: ulp 0.125)


# --------------------------------------------------------------------------------------- ABI behaviour
def test_run_entry_point_error_codes(cuda_device):
    import torch

    from subcuber_b200 import runner

    a = torch.zeros((1, 128), dtype=torch.float16, device=cuda_device)   # one row cannot be cut in two block rows
    b = torch.zeros((128, 256), dtype=torch.float16, device=cuda_device)
    with pytest.raises(runner.KernelError) as e:
        runner.run_kernel("blackwell_f16_sw_interleaved_presum", a, b)
    assert e.value.code == 4
    a = torch.zeros((256, 128), dtype=torch.float16, device=cuda_device)
    with pytest.raises(runner.KernelError) as e:
        runner.run_kernel("blackwell_f16_sw_interleaved_presum", a, b, split_k=2)
    assert e.value.code == 5
    b = torch.zeros((128, 261), dtype=torch.float16, device=cuda_device)  # rows off the 16-byte grid run on copies
    assert runner.run_kernel("blackwell_f16_sw_interleaved_presum", a, b)[1] > 0


def test_workspace_checks(lib, cuda_device):
    import torch

    a = torch.zeros((256, 128), dtype=torch.float16, device=cuda_device)
    b = torch.zeros((128, 256), dtype=torch.float16, device=cuda_device)
    d = torch.zeros((256, 256), dtype=torch.float16, device=cuda_device)
    name = b"blackwell_f16_sw_interleaved_presum"
    assert lib.sb200_gemm(name, a.data_ptr(), b.data_ptr(), d.data_ptr(), 256, 256, 128, None, 0, None) == 6
    need = lib.sb200_gemm_workspace_bytes(name, 256, 256, 128)
    ws = torch.empty(need + 512, dtype=torch.uint8, device=cuda_device)
    base = ws.data_ptr() + ((-ws.data_ptr()) % 256)
    assert lib.sb200_gemm(name, a.data_ptr(), b.data_ptr(), d.data_ptr(), 256, 256, 128, base, need - 1, None) == 6
    assert lib.sb200_gemm(name, a.data_ptr(), b.data_ptr(), d.data_ptr(), 256, 256, 128, base + 16, need, None) == 6
    assert lib.sb200_gemm(name, a.data_ptr(), b.data_ptr(), d.data_ptr(), 256, 256, 128, base, need, None) == 0
    assert lib.sb200_gemm_status(base, None) == 0


def test_host_pipeline_overlaps_copies_and_keeps_results(cuda_device):
    """Operands in pinned host memory, copies overlapped with the kernels: every step's result equals the plain call's."""
    import torch

    from subcuber_b200 import inputs, runner

    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    m, n, k = 768, 1024, 512
    pipe = runner.HostPipeline(kernel, m, n, k, torch.float16, cuda_device)
    work, want = [], []
    for step in range(5):
        a, b = inputs.operands("f16", "uniform1", m, n, k, seed=30 + step)
        work.append((torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory(),
                     torch.full((m, n), float("nan"), dtype=torch.float16).pin_memory()))
        want.append(_run(kernel, a, b, cuda_device))
    for a_h, b_h, d_h in work:
        pipe.submit(a_h, b_h, d_h)
    pipe.finish()
    for (_, _, d_h), w in zip(work, want):
        assert np.array_equal(d_h.numpy(), w)
    with pytest.raises(ValueError):
        pipe.submit(torch.zeros((m, k), dtype=torch.float16), work[0][1], work[0][2])   # not pinned


def test_host_buffer_call_and_determinism(oracle, cuda_device):
    from subcuber_b200 import inputs, runner

    a, b = inputs.operands("f16", "uniform1", 512, 768, 384, seed=4)
    d1 = runner.gemm_host("blackwell_f16_sw_interleaved_presum", a, b)
    d2 = _run("blackwell_f16_sw_interleaved_presum", a, b, cuda_device)
    d3 = _run("blackwell_f16_sw_interleaved_presum", a, b, cuda_device)
    assert np.array_equal(d1, d2) and np.array_equal(d2, d3)
    # the on-the-fly presum variant forms the same operands but chains its accumulators in another order
    d4 = _run("blackwell_f16_sw_fused_presum", a, b, cuda_device)
    assert np.allclose(d2.astype(np.float64), d4.astype(np.float64), rtol=2e-3, atol=2e-2)


@pytest.mark.parametrize("dt", ["f16", "f32", "f64", "bf16"])
@pytest.mark.parametrize("dist", ["uniform1", "harness", "normal"])
def test_device_fill_matches_host_fill(dt, dist, cuda_device):
    from subcuber_b200 import inputs, runner

    h = inputs.fill_host(dt, dist, (257, 129), seed=6, subsequence=1)
    d = runner.to_numpy(inputs.fill_device(dt, dist, (257, 129), seed=6, subsequence=1, device=cuda_device))
    if dist == "normal":
        assert np.allclose(h.astype(np.float64), d.astype(np.float64), rtol=1e-2 if dt == "bf16" else 2e-3, atol=2e-3)
    else:
        assert np.array_equal(h, d)


def test_timed_call_reports_every_launch(lib, cuda_device):
    import torch

    from subcuber_b200 import inputs, runner

    a = inputs.fill_device("f16", "uniform1", (1024, 1024), 1, 0, cuda_device)
    b = inputs.fill_device("f16", "uniform1", (1024, 1024), 1, 1, cuda_device)
    d = torch.empty((1024, 1024), dtype=torch.float16, device=cuda_device)
    name = "blackwell_f16_sw_interleaved_presum"
    ws = runner.Workspace(name, 1024, 1024, 1024, cuda_device)
    ms = (C.c_float * 16)()
    nl = C.c_int(0)
    rc = lib.sb200_gemm_timed(name.encode(), a.data_ptr(), b.data_ptr(), d.data_ptr(), 1024, 1024, 1024, ws.ptr,
                              ws.nbytes, None, ms, C.byref(nl))
    assert rc == 0 and nl.value == 2 and ms[0] > 0 and ms[1] > 0
