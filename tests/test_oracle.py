"""The CPU oracle is pinned against the reference project's own oracle kernels: against committed
golden vectors made from them (tests/golden/make_golden.py) and, where the host build of those kernels is
present (oracle/_ref), against fresh runs of it."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_oracle_vectors.npz")
DT = {0: "f16", 1: "f32", 2: "f64", 4: "bf16"}


def _load(z, key, code):
    """bfloat16 arrays are stored as their 16-bit patterns."""
    x = z[key]
    if code == 4:
        import ml_dtypes

        return x.view(ml_dtypes.bfloat16)
    return x


def _cases():
    z = np.load(GOLD)
    names = sorted({k.split("_")[0] for k in z.files if k.startswith("case")})
    return z, names


def test_golden_vectors_bit_exact(oracle):
    z, names = _cases()
    assert len(names) >= 10
    for nm in names:
        code, level, m, n, k, _ = (int(v) for v in z[nm + "_meta"])
        alpha, beta = (float(v) for v in z[nm + "_ab"])
        cin = _load(z, nm + "_c", code) if (nm + "_c") in z.files else None
        got = oracle.sw_gemm(DT[code], level, _load(z, nm + "_a", code), _load(z, nm + "_b", code), alpha=alpha,
                             beta=beta, Cin=cin)
        want = _load(z, nm + "_d", code)
        assert got.dtype == want.dtype and got.shape == (m, n)
        assert np.array_equal(got, want), f"{nm}: oracle differs from the reference kernels' output"


def test_golden_inputs_come_from_the_seeded_generator():
    from subcuber_b200 import inputs

    z, names = _cases()
    dist_name = {v: k for k, v in inputs.DIST_CODE.items()}
    for idx, nm in enumerate(names):
        code, level, m, n, k, dist = (int(v) for v in z[nm + "_meta"])
        a, b = inputs.operands(DT[code], dist_name[dist], m, n, k, seed=100 + idx)
        if dist_name[dist] == "normal":
            assert np.allclose(a, z[nm + "_a"], rtol=1e-5, atol=1e-6)
        else:
            assert np.array_equal(a, _load(z, nm + "_a", code)) and np.array_equal(b, _load(z, nm + "_b", code))


def test_golden_presums(oracle):
    z = np.load(GOLD)
    for dt in ("f32", "f64"):
        pa, pb = oracle.sw_presums(dt, z[f"presum_{dt}_a"], z[f"presum_{dt}_b"])
        assert np.array_equal(pa, z[f"presum_{dt}_pa"])
        assert np.array_equal(pb, z[f"presum_{dt}_pb"])


@pytest.mark.parametrize("dt", ["f16", "f32", "f64", "bf16"])
@pytest.mark.parametrize("shape", [(8, 8, 8), (64, 48, 32), (130, 66, 34), (33, 20, 16), (2, 2, 2)])
def test_against_reference_host_build(oracle, dt, shape):
    if oracle.ref_oracle() is None:
        pytest.skip("reference host build absent (needs the reference tree); golden vectors cover this")
    rng = np.random.default_rng(sum(shape))
    m, n, k = shape
    a = rng.uniform(-1, 1, (m, k)).astype(oracle.NP_DTYPE[dt])
    b = rng.uniform(-1, 1, (k, n)).astype(oracle.NP_DTYPE[dt])
    for level in (0, 1):
        assert np.array_equal(oracle.sw_gemm(dt, level, a, b), oracle.ref_sw_gemm(dt, level, a, b))


def test_presum_rounding_convention_f16(oracle):
    """Presums are formed in fp32 from the raw values and rounded once (strassen_reference_l1.cuh:68-85)."""
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (16, 24)).astype(np.float16)
    b = rng.uniform(-1, 1, (24, 8)).astype(np.float16)
    pa, pb = oracle.sw_presums("f16", a, b)
    a0, a1, a2, a3 = (x.astype(np.float32) for x in (a[:8, :12], a[:8, 12:], a[8:, :12], a[8:, 12:]))
    s1 = a2 + a3
    s2 = s1 - a0
    assert np.array_equal(pa[0], s1.astype(np.float16))
    assert np.array_equal(pa[1], s2.astype(np.float16))
    assert np.array_equal(pa[2], (a0 - a2).astype(np.float16))
    assert np.array_equal(pa[3], (a1 - s2).astype(np.float16))
    b0, b1, b2, b3 = (x.astype(np.float32) for x in (b[:12, :4], b[:12, 4:], b[12:, :4], b[12:, 4:]))
    b31 = b3 - b1
    s3 = b31 + b0
    assert np.array_equal(pb[0], (b1 - b0).astype(np.float16))
    assert np.array_equal(pb[1], b31.astype(np.float16))
    assert np.array_equal(pb[2], s3.astype(np.float16))
    assert np.array_equal(pb[3], (s3 - b2).astype(np.float16))


@pytest.mark.parametrize("dt,tol", [("f16", 2e-2), ("f32", 2e-5), ("f64", 1e-13), ("tf32", 5e-3), ("bf16", 2e-2)])
@pytest.mark.parametrize("level", [0, 1, 2])
def test_levels_agree_with_fp64_matmul(oracle, dt, tol, level):
    rng = np.random.default_rng(level)
    m, n, k = 64, 96, 128
    a = rng.uniform(-1, 1, (m, k)).astype(oracle.NP_DTYPE[dt])
    b = rng.uniform(-1, 1, (k, n)).astype(oracle.NP_DTYPE[dt])
    truth = a.astype(np.float64) @ b.astype(np.float64)
    got = oracle.sw_gemm(dt, level, a, b).astype(np.float64)
    rel = np.linalg.norm(got - truth) / np.linalg.norm(truth)
    assert rel < tol * (3 if level == 2 else 1)


def test_exact_on_harness_values(oracle):
    """With the harness' value set every partial sum is exact, so all levels agree bit for bit."""
    from subcuber_b200 import inputs

    a, b = inputs.operands("f32", "harness", 64, 64, 64, seed=5)
    d0 = oracle.sw_gemm("f32", 0, a, b)
    assert np.array_equal(d0, oracle.sw_gemm("f32", 1, a, b))
    assert np.array_equal(d0, oracle.sw_gemm("f32", 2, a, b))
    assert np.array_equal(d0.astype(np.float64), a.astype(np.float64) @ b.astype(np.float64))


def test_row_sampling_matches_full(oracle):
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, (48, 40)).astype(np.float16)
    b = rng.uniform(-1, 1, (40, 56)).astype(np.float16)
    full = oracle.sw_gemm("f16", 1, a, b)
    rows = [0, 5, 23]
    part = oracle.sw_gemm("f16", 1, a, b, rows=rows)
    for r in rows:
        assert np.array_equal(part[r], full[r]) and np.array_equal(part[r + 24], full[r + 24])
    assert not part[1].any()
    t = oracle.truth_rows("f16", a, b, [3, 47])
    assert np.allclose(t, (a.astype(np.float64) @ b.astype(np.float64))[[3, 47]], rtol=0, atol=1e-12)


def test_row_sampling_matches_full_at_level2(oracle):
    rng = np.random.default_rng(12)
    a = rng.uniform(-1, 1, (96, 80)).astype(np.float16)
    b = rng.uniform(-1, 1, (80, 112)).astype(np.float16)
    rows = [0, 7, 23]   # rows of the innermost quadrants: each yields four C rows
    for interim_round in (False, True):
        full = oracle.sw_gemm("f16", 2, a, b, interim_round=interim_round)
        part = oracle.sw_gemm("f16", 2, a, b, rows=rows, interim_round=interim_round)
        for r in rows:
            for blk in range(4):
                assert np.array_equal(part[r + 24 * blk], full[r + 24 * blk])
        assert not part[1].any()


def test_level2_interim_rounding_is_the_less_accurate_variant(oracle):
    rng = np.random.default_rng(2)
    a = rng.uniform(-1, 1, (128, 128)).astype(np.float16)
    b = rng.uniform(-1, 1, (128, 128)).astype(np.float16)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    e_acc = np.linalg.norm(oracle.sw_gemm("f16", 2, a, b, interim_round=False).astype(np.float64) - truth)
    e_rnd = np.linalg.norm(oracle.sw_gemm("f16", 2, a, b, interim_round=True).astype(np.float64) - truth)
    assert e_acc <= e_rnd * 1.05


def test_bad_arguments(oracle):
    a = np.zeros((6, 6), dtype=np.float32)
    with pytest.raises(ValueError):
        oracle.sw_gemm("f32", 2, a, a)  # level 2 needs sizes divisible by 4
