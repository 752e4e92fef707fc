"""The C-ABI library loads without a GPU, exports every symbol the public header declares, and its
host-side argument checks behave like the reference operator's can_implement / get_workspace_size."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "subcuber_b200.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    runs = re.findall(r"^SB200_DECLARE_RUN\((run_\w+)\);", text, flags=re.M)
    funcs = re.findall(r"^\s*(?:const\s+)?[\w\s\*]+?\b(sb200_\w+)\s*\(", text, flags=re.M)
    funcs = [f for f in funcs if not f.endswith("_t")]
    return runs, sorted(set(funcs))


def test_header_symbols_are_exported(lib):
    runs, funcs = _declared_symbols()
    assert len(runs) >= 15 and "sb200_gemm" in funcs and "sb200_fill_device" in funcs
    for name in runs + funcs:
        assert hasattr(lib, name), f"{name} is declared in include/subcuber_b200.h but not exported"


def test_registry_rows(lib):
    from subcuber_b200 import runner

    rows = runner.kernels()
    names = [r.name for r in rows]
    assert len(names) == len(set(names))
    assert all(r.arch == "blackwell" for r in rows)
    # every registry row has a run_<name> entry point and vice versa
    runs, _ = _declared_symbols()
    assert sorted("run_" + n for n in names) == sorted(runs)
    assert [r.name for r in runner.kernels(dtype="half", level=1)] == [
        "blackwell_f16_sw_fused_presum", "blackwell_f16_sw_interleaved_presum",
        "blackwell_f16_sw_fused_presum_2sm", "blackwell_f16_sw_interleaved_presum_2sm",
        "blackwell_f16_sw_merged_presum_2sm", "blackwell_f16_strassen_fused_presum", "blackwell_f16_strassen_fused_presum_2sm",
        "blackwell_f16_strassen_presum_2sm", "blackwell_f16_sw_auto"]
    assert [r.name for r in runner.kernels(dtype="f32", level=0, regex="cubic")] == [
        "blackwell_f32_cubic_128x256", "blackwell_f32_cubic_128x128", "blackwell_f32_cubic_2sm_256x256"]


def test_auto_kernel_choice(lib):
    """Size-based choice of level and family: small problems run the plain pair kernel, large ones recurse, whatever
    the extents divide by (the last block row / column may be short)."""
    import ctypes as C

    lib.sb200_auto_kernel.restype = C.c_char_p
    lib.sb200_auto_kernel.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int]
    pick = lambda dt, m, n, k: lib.sb200_auto_kernel(dt.encode(), m, n, k).decode()
    assert pick("f16", 8192, 8192, 8192) == "blackwell_f16_cubic_2sm_256x256"
    assert pick("f16", 16384, 16384, 16384) == "blackwell_f16_sw_interleaved_presum_2sm"
    assert pick("f16", 32768, 32768, 32768) == "blackwell_f16_sw_level2_2sm"
    assert pick("f16", 32768, 32768, 4096) == "blackwell_f16_cubic_2sm_256x256"      # the smallest extent decides
    assert pick("f16", 32770, 32768, 32768) == "blackwell_f16_sw_level2_2sm"  # need not divide by 4
    assert pick("f32", 16384, 8192, 32768) == "blackwell_f32_cubic_2sm_256x256"
    assert pick("f32", 16384, 16384, 16384) == "blackwell_f32_sw_level2_2sm"
    assert pick("f64", 8192, 8192, 8192) == "blackwell_f64_sw_level1"
    assert pick("f64", 16384, 16384, 16384) == "blackwell_f64_sw_level2"
    assert pick("bf16", 16384, 16384, 16384) == "blackwell_bf16_sw_interleaved_presum_2sm"
    assert lib.sb200_auto_kernel(b"int8", 1, 1, 1) is None
    assert lib.sb200_gemm_can_implement(b"blackwell_f16_sw_auto", 512, 512, 512) == 0
    assert lib.sb200_gemm_workspace_bytes(b"blackwell_f16_sw_auto", 512, 512, 512) == \
        lib.sb200_gemm_workspace_bytes(b"blackwell_f16_cubic_2sm_256x256", 512, 512, 512)


def test_alias_tables():
    from subcuber_b200 import runner

    assert runner.normalize_arch("sm100a") == "blackwell" and runner.normalize_arch("SM90a") == "hopper"
    assert runner.normalize_arch("80") == "ampere" and runner.normalize_arch("blackwell") == "blackwell"
    assert runner.normalize_dtype("half") == "f16" and runner.normalize_dtype("d") == "f64"
    assert runner.normalize_dtype("FP32") == "f32"


@pytest.mark.parametrize("kernel,m,n,k,rc", [
    ("blackwell_f16_cubic_128x256", 128, 256, 64, 0),
    ("blackwell_f16_cubic_128x256", 100, 264, 72, 0),       # ragged sizes are fine (TMA zero fill, masked stores)
    ("blackwell_f16_cubic_128x256", 128, 260, 64, 0),       # rows off the 16-byte grid: runs on padded copies
    ("blackwell_f16_cubic_128x256", 0, 256, 64, 4),
    ("blackwell_f16_sw_interleaved_presum", 256, 512, 128, 0),
    ("blackwell_f16_sw_interleaved_presum", 255, 512, 128, 0),  # short last block row
    ("blackwell_f16_sw_interleaved_presum", 256, 520, 128, 0),  # blocks are cut on the 16-byte grid: 264 + 256 columns
    ("blackwell_f16_sw_interleaved_presum", 255, 517, 129, 0),  # padded copies, then short blocks
    ("blackwell_f16_sw_interleaved_presum", 1, 512, 128, 4),    # a block row would be empty
    ("blackwell_f16_sw_level2", 1000, 520, 136, 0),
    ("blackwell_f16_sw_level2", 1000, 520, 24, 4),              # 24 columns cannot be cut in four 16-byte aligned blocks
    ("blackwell_f64_sw_level1", 1001, 515, 129, 0),
    ("blackwell_f32_sw_fused_presum", 64, 72, 40, 0),
    ("no_such_kernel", 128, 128, 128, 8),
])
def test_can_implement(lib, kernel, m, n, k, rc):
    assert lib.sb200_gemm_can_implement(kernel.encode(), m, n, k) == rc


def test_workspace_layout(lib):
    from subcuber_b200 import _lib as L

    w = L.WorkspaceLayout()
    assert lib.sb200_gemm_workspace_layout(b"blackwell_f16_sw_interleaved_presum", 8192, 8192, 8192, C.byref(w)) == 0
    assert (w.mq, w.nq, w.kq, w.tiles_m, w.tiles_n, w.bn) == (4096, 4096, 4096, 32, 16, 256)
    q = 4096 * 4096 * 2
    assert w.presum_a == 256 and w.presum_b == 256 + 4 * q and w.handoff[0] == 256 + 8 * q
    tile = 128 * 256 * 4
    # buffer 0 (M0) holds one tile per tile of the grid (plus slots for cut tiles), buffers 1..3 one tile per worker
    assert w.handoff[1] - w.handoff[0] >= 32 * 16 * tile and (w.handoff[1] - w.handoff[0]) % tile == 0
    per_worker = w.handoff[2] - w.handoff[1]
    assert per_worker >= tile and per_worker % tile == 0 and w.handoff[3] - w.handoff[2] == per_worker
    assert w.total >= w.handoff[3] + per_worker
    assert lib.sb200_gemm_workspace_bytes(b"blackwell_f16_sw_interleaved_presum", 8192, 8192, 8192) == w.total
    assert lib.sb200_gemm_workspace_bytes(b"blackwell_f16_cubic_128x256", 8192, 8192, 8192) == 256
    assert lib.sb200_gemm_workspace_bytes(b"nope", 8, 8, 8) == 0
    assert lib.sb200_gemm_launches(b"blackwell_f16_sw_interleaved_presum") == 2
    assert lib.sb200_gemm_launches(b"blackwell_f16_sw_fused_presum") == 1


def test_seeded_generator_pins():
    """First values per dtype and distribution (element i is a pure function of seed, subsequence, i)."""
    from subcuber_b200 import inputs

    assert inputs.fill_host("f32", "uniform1", (6,), 1, 0).tolist() == [
        0.7805182933807373, 0.343996524810791, -0.5051971673965454, 0.515252947807312, -0.5044735670089722,
        -0.6794435977935791]
    assert inputs.fill_host("f16", "uniform1", (6,), 1, 0).tolist() == [
        0.78076171875, 0.343994140625, -0.50537109375, 0.51513671875, -0.50439453125, -0.6796875]
    assert inputs.fill_host("f16", "harness", (6,), 1, 0).tolist() == [3.75, 3.25, -1.75, 0.5, 2.0, -4.0]
    assert inputs.fill_host("f32", "harness", (6,), 1, 0).tolist() == [12.75, -0.5, 10.25, 3.5, 13.25, -7.0]
    n = inputs.fill_host("f32", "normal", (4,), 1, 0)
    assert abs(float(n[0]) - 0.380400687456131) < 1e-6 and abs(float(n[2]) + 1.5671557188034058) < 1e-6
    a = inputs.fill_host("f64", "uniform1", (3, 5), 9, 0)
    b = inputs.fill_host("f64", "uniform1", (3, 5), 9, 1)
    assert (a != b).any() and a.shape == (3, 5)
    big = inputs.fill_host("f32", "normal", (400, 400), 3, 0)
    assert abs(float(big.mean())) < 0.02 and abs(float(big.std()) - 1.0) < 0.02
    h = inputs.fill_host("f16", "harness", (300, 300), 3, 0)
    assert float(h.min()) == -4.0 and float(h.max()) == 4.0 and ((h * 4) % 1 == 0).all()


def test_cpu_only_call_fails_loudly():
    """No CPU fallback: operands that are not on a CUDA device are refused."""
    import torch

    from subcuber_b200 import runner

    a = torch.zeros((128, 64), dtype=torch.float16)
    with pytest.raises(ValueError):
        runner.gemm("blackwell_f16_cubic_128x256", a, a.t().contiguous())
