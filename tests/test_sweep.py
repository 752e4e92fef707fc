"""Host logic of the sweep driver (cell list, resuming from a partial output file); no GPU needed."""
import json

from subcuber_b200 import sweep


def test_cells_and_resume(tmp_path):
    cells = sweep.plan_cells([2048, 4096], [(16384, 8192, 32768)], ["f16", "f32"], [0, 1, 2])
    assert len(cells) == 2 * 3 * 3 and (16384, 8192, 32768, "f32", 2) in cells
    out = tmp_path / "sweep.jsonl"
    lines = [json.dumps({"cell": sweep.cell_key(2048, 2048, 2048, "f16", 0), "tflops": 1.0}),
             json.dumps({"cell": sweep.cell_key(2048, 2048, 2048, "f16", 1), "tflops": 2.0}),
             '{"cell": "4096x4096x4096:f16:L0", "tfl']            # cut short by an interruption
    out.write_text("\n".join(lines) + "\n")
    done = sweep.done_cells(str(out))
    assert done == {"2048x2048x2048:f16:L0", "2048x2048x2048:f16:L1"}
    assert sweep.done_cells(str(tmp_path / "absent.jsonl")) == set()
    assert set(sweep.CUBLAS) == {d for d, _ in sweep.KERNELS}
