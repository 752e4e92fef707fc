"""Generate tests/golden/frontend_golden.json by running the reference project's Python front end.

Needs the reference tree; it is imported from where it lies, nothing is copied:

    python tests/golden/make_frontend_golden.py [/path/to/reference]

Captured: the expression tree of strassen_winograd (print_tree text, base matrices of every product operand),
StrassenCompiler.gen_sched / last_fusion_schedule / iter_all_schedules / count_all_schedules for several sizes
and levels, and the printed output of generate_sched.gen_schedule.  The reference's command-line entry points are
not exercised: they fail on stale example paths (src/compile.py:51-58), only its library functions run.
"""
import contextlib
import io
import json
import os
import sys

# the reference tree: first argument, else REFERENCE_ROOT, else a directory "reference" beside this repository
ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
    "REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__))))), "reference"))
sys.dont_write_bytecode = True
sys.path.insert(0, os.path.join(ref, "src"))

import dsl  # noqa: E402
import compile as ref_compile  # noqa: E402
import generate_sched as ref_gs  # noqa: E402
from algos.strassen_winograd_level1 import strassen_winograd  # noqa: E402

out = {}

c, ms = strassen_winograd(64, 48, 32)
buf = io.StringIO()
with contextlib.redirect_stdout(buf):
    c.print_tree(set())
out["print_tree_64_48_32"] = buf.getvalue()
out["product_names"] = [str(m) for m in ms]
out["product_shapes"] = [list(m.shape) for m in ms]
out["c_shape"] = list(c.shape)
out["base_matrices"] = {
    str(m): {"a": sorted(str(x) for x in m.get_base_matrices_op1()), "b": sorted(str(x) for x in m.get_base_matrices_op2())}
    for m in ms
}
out["quadrant_starts"] = {str(x): [list(x.start), list(x.shape)] for m in ms for x in m.get_base_matrices()}
out["c_parts"] = [str(p) for p in c.parts]
out["matmuls_of_c_parts"] = {str(p): sorted(str(x) for x in p.get_matmul_matrices()) for p in c.parts}

sched = {}
for level, mnk in [(1, (1024, 1024, 1024)), (1, (8192, 8192, 8192)), (1, (2048, 1024, 1024)), (1, (4096, 4096, 4096)),
                   (2, (8192, 8192, 8192)), (2, (2048, 2048, 2048)), (2, (16384, 16384, 16384)), (3, (16384, 16384, 16384))]:
    for hw in ("A100", "H200"):
        comp = ref_compile.StrassenCompiler(hw_name=hw)
        s = comp.gen_sched(strassen_winograd, level, mnk)
        sched[f"{hw}|{level}|{mnk[0]}x{mnk[1]}x{mnk[2]}"] = {"schedule": s, "fusion": comp.last_fusion_schedule}
out["gen_sched"] = sched
comp = ref_compile.StrassenCompiler()
out["count_all_schedules"] = {str(l): comp.count_all_schedules(l) for l in (0, 1, 2, 3)}
out["iter_all_level1"] = list(comp.iter_all_schedules(strassen_winograd, 1, (4096, 4096, 4096)))
it2 = list(comp.iter_all_schedules(strassen_winograd, 2, (4096, 4096, 4096)))
out["iter_all_level2_count"] = len(it2)
out["iter_all_level2_first"] = it2[0]
out["iter_all_level2_last"] = it2[-1]
out["should_use_k2"] = {f"{a}x{b}x{c_}": comp.should_use_k2((a, b, c_)) for (a, b, c_) in [(1024, 1024, 1024), (2048, 1024, 1024), (2047, 2047, 2047)]}
out["fusion_without_dag"] = comp.output_sum_fusion({}, out["iter_all_level1"][1], (8192, 8192, 8192), "K4")
out["fusion_k2"] = comp.output_sum_fusion({}, out["iter_all_level1"][0], (1024, 1024, 1024), "K2")
out["fusion_bad_kernel"] = comp.output_sum_fusion({}, out["iter_all_level1"][1], (1024, 1024, 1024), "K1")

gs = {}
for (m, n, k, tile, reg) in [(2048, 2048, 2048, (256, 128, 8), (16, 8)), (8192, 8192, 8192, (128, 256, 64), (8, 8)),
                             (4096, 2048, 1024, (128, 128, 8), (8, 8))]:
    c2, ms2 = strassen_winograd(m, n, k)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        ref_gs.gen_schedule(c2, ms2, m, n, k, tile, reg)
    gs[f"{m}x{n}x{k}|{tile}|{reg}"] = buf.getvalue()
out["gen_schedule"] = gs

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "frontend_golden.json")
with open(path, "w") as f:
    json.dump(out, f, indent=1, sort_keys=True)
print("wrote", path, os.path.getsize(path), "bytes")
