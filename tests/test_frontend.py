"""Python front end (DSL, schedule generators, emitter) against golden outputs produced by running the reference
project's own front end (tests/golden/make_frontend_golden.py -> tests/golden/frontend_golden.json)."""
import ast
import contextlib
import io
import json
import os

import numpy as np
import pytest

from subcuber_b200 import compile as sbc
from subcuber_b200 import dsl, emit
from subcuber_b200 import generate_sched as gs
from subcuber_b200 import tile_program as tp
from subcuber_b200.algos.strassen_winograd_level1 import strassen_winograd

GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "frontend_golden.json")))


def _capture(fn, *args, **kw):
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        ret = fn(*args, **kw)
    return buf.getvalue(), ret


def test_expression_tree_matches_reference():
    c, ms = strassen_winograd(64, 48, 32)
    text, _ = _capture(c.print_tree)
    assert text == GOLD["print_tree_64_48_32"]
    assert [str(m) for m in ms] == GOLD["product_names"]
    assert [list(m.shape) for m in ms] == GOLD["product_shapes"] and list(c.shape) == GOLD["c_shape"]
    bases = {str(m): {"a": sorted(str(x) for x in m.get_base_matrices_op1()),
                      "b": sorted(str(x) for x in m.get_base_matrices_op2())} for m in ms}
    assert bases == GOLD["base_matrices"]
    starts = {str(x): [list(x.start), list(x.shape)] for m in ms for x in m.get_base_matrices()}
    assert starts == GOLD["quadrant_starts"]
    assert {str(p): sorted(str(x) for x in p.get_matmul_matrices()) for p in c.parts} == GOLD["matmuls_of_c_parts"]


def test_dsl_numeric_evaluation_is_a_matrix_product():
    """Evaluate the DAG numerically: the four output expressions assemble A @ B."""
    m, n, k = 8, 12, 6
    c, _ = strassen_winograd(m, n, k)
    rng = np.random.default_rng(0)
    roots = {"a": rng.integers(-3, 4, (m, k)).astype(np.float64), "b": rng.integers(-3, 4, (k, n)).astype(np.float64)}

    def ev(node):
        if isinstance(node, dsl.BinOp):
            x, y = ev(node.op1), ev(node.op2)
            return x + y if node.op == "+" else x - y if node.op == "-" else x @ y
        base = roots["a"] if node.name.startswith("a") else roots["b"]
        (r0, c0), (h, w) = node.start, node.shape
        return base[r0:r0 + h, c0:c0 + w]

    got = np.block([[ev(c.parts[0]), ev(c.parts[1])], [ev(c.parts[2]), ev(c.parts[3])]])
    assert np.array_equal(got, roots["a"] @ roots["b"])


def test_expand_terms_reproduces_the_oracle_evaluation_order():
    _, ms = strassen_winograd(4, 4, 4)
    by = {m.name: m for m in ms}
    names = lambda terms: [(c, t.name) for c, t in terms]  # noqa: E731
    assert names(dsl.expand_terms(by["m2"].op1)) == [(1, "a2"), (1, "a3"), (-1, "a0")]
    assert names(dsl.expand_terms(by["m5"].op1)) == [(-1, "a2"), (-1, "a3"), (1, "a0"), (1, "a1")]
    assert names(dsl.expand_terms(by["m6"].op2)) == [(1, "b3"), (-1, "b1"), (1, "b0"), (-1, "b2")]
    assert names(dsl.expand_terms(by["m0"].op1)) == [(1, "a0")]
    with pytest.raises(ValueError):
        dsl.expand_terms(by["m0"])


@pytest.mark.parametrize("key", sorted(GOLD["gen_sched"].keys()))
def test_gen_sched_matches_reference(key):
    hw, level, mnk = key.split("|")
    mnk = tuple(int(x) for x in mnk.split("x"))
    comp = sbc.StrassenCompiler(hw_name=hw)
    schedule = comp.gen_sched(strassen_winograd, int(level), mnk)
    assert schedule == GOLD["gen_sched"][key]["schedule"]
    assert json.loads(json.dumps(comp.last_fusion_schedule)) == GOLD["gen_sched"][key]["fusion"]


def test_schedule_enumeration_and_fusion_match_reference():
    comp = sbc.StrassenCompiler()
    assert {str(l): comp.count_all_schedules(l) for l in (0, 1, 2, 3)} == GOLD["count_all_schedules"]
    level1 = list(comp.iter_all_schedules(strassen_winograd, 1, (4096, 4096, 4096)))
    assert level1 == GOLD["iter_all_level1"]
    level2 = list(comp.iter_all_schedules(strassen_winograd, 2, (4096, 4096, 4096)))
    assert len(level2) == GOLD["iter_all_level2_count"] == 64
    assert level2[0] == GOLD["iter_all_level2_first"] and level2[-1] == GOLD["iter_all_level2_last"]
    assert {k: comp.should_use_k2(tuple(int(x) for x in k.split("x"))) for k in GOLD["should_use_k2"]} == GOLD["should_use_k2"]
    norm = lambda d: json.loads(json.dumps(d))  # noqa: E731
    assert norm(comp.output_sum_fusion({}, level1[1], (8192, 8192, 8192), "K4")) == GOLD["fusion_without_dag"]
    assert norm(comp.output_sum_fusion({}, level1[0], (1024, 1024, 1024), "K2")) == GOLD["fusion_k2"]
    assert comp.output_sum_fusion({}, level1[1], (1024, 1024, 1024), "K1") == GOLD["fusion_bad_kernel"]


@pytest.mark.parametrize("key", sorted(GOLD["gen_schedule"].keys()))
def test_gen_schedule_output_matches_reference(key):
    mnk, tile, reg = key.split("|")
    m, n, k = (int(x) for x in mnk.split("x"))
    c, ms = strassen_winograd(m, n, k)
    text, ranked = _capture(gs.gen_schedule, c, ms, m, n, k, ast.literal_eval(tile), ast.literal_eval(reg))
    assert text == GOLD["gen_schedule"][key]
    assert len(ranked) == 1 and [str(p[0]) for p in ranked[0].presums_todo["a"]] == ["s1"]


def test_set_partitions_count():
    assert sum(1 for _ in gs.get_all_set_partitions([1, 2, 3, 4])) == 15   # Bell numbers
    assert sum(1 for _ in gs.get_all_set_partitions(list(range(7)))) == 877


def test_b200_target_and_build(tmp_path):
    assert sbc.HW_SPECS["B200"]["sm_count"] == 148 and "A100" in sbc.HW_SPECS and "H200" in sbc.HW_SPECS
    text, schedule = _capture(sbc.build, 1, 8192, 8192, 8192, "fp16", str(tmp_path), hw="B200")
    assert schedule == ["K1(m0)", "K4(m1)", "K4(m2)", "K4(m4)", "K4(m5)", "K4(m3)", "K4(m6)"]
    assert "Generated Optimal Schedule:" in text and "Generated Fusion Schedule:" in text
    plan = json.load(open(tmp_path / "schedule.json"))["plan"]
    assert plan["kernel"] == "blackwell_f16_sw_interleaved_presum_2sm"
    assert [l["program"] for l in plan["launches"]] == ["level1_first_early", "level1_second_taps"]
    programs = json.load(open(tmp_path / "tile_programs.json"))
    assert [p["a"] for p in programs["level1_second_taps"]["products"]][0] == [[1, "S1"]]
    assert "sb200_program_level1_second_taps" in open(tmp_path / "sw_tile_programs.inc").read()
    # below 2048 the all-in-one tile kernel is chosen: presums formed on the fly, one launch
    text, schedule = _capture(sbc.build, 1, 1024, 1024, 1024, "f32", str(tmp_path / "small"), hw="B200")
    assert schedule == ["K2(Base)"]
    plan = json.load(open(tmp_path / "small" / "schedule.json"))["plan"]
    assert plan["kernel"] == "blackwell_f32_sw_fused_presum" and len(plan["launches"]) == 1
    # dry run writes nothing; the command line entry point works (the reference's fails on stale paths)
    text, _ = _capture(sbc.main, ["--level", "2", "--m", "4096", "--n", "4096", "--k", "4096", "--datatype", "fp16",
                                  "--output_dir", str(tmp_path / "dry"), "--dry-run", "--hw", "B200"])
    assert "[dry-run] would write" in text and not (tmp_path / "dry").exists()
    with pytest.raises(ValueError):
        sbc.build(1, 64, 64, 64, "int8", str(tmp_path))


def test_emitted_programs_equal_the_tables_in_the_library(lib):
    programs = emit.all_programs()
    emit.verify_programs(programs)
    for name, pg in programs.items():
        assert tp.to_bytes(pg) == tp.to_bytes(tp.from_library(name)), name


def test_bilinear_forms_from_the_dsl():
    c, ms = strassen_winograd(4, 4, 4)
    want = {0: [(0, 0), (1, 2)], 1: [(0, 1), (1, 3)], 2: [(2, 0), (3, 2)], 3: [(2, 1), (3, 3)]}
    for q, part in enumerate(c.parts):
        t = emit.bilinear_form(part)
        assert sorted(zip(*np.nonzero(t))) == want[q] and t.sum() == 2
    assert emit.quadrant_vector(ms[5].op1).tolist() == [1, 1, -1, -1]   # a1s2 = a1 - (a2 + a3 - a0)


def test_strassen_original_algorithm_through_the_dsl(tmp_path, capsys):
    """A second <2,2,2;7> algorithm stated in the DSL: the same block product, a generated tile program that the
    checker accepts, and a build() plan that names the kernels that run it."""
    import json

    from subcuber_b200.algos.strassen_level1 import strassen

    c, ms = strassen(4, 4, 4)
    assert [m.name for m in ms] == ["m1", "m2", "m3", "m4", "m5", "m6", "m7"]
    want = {0: [(0, 0), (1, 2)], 1: [(0, 1), (1, 3)], 2: [(2, 0), (3, 2)], 3: [(2, 1), (3, 3)]}
    for q, part in enumerate(c.parts):
        t = emit.bilinear_form(part)
        assert sorted(zip(*np.nonzero(t))) == want[q] and t.sum() == 2
    pg = emit.level1_strassen_program(ms)
    assert pg.nproducts == 7 and pg.nepilogues == 6 and pg.needs_feed == 1
    assert max(pr.a.nterms for pr in (pg.product[i] for i in range(7))) == 2   # no operand sums more than two blocks
    # numeric run of the program on integer blocks
    rng = np.random.default_rng(3)
    a = rng.integers(-3, 4, size=(8, 12)).astype(np.int64)
    b = rng.integers(-3, 4, size=(12, 6)).astype(np.int64)
    qa, qb = emit._quadrants(a), emit._quadrants(b)
    views = {i: qa[i] for i in range(4)}
    views.update({8 + i: qb[i] for i in range(4)})
    out = {}
    emit.run_program_numeric(pg, views, {}, out)
    assert np.array_equal(np.block([[out[0], out[1]], [out[2], out[3]]]), a @ b)
    sched = sbc.build(1, 8192, 8192, 8192, "f16", str(tmp_path), hw="B200", algorithm="strassen")
    capsys.readouterr()
    assert len(sched) == 7 and sched[0].startswith("K1(")
    plan = json.loads((tmp_path / "schedule.json").read_text())["plan"]
    assert plan["kernel"] == "blackwell_f16_strassen_fused_presum_2sm"
    assert [l["program"] for l in plan["launches"]] == ["level1_strassen"]
    assert "level1_strassen" in json.loads((tmp_path / "tile_programs.json").read_text())
    with pytest.raises(ValueError):
        sbc.build(2, 8192, 8192, 8192, "f16", str(tmp_path), hw="B200", algorithm="strassen")
