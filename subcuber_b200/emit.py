"""Emitter: from the algorithm DSL and a schedule to the tile programs the Blackwell kernels interpret.

The reference front end prints its schedules and copies pre-written example sources (src/compile.py:48-131,
646-653); nothing downstream reads the schedule.  Here the schedule selects a launch plan of this library's
kernels, and the per-tile programs of every launch (product order, operand term lists, tensor-memory slot plan,
postsum steps) are GENERATED from the DSL expressions and checked (`tile_program.check_program`) before they are
written out.  The tables compiled into the CUDA library (csrc/sw_programs.h) are the same tables; a test compares
them byte for byte.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import tile_program as tp
from .dsl import BinOp, Matrix, expand_terms

# operand view indices (csrc/tile_program.h)
QUADRANT_VIEW = {"a0": 0, "a1": 1, "a2": 2, "a3": 3, "b0": 8, "b1": 9, "b2": 10, "b3": 11}
PRESUM_VIEW = {"s1": 4, "s2": 5, "a02": 6, "a1s2": 7, "b10": 12, "b31": 13, "s3": 14, "s3b2": 15}
P, Q = 0, 1
WS_M0, WS_M4, WS_U, WS_V = 0, 1, 2, 3


# ------------------------------------------------------------------------------------------- algebra from the DSL
def quadrant_vector(expr: Matrix) -> np.ndarray:
    """Coefficients of a presum expression over its side's four quadrants."""
    v = np.zeros(4, dtype=np.int64)
    for coef, leaf in expand_terms(expr):
        v[QUADRANT_VIEW[leaf.name] % 8] += coef
    return v


def bilinear_form(expr: Matrix) -> np.ndarray:
    """4x4 integer matrix T with expr = sum_ij T[i, j] * (a_i @ b_j), for a postsum expression of the DSL."""
    if isinstance(expr, BinOp) and expr.op == "@":
        return np.outer(quadrant_vector(expr.op1), quadrant_vector(expr.op2))
    if isinstance(expr, BinOp):
        left, right = bilinear_form(expr.op1), bilinear_form(expr.op2)
        return left + right if expr.op == "+" else left - right
    raise ValueError("postsum expressions are sums of products")


# --------------------------------------------------------------------------------------------- program building
def _operand(expr: Matrix, fly: bool) -> tp.Operand:
    op = tp.Operand()
    if not isinstance(expr, BinOp):
        terms = [(1, QUADRANT_VIEW[expr.name])]
    elif fly:
        terms = [(coef, QUADRANT_VIEW[leaf.name]) for coef, leaf in expand_terms(expr)]
    else:
        terms = [(1, PRESUM_VIEW[expr.name])]
    op.nterms = len(terms)
    for i, (coef, view) in enumerate(terms):
        op.view[i] = view
        op.coef[i] = coef
    return op


class ProgramBuilder:
    def __init__(self, products: Dict[str, BinOp], fly: bool):
        self.pg = tp.Program()
        self.products = products
        self.fly = fly

    def product(self, name: str, slot: int, accumulate: int = 0, negate: int = 0, wait_free: int = 1, commit: int = 1,
                a_view: Optional[int] = None, b_view: Optional[int] = None):
        pr = self.pg.product[self.pg.nproducts]
        if name in self.products:
            node = self.products[name]
            pr.a, pr.b = _operand(node.op1, self.fly), _operand(node.op2, self.fly)
        else:  # level 0: whole operands
            pr.a.nterms, pr.a.view[0], pr.a.coef[0] = 1, a_view, 1
            pr.b.nterms, pr.b.view[0], pr.b.coef[0] = 1, b_view, 1
        pr.slot, pr.accumulate, pr.negate, pr.wait_free, pr.commit = slot, accumulate, negate, wait_free, commit
        if pr.a.nterms > 1 or pr.b.nterms > 1:
            self.pg.needs_feed = 1
        self.pg.nproducts += 1
        return self

    def epilogue(self, slots: Sequence[int], srcs: Sequence[int], wait: Sequence[int], release: Sequence[int],
                 dst_kind: int, dst: int, signs: Optional[Sequence[int]] = None):
        ep = self.pg.epilogue[self.pg.nepilogues]
        ep.nslots = len(slots)
        for i, s in enumerate(slots):
            ep.slot[i] = s
            ep.slot_sign[i] = 1 if signs is None else signs[i]
        ep.nsrc = len(srcs)
        for i, s in enumerate(srcs):
            ep.src[i] = s
        ep.wait_full_mask = sum(1 << s for s in wait)
        ep.release_mask = sum(1 << s for s in release)
        ep.dst_kind, ep.dst = dst_kind, dst
        self.pg.epilogue_after[self.pg.nepilogues] = self.pg.nproducts - 1
        self.pg.nepilogues += 1
        return self


def _products_by_name(ms) -> Dict[str, BinOp]:
    return {m.name: m for m in ms}


def level0_program() -> tp.Program:
    b = ProgramBuilder({}, fly=False)
    b.pg.alternate_slots = 1
    b.product("whole", P, a_view=0, b_view=8)
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=0, dst=0)
    return b.pg


def level1_full_program(ms, fly: bool) -> tp.Program:
    """All seven products of a tile in one CTA, two TMEM slots, one fp32 hand-off (M4)."""
    b = ProgramBuilder(_products_by_name(ms), fly)
    b.product("m1", Q).product("m0", P)
    b.epilogue([P, Q], [], wait=[P, Q], release=[P, Q], dst_kind=0, dst=0)          # c0 = m0 + m1
    b.product("m4", Q).product("m2", P, accumulate=1)                                # P = m0 + m2 (v1)
    b.epilogue([Q], [], wait=[Q], release=[Q], dst_kind=1, dst=WS_M4)                # hand-off: m4
    b.product("m5", Q, accumulate=1)                                                 # Q = m4 + m5
    b.epilogue([P, Q], [], wait=[P, Q], release=[P, Q], dst_kind=0, dst=1)          # c1 = v1 + m4 + m5
    b.product("m3", P, accumulate=1)                                                 # P = v2
    b.epilogue([P], [WS_M4], wait=[P], release=[P], dst_kind=0, dst=3)               # c3 = v2 + m4
    b.product("m6", P, accumulate=1, negate=1)                                       # P = v2 - m6
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=0, dst=2)                    # c2
    return b.pg


def level1_first_program(ms) -> tp.Program:
    """Launch 1 of the interleaved-presum plan: the two products that need no presum (K1 and the first K4)."""
    b = ProgramBuilder(_products_by_name(ms), fly=False)
    b.product("m0", P).product("m1", Q)
    b.epilogue([P], [], wait=[P], release=[], dst_kind=1, dst=WS_M0)                 # hand-off: m0 to launch 2
    b.epilogue([P, Q], [], wait=[Q], release=[P, Q], dst_kind=0, dst=0)              # c0
    return b.pg


def level1_second_program(ms) -> tp.Program:
    """Launch 2 of the interleaved-presum plan: the five products that read materialised presums."""
    b = ProgramBuilder(_products_by_name(ms), fly=False)
    b.product("m4", Q).product("m2", P)
    b.epilogue([Q], [], wait=[Q], release=[Q], dst_kind=1, dst=WS_M4)
    b.product("m5", Q, accumulate=1)
    b.epilogue([P, Q], [WS_M0], wait=[P, Q], release=[P, Q], dst_kind=0, dst=1)      # c1 = m0 + m2 + m4 + m5
    b.product("m3", P, accumulate=1)
    b.epilogue([P], [WS_M0, WS_M4], wait=[P], release=[P], dst_kind=0, dst=3)        # c3 = m0 + m2 + m3 + m4
    b.product("m6", P, accumulate=1, negate=1)
    b.epilogue([P], [WS_M0], wait=[P], release=[P], dst_kind=0, dst=2)               # c2 = m0 + m2 + m3 - m6
    return b.pg


def level1_second_taps_program(ms) -> tp.Program:
    """Launch 2 with short taps: a product never waits for an epilogue step that reads global memory.  Hand-offs:
    m4, u = m2, v = m2 + m3 (and m0 from launch 1); c1 and c3 are summed from hand-offs off the critical path."""
    b = ProgramBuilder(_products_by_name(ms), fly=False)
    b.product("m4", Q).product("m2", P)
    b.epilogue([Q], [], wait=[Q], release=[Q], dst_kind=1, dst=WS_M4)
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=1, dst=WS_U)
    b.product("m5", Q).product("m3", P, accumulate=1)
    b.epilogue([Q], [WS_M0, WS_U, WS_M4], wait=[Q], release=[Q], dst_kind=0, dst=1)  # c1 = m0 + m2 + m4 + m5
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=1, dst=WS_V)
    b.product("m6", P, accumulate=1, negate=1)
    b.epilogue([], [WS_M0, WS_V, WS_M4], wait=[], release=[], dst_kind=0, dst=3)     # c3 = m0 + m2 + m3 + m4
    b.epilogue([P], [WS_M0], wait=[P], release=[P], dst_kind=0, dst=2)               # c2 = m0 + m2 + m3 - m6
    return b.pg


def all_programs() -> Dict[str, tp.Program]:
    """The named tables, generated from the DSL (names as in `sb200_tile_program`)."""
    from .algos.strassen_winograd_level1 import strassen_winograd

    _, ms = strassen_winograd(4, 4, 4)
    return {
        "level0": level0_program(),
        "level1_full_fly": level1_full_program(ms, fly=True),
        "level1_full_ws": level1_full_program(ms, fly=False),
        "level1_first": level1_first_program(ms),
        "level1_second": level1_second_program(ms),
        "level1_second_taps": level1_second_taps_program(ms),
    }


def verify_programs(programs: Dict[str, tp.Program]) -> None:
    """Protocol and algebra of every table; the expected outputs come from the DSL's own postsum expressions."""
    from .algos.strassen_winograd_level1 import strassen_winograd

    c, _ = strassen_winograd(4, 4, 4)
    want = {q: bilinear_form(part) for q, part in enumerate(c.parts)}
    tp.check_program(programs["level0"], level=0)
    for name in ("level1_full_fly", "level1_full_ws"):
        got = tp.check_program(programs[name], level=1)["outputs"]
        for q in range(4):
            assert np.array_equal(got[q], want[q]), (name, q)
    r1 = tp.check_program(programs["level1_first"], level=1, expect=[0])
    assert np.array_equal(r1["outputs"][0], want[0])
    for name in ("level1_second", "level1_second_taps"):
        r2 = tp.check_program(programs[name], level=1, ws_in=r1["ws"], expect=[1, 2, 3])
        for q in (1, 2, 3):
            assert np.array_equal(r2["outputs"][q], want[q]), (name, q)


# --------------------------------------------------------------------------------------------- schedule -> plan
def plan_for_schedule(schedule: list, level: int, mnk: Tuple[int, int, int], dtype: str) -> dict:
    """Map a schedule of the generator (K1/K2/K4 vocabulary) to launches of this library.

      ['K2(..)']                       -> one launch: all seven products per tile, presums formed in shared memory
      ['K1(m0)', 'K4(m1)', ... 'K4(m6)'] -> two launches: {m0, m1} + presum materialisation, then {m4, m2, m5, m3, m6}
    Level 2 and deeper apply the level-1 plan to the half-size problem of every K4 branch.
    """
    m, n, k = mnk
    if level <= 0:
        return {"level": 0, "kernel": f"blackwell_{dtype}_cubic_2sm_256x256", "launches": [{"program": "level0"}]}
    labels = [s if isinstance(s, str) else next(iter(s)) for s in schedule]
    if len(labels) == 1 and labels[0].startswith("K2("):
        plan = {"level": 1, "kernel": f"blackwell_{dtype}_sw_fused_presum",
                "launches": [{"program": "level1_full_fly", "products": ["m1", "m0", "m4", "m2", "m5", "m3", "m6"],
                              "presum": "formed in shared memory by the presum warps"}]}
    else:
        plan = {"level": 1, "kernel": f"blackwell_{dtype}_sw_interleaved_presum_2sm",
                "launches": [{"program": "level1_first", "products": ["m0", "m1"],
                              "presum": "materialised by the presum warps of this launch"},
                             {"program": "level1_second_taps", "products": ["m4", "m2", "m5", "m3", "m6"],
                              "presum": "read from the workspace by TMA"}]}
    plan["mnk"] = [m, n, k]
    if level > 1:
        plan["level"] = level
        plan["children"] = {}
        for item in schedule:
            if isinstance(item, dict):
                for label, child in item.items():
                    plan["children"][label] = plan_for_schedule(child, level - 1, (m // 2, n // 2, k // 2), dtype)
    return plan


def program_to_dict(pg: tp.Program) -> dict:
    def operand(op):
        return [[int(op.coef[i]), tp.VIEW_NAMES[op.view[i]]] for i in range(op.nterms)]

    return {
        "alternate_slots": int(pg.alternate_slots), "needs_feed": int(pg.needs_feed),
        "products": [{"a": operand(pr.a), "b": operand(pr.b), "slot": int(pr.slot), "accumulate": int(pr.accumulate),
                      "negate": int(pr.negate), "wait_free": int(pr.wait_free), "commit": int(pr.commit)}
                     for pr in (pg.product[i] for i in range(pg.nproducts))],
        "epilogues": [{"slots": [[int(ep.slot_sign[i]), int(ep.slot[i])] for i in range(ep.nslots)],
                       "sources": [int(ep.src[i]) for i in range(ep.nsrc)], "wait_full_mask": int(ep.wait_full_mask),
                       "release_mask": int(ep.release_mask), "dst_kind": int(ep.dst_kind), "dst": int(ep.dst),
                       "after_product": int(pg.epilogue_after[j])}
                      for j, ep in ((j, pg.epilogue[j]) for j in range(pg.nepilogues))],
    }


def program_to_c(name: str, pg: tp.Program) -> str:
    """A C initialiser of `sb200_program_t` (csrc/tile_program.h) as raw bytes, plus a readable comment."""
    raw = tp.to_bytes(pg)
    lines = [f"/* tile program '{name}': {pg.nproducts} products, {pg.nepilogues} epilogue steps */",
             f"static const unsigned char sb200_program_{name}[{len(raw)}] = {{"]
    for i in range(0, len(raw), 24):
        lines.append("  " + ", ".join(str(b) for b in raw[i:i + 24]) + ",")
    lines.append("};")
    return "\n".join(lines) + "\n"


def artefacts(schedule: list, fusion: Optional[dict], plan: dict) -> Dict[str, str]:
    programs = all_programs()
    verify_programs(programs)
    used = sorted({launch["program"] for launch in plan.get("launches", [])})
    files = {"schedule.json": json.dumps({"schedule": schedule, "fusion": fusion, "plan": plan}, indent=1, default=list)}
    files["tile_programs.json"] = json.dumps({name: program_to_dict(programs[name]) for name in used}, indent=1)
    files["sw_tile_programs.inc"] = "".join(program_to_c(name, programs[name]) for name in used)
    return files
