"""Emitter: from the algorithm DSL and a schedule to the tile programs the Blackwell kernels interpret.

The reference front end prints its schedules and copies pre-written example sources (src/compile.py:48-131,
646-653); nothing downstream reads the schedule.  Here the schedule selects a launch plan of this library's
kernels, and the per-tile programs of every launch (product order, operand term lists, tensor-memory slot plan,
postsum steps) are GENERATED from the DSL expressions and checked (`tile_program.check_program`) before they are
written out.  The tables the CUDA library runs are these tables: the build (subcuber_b200/build.py) calls
`generate_tables` and compiles its output (csrc/sw_tile_programs.inc, included by csrc/sw_programs.h) into the
library; no tile program is written by hand on the C++ side.
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
# Strassen's original algorithm with materialised presums: ten two-term presums, five per side.  Four use the presum
# view slots of their side; the fifth takes the slot of a raw quadrant that no product of the algorithm reads alone
# (a1 and b1).  The order of a side's list is the order of the presum workspace.
STRASSEN_PRESUM_VIEW = {"a03": 4, "a23": 5, "a01": 6, "a20": 7, "a13": 1,
                        "b03": 12, "b13": 13, "b20": 14, "b01": 15, "b23": 9}
P, Q = 0, 1
WS_M0, WS_M4, WS_U, WS_V = 0, 1, 2, 2  # u is dead once c1 is formed, before v is written: one buffer
WS_T1, WS_T4 = 1, 2                     # Strassen's original algorithm: taps of m1 and m4 (per-CTA scratch tiles)
WS_M0_CTA = 3                           # one-launch plan: m0 never leaves the CTA, it lives in a per-CTA scratch tile


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
def _operand(expr: Matrix, fly: bool, presum_view: Optional[Dict[str, int]] = None) -> tp.Operand:
    op = tp.Operand()
    if not isinstance(expr, BinOp):
        terms = [(1, QUADRANT_VIEW[expr.name])]
    elif fly:
        terms = [(coef, QUADRANT_VIEW[leaf.name]) for coef, leaf in expand_terms(expr)]
    else:
        terms = [(1, (presum_view or PRESUM_VIEW)[expr.name])]
    op.nterms = len(terms)
    for i, (coef, view) in enumerate(terms):
        op.view[i] = view
        op.coef[i] = coef
    return op


class ProgramBuilder:
    def __init__(self, products: Dict[str, BinOp], fly: bool, presum_view: Optional[Dict[str, int]] = None):
        self.pg = tp.Program()
        self.products = products
        self.fly = fly
        self.presum_view = presum_view

    def product(self, name: str, slot: int, accumulate: int = 0, negate: int = 0, wait_free: int = 1, commit: int = 1,
                a_view: Optional[int] = None, b_view: Optional[int] = None):
        pr = self.pg.product[self.pg.nproducts]
        if name in self.products:
            node = self.products[name]
            pr.a = _operand(node.op1, self.fly, self.presum_view)
            pr.b = _operand(node.op2, self.fly, self.presum_view)
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


def level1_first_early_program(ms) -> tp.Program:
    """Launch 1 with an early release of slot P: c0 is summed from the m0 hand-off tile and slot Q, so the next tile's
    first product never waits for an epilogue step (used when the launch is not tied into a level above)."""
    b = ProgramBuilder(_products_by_name(ms), fly=False)
    b.product("m0", P).product("m1", Q)
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=1, dst=WS_M0)
    b.epilogue([Q], [WS_M0], wait=[Q], release=[Q], dst_kind=0, dst=0)               # c0 = m0 + m1
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
    """Launch 2, the plan in use: no product waits for an epilogue step that has not had a whole product's time.
    Every product's slot is read by an epilogue step while the other slot's product runs; m6 goes to slot Q
    (c2 = v - Q) so that the step after m3 overlaps it; slot roles swap from tile to tile.  Hand-offs: m4,
    u = m0 + m2, v = u + m3 (written over u, which is dead once c1 is formed), and m0 from launch 1, which is read
    once - it is the one hand-off that comes from DRAM.  No step reads more than two hand-off tiles."""
    b = ProgramBuilder(_products_by_name(ms), fly=False)
    b.pg.alternate_slots = 1
    b.product("m4", Q).product("m2", P)
    b.epilogue([Q], [], wait=[Q], release=[Q], dst_kind=1, dst=WS_M4)
    b.epilogue([P], [WS_M0], wait=[P], release=[P], dst_kind=1, dst=WS_U)            # u = m0 + m2
    b.product("m5", Q).product("m3", P)
    b.epilogue([Q], [WS_U, WS_M4], wait=[Q], release=[Q], dst_kind=0, dst=1)         # c1 = u + m4 + m5
    b.epilogue([P], [WS_U], wait=[P], release=[P], dst_kind=1, dst=WS_V)             # v = u + m3
    b.product("m6", Q)
    b.epilogue([], [WS_V, WS_M4], wait=[], release=[], dst_kind=0, dst=3)            # c3 = v + m4
    b.epilogue([Q], [WS_V], wait=[Q], release=[Q], dst_kind=0, dst=2, signs=[-1])    # c2 = v - m6
    return b.pg


def level1_merged_program(ms) -> tp.Program:
    """All seven products of a tile in ONE launch with materialised presums (the presum warps of the same launch
    publish them panel by panel; m0 and m1, which read raw quadrants, come first and cover the start).  Every product
    goes to the slot the step before last has released, every slot is read by an epilogue step while the other slot's
    product runs, and with seven products the slot roles swap from tile to tile.  Hand-offs stay in per-CTA scratch
    tiles: m0, m4, u = m0 + m2, v = u + m3 (over u).  No step reads more than two of them."""
    b = ProgramBuilder(_products_by_name(ms), fly=False)
    b.pg.alternate_slots = 1
    b.product("m0", P).product("m1", Q)
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=1, dst=WS_M0_CTA)             # m0            (during m1)
    b.product("m4", P)
    b.epilogue([Q], [WS_M0_CTA], wait=[Q], release=[Q], dst_kind=0, dst=0)            # c0 = m0 + m1  (during m4)
    b.product("m2", Q)
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=1, dst=WS_M4)                 # m4            (during m2)
    b.product("m5", P)
    b.epilogue([Q], [WS_M0_CTA], wait=[Q], release=[Q], dst_kind=1, dst=WS_U)         # u = m0 + m2   (during m5)
    b.product("m3", Q)
    b.epilogue([P], [WS_U, WS_M4], wait=[P], release=[P], dst_kind=0, dst=1)          # c1 = u + m4 + m5 (during m3)
    b.product("m6", P)
    b.epilogue([Q], [WS_U], wait=[Q], release=[Q], dst_kind=1, dst=WS_V)              # v = u + m3    (during m6)
    b.epilogue([], [WS_V, WS_M4], wait=[], release=[], dst_kind=0, dst=3)             # c3 = v + m4
    b.epilogue([P], [WS_V], wait=[P], release=[P], dst_kind=0, dst=2, signs=[-1])     # c2 = v - m6   (during next m0)
    return b.pg


def level1_strassen_program(ms, fly: bool = True) -> tp.Program:
    """Strassen's original algorithm (algos/strassen_level1.py), all seven products of a tile in one CTA.  Operand
    sums are formed on the fly (fly=True) or read from the presum workspace (fly=False: STRASSEN_PRESUM_VIEW, a launch
    of its own materialises them first).  Slot P accumulates m1 + m7, then m3 + m6; slot Q accumulates m4 - m5, then
    holds m2; m1 and m4 are tapped into fp32 tiles before their slots go on accumulating:
        c0 = P + Q          c1 = m3 - (m4 - m5) + m4          c2 = m2 + m4          c3 = (m3 + m6) - m2 + m1"""
    b = ProgramBuilder(_products_by_name(ms), fly=fly, presum_view=STRASSEN_PRESUM_VIEW)
    b.product("m1", P)
    b.epilogue([P], [], wait=[P], release=[P], dst_kind=1, dst=WS_T1)                # tap: m1
    b.product("m4", Q)
    b.epilogue([Q], [], wait=[Q], release=[Q], dst_kind=1, dst=WS_T4)                # tap: m4
    b.product("m7", P, accumulate=1).product("m5", Q, accumulate=1, negate=1)
    b.epilogue([P, Q], [], wait=[P, Q], release=[P], dst_kind=0, dst=0)              # c0 = (m1 + m7) + (m4 - m5)
    b.product("m3", P)
    b.epilogue([P, Q], [WS_T4], wait=[P], release=[P, Q], dst_kind=0, dst=1, signs=[1, -1])  # c1 = m3 + m5
    b.product("m6", P, accumulate=1).product("m2", Q)
    b.epilogue([Q], [WS_T4], wait=[Q], release=[], dst_kind=0, dst=2)                # c2 = m2 + m4
    b.epilogue([P, Q], [WS_T1], wait=[P], release=[P, Q], dst_kind=0, dst=3, signs=[1, -1])  # c3
    return b.pg


# ------------------------------------------------------------------------------------------------------ level 2
# One outer recursion step: the same algorithm over half-size blocks, every outer product a level-1 group (two
# launches).  The outer postsums ride on the groups' epilogue steps through three fp32 chain buffers X0, X1, X2:
#   m0: X0 = m0 | m1: c0 = X0 + m1 | m2: X1 = X0 + m2 | m4: X2 = m4, X0 = X2 + X1 | m5: c1 = X0 + m5
#   m3: X0 = X1 + m3, c3 = X0 + X2 | m6: c2 = X0 - m6
# Fields: link = (dst_fp32, src, extra, negate) as in csrc/sw_programs.h `OuterLink`; dst/src/src2/extra_dst = X ids.
LEVEL2_CHAIN = [
    # name, link,          dst, src, src2, extra_dst, out quadrant
    ("m0", (1, 0, 0, 0), 0, -1, -1, -1, -1),
    ("m1", (0, 1, 0, 0), -1, 0, -1, -1, 0),
    ("m2", (1, 1, 0, 0), 1, 0, -1, -1, -1),
    ("m4", (1, 0, 1, 0), 2, -1, 1, 0, -1),
    ("m5", (0, 1, 0, 0), -1, 0, -1, -1, 1),
    ("m3", (1, 1, 2, 0), 0, 1, 2, -1, 3),
    ("m6", (0, 1, 0, 1), -1, 0, -1, -1, 2),
]


def strassen_presum_table(ms) -> Dict[str, List[Tuple[int, int, int, int, int]]]:
    """Per side ("a", "b"): the presums of Strassen's original algorithm in workspace order, each as
    (view slot, quadrant 0, coefficient 0, quadrant 1, coefficient 1), taken from the operands of the DSL products."""
    found: Dict[str, Tuple[int, int, int, int, int]] = {}
    for m in ms:
        for expr in (m.op1, m.op2):
            if isinstance(expr, BinOp):
                (c0, l0), (c1, l1) = expand_terms(expr)
                found[expr.name] = (STRASSEN_PRESUM_VIEW[expr.name], QUADRANT_VIEW[l0.name] % 8, c0,
                                    QUADRANT_VIEW[l1.name] % 8, c1)
    assert set(found) == set(STRASSEN_PRESUM_VIEW)
    order = list(STRASSEN_PRESUM_VIEW)
    return {"a": [found[n] for n in order if n.startswith("a")], "b": [found[n] for n in order if n.startswith("b")]}


def strassen_view_coef(ms) -> Dict[int, Tuple[int, ...]]:
    """What every view slot holds under the presum plan of Strassen's original algorithm (for `check_program`)."""
    out: Dict[int, Tuple[int, ...]] = {}
    for side in strassen_presum_table(ms).values():
        for view, q0, c0, q1, c1 in side:
            v = [0, 0, 0, 0]
            v[q0] += c0
            v[q1] += c1
            out[view] = tuple(v)
    return out


def operand_code(expr: Matrix) -> int:
    """0..3 = raw quadrant, 4..7 = presum (the order of the presum workspace), for an operand of a DSL product."""
    if not isinstance(expr, BinOp):
        return QUADRANT_VIEW[expr.name] % 8
    return 4 + PRESUM_VIEW[expr.name] % 4


def level2_children(ms) -> List[dict]:
    """The seven level-1 groups of a level-2 run in execution order, operands taken from the DSL products."""
    by_name = _products_by_name(ms)
    out = []
    for name, link, dst, src, src2, extra_dst, quadrant in LEVEL2_CHAIN:
        node = by_name[name]
        out.append({"name": name, "a": operand_code(node.op1), "b": operand_code(node.op2), "link": link, "dst": dst,
                    "src": src, "src2": src2, "extra_dst": extra_dst, "out_quadrant": quadrant})
    return out


def link_outer(base: tp.Program, link: Tuple[int, int, int, int], launch: int) -> tp.Program:
    """Tie a level-1 program into the outer chain (same rewriting as csrc/sw_programs.h `link_outer`)."""
    dst_fp32, src, extra, negate = link
    pg = tp.Program.from_buffer_copy(tp.to_bytes(base))
    C.memset(C.byref(pg.epilogue), 0, C.sizeof(pg.epilogue))
    C.memset(C.byref(pg.epilogue_after), 0, C.sizeof(pg.epilogue_after))
    pg.nepilogues = 0
    if negate:
        for i in range(pg.nproducts):
            pg.product[i].negate ^= 1

    def push(e: tp.Epilogue, after: int):
        C.memmove(C.byref(pg.epilogue[pg.nepilogues]), C.byref(e), C.sizeof(tp.Epilogue))
        pg.epilogue_after[pg.nepilogues] = after
        pg.nepilogues += 1

    def push_extra(q: int, after: int):
        e = tp.Epilogue()
        e.nsrc = 2
        e.src[0], e.src[1] = tp.WS_OUTER_DST + q, tp.WS_OUTER_SRC2 + q
        e.dst_kind = 1 if extra == 1 else 0
        e.dst = tp.WS_EXTRA_DST + q if extra == 1 else q
        push(e, after)

    if launch == 2 and extra:
        push_extra(0, 0)
    for i in range(base.nepilogues):
        e = tp.Epilogue.from_buffer_copy(bytes(memoryview(base.epilogue[i])))
        after = base.epilogue_after[i]
        if e.dst_kind != 0:
            push(e, after)
            continue
        q = e.dst
        if src:
            e.src[e.nsrc] = tp.WS_OUTER_SRC + q
            e.nsrc += 1
        if dst_fp32:
            e.dst_kind, e.dst = 1, tp.WS_OUTER_DST + q
        push(e, after)
        if launch == 2 and extra:
            push_extra(q, after)
    return pg


def run_program_numeric(pg: tp.Program, views: Dict[int, np.ndarray], ws: Dict[int, np.ndarray],
                        out: Dict[int, np.ndarray]) -> None:
    """Execute a tile program on whole blocks with numpy (one 'tile' = one block): products in order, every epilogue
    step as soon as the product it follows has been issued.  Protocol questions are `check_program`'s business."""
    slots: Dict[int, np.ndarray] = {}

    def operand(op):
        return sum(int(op.coef[t]) * views[op.view[t]] for t in range(op.nterms))

    e = 0
    for i in range(pg.nproducts):
        pr = pg.product[i]
        val = operand(pr.a) @ operand(pr.b) * (-1 if pr.negate else 1)
        slots[pr.slot] = slots[pr.slot] + val if pr.accumulate else val
        while e < pg.nepilogues and pg.epilogue_after[e] <= i:
            ep = pg.epilogue[e]
            acc = 0
            for t in range(ep.nsrc):
                acc = acc + ws[ep.src[t]]
            for t in range(ep.nslots):
                acc = acc + int(ep.slot_sign[t]) * slots[ep.slot[t]]
            if ep.dst_kind == 1:
                ws[ep.dst] = acc
            else:
                out[ep.dst] = acc
            e += 1
    assert e == pg.nepilogues


def _quadrants(x: np.ndarray) -> List[np.ndarray]:
    r, c = x.shape[0] // 2, x.shape[1] // 2
    return [x[:r, :c], x[:r, c:], x[r:, :c], x[r:, c:]]


def _presums(quads: List[np.ndarray], side: str) -> List[np.ndarray]:
    names = ["S1", "S2", "A02", "A1S2"] if side == "a" else ["B10", "B31", "S3", "S3B2"]
    return [sum(cf * quads[i] for i, cf in enumerate(tp.VIEW_COEF[nm])) for nm in names]


def simulate_level1(first: tp.Program, second: tp.Program, a: np.ndarray, b: np.ndarray, ws: Dict[int, np.ndarray],
                    out: Dict[int, np.ndarray]) -> None:
    qa, qb = _quadrants(a), _quadrants(b)
    views = {i: v for i, v in enumerate(qa + _presums(qa, "a") + qb + _presums(qb, "b"))}
    run_program_numeric(first, views, ws, out)
    run_program_numeric(second, views, ws, out)


def simulate_level2(programs: Dict[str, tp.Program], children: List[dict], a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """The whole level-2 launch plan on integer matrices: returns the product it computes."""
    qa, qb = _quadrants(a), _quadrants(b)
    oa, ob = qa + _presums(qa, "a"), qb + _presums(qb, "b")
    x: Dict[int, Dict[int, np.ndarray]] = {0: {}, 1: {}, 2: {}}   # chain buffer -> inner quadrant -> block
    mh, nh = a.shape[0] // 2, b.shape[1] // 2
    c = np.zeros((a.shape[0], b.shape[1]), dtype=a.dtype)
    for ch in children:
        ws: Dict[int, np.ndarray] = {}
        for q in range(4):
            if ch["src"] >= 0:
                ws[tp.WS_OUTER_SRC + q] = x[ch["src"]][q]
            if ch["src2"] >= 0:
                ws[tp.WS_OUTER_SRC2 + q] = x[ch["src2"]][q]
        out: Dict[int, np.ndarray] = {}
        simulate_level1(programs[f"level2_{ch['name']}_launch1"], programs[f"level2_{ch['name']}_launch2"],
                        oa[ch["a"]], ob[ch["b"]], ws, out)
        for q in range(4):
            if ch["dst"] >= 0:
                x[ch["dst"]][q] = ws[tp.WS_OUTER_DST + q]
            if ch["extra_dst"] >= 0:
                x[ch["extra_dst"]][q] = ws[tp.WS_EXTRA_DST + q]
        if ch["out_quadrant"] >= 0:
            oq = ch["out_quadrant"]
            r0, c0 = (oq >> 1) * mh, (oq & 1) * nh
            for q in range(4):
                rr, cc = r0 + (q >> 1) * (mh // 2), c0 + (q & 1) * (nh // 2)
                c[rr:rr + mh // 2, cc:cc + nh // 2] = out[q]
    return c


def all_programs() -> Dict[str, tp.Program]:
    """The named tables, generated from the DSL (names as in `sb200_tile_program`)."""
    from .algos.strassen_winograd_level1 import strassen_winograd

    from .algos.strassen_level1 import strassen

    _, ms = strassen_winograd(4, 4, 4)
    return {
        "level0": level0_program(),
        "level1_strassen": level1_strassen_program(strassen(4, 4, 4)[1]),
        "level1_strassen_presum": level1_strassen_program(strassen(4, 4, 4)[1], fly=False),
        "level1_full_fly": level1_full_program(ms, fly=True),
        "level1_full_ws": level1_full_program(ms, fly=False),
        "level1_first": level1_first_program(ms),
        "level1_first_early": level1_first_early_program(ms),
        "level1_second": level1_second_program(ms),
        "level1_second_taps": level1_second_taps_program(ms),
        "level1_merged": level1_merged_program(ms),
        **{f"level2_{ch['name']}_launch{launch}":
           link_outer(level1_first_program(ms) if launch == 1 else level1_second_taps_program(ms), ch["link"], launch)
           for ch in level2_children(ms) for launch in (1, 2)},
    }


def verify_programs(programs: Dict[str, tp.Program]) -> None:
    """Protocol and algebra of every table; the expected outputs come from the DSL's own postsum expressions."""
    from .algos.strassen_winograd_level1 import strassen_winograd

    c, _ = strassen_winograd(4, 4, 4)
    want = {q: bilinear_form(part) for q, part in enumerate(c.parts)}
    tp.check_program(programs["level0"], level=0)
    for name in ("level1_full_fly", "level1_full_ws", "level1_merged"):
        got = tp.check_program(programs[name], level=1, tiles=5)["outputs"]
        for q in range(4):
            assert np.array_equal(got[q], want[q]), (name, q)
    # Strassen's original algorithm: its own postsum expressions must give the same four blocks
    from .algos.strassen_level1 import strassen

    got = tp.check_program(programs["level1_strassen"], level=1)["outputs"]
    for q, part in enumerate(strassen(4, 4, 4)[0].parts):
        assert np.array_equal(bilinear_form(part), want[q]) and np.array_equal(got[q], want[q]), ("level1_strassen", q)
    got = tp.check_program(programs["level1_strassen_presum"], level=1,
                           view_coef=strassen_view_coef(strassen(4, 4, 4)[1]))["outputs"]
    for q in range(4):
        assert np.array_equal(got[q], want[q]), ("level1_strassen_presum", q)
    assert programs["level1_strassen_presum"].needs_feed == 0
    for name in ("level1_first_early", "level1_first"):
        r1 = tp.check_program(programs[name], level=1, expect=[0])
        assert np.array_equal(r1["outputs"][0], want[0]), name
    for name in ("level1_second", "level1_second_taps"):
        r2 = tp.check_program(programs[name], level=1, ws_in=r1["ws"], expect=[1, 2, 3])
        for q in (1, 2, 3):
            assert np.array_equal(r2["outputs"][q], want[q]), (name, q)
    # level 2: the protocol of every rewritten program, then the whole 14-launch plan on integer matrices
    _, ms = strassen_winograd(4, 4, 4)
    children = level2_children(ms)
    outer = {i: np.zeros((4, 4), dtype=np.int64) for i in range(tp.WS_OUTER_DST, tp.NUM_WS)}
    for ch in children:
        r1 = tp.check_program(programs[f"level2_{ch['name']}_launch1"], level=1, ws_in=outer, algebra=False)
        tp.check_program(programs[f"level2_{ch['name']}_launch2"], level=1, ws_in={**outer, **r1["ws"]}, algebra=False)
    rng = np.random.default_rng(7)
    a = rng.integers(-3, 4, size=(8, 12)).astype(np.int64)
    b = rng.integers(-3, 4, size=(12, 16)).astype(np.int64)
    assert np.array_equal(simulate_level2(programs, children, a, b), a @ b)


# --------------------------------------------------------------------------------------------- schedule -> plan
def plan_for_schedule(schedule: list, level: int, mnk: Tuple[int, int, int], dtype: str,
                      algorithm: str = "strassen_winograd") -> dict:
    """Map a schedule of the generator (K1/K2/K4 vocabulary) to launches of this library.

    algorithm "strassen" (Strassen's original algorithm, algos/strassen_level1.py) has one plan: level 1, all seven
    products of a tile in one launch with the operand sums formed in shared memory.

      ['K2(..)']                       -> one launch: all seven products per tile, presums formed in shared memory
      ['K1(m0)', 'K4(m1)', ... 'K4(m6)'] -> two launches: {m0, m1} + presum materialisation, then {m4, m2, m5, m3, m6}
    Level 2 and deeper apply the level-1 plan to the half-size problem of every K4 branch.
    """
    m, n, k = mnk
    if level <= 0:
        return {"level": 0, "kernel": f"blackwell_{dtype}_cubic_2sm_256x256", "launches": [{"program": "level0"}]}
    if algorithm == "strassen":
        if level != 1:
            raise ValueError("Strassen's original algorithm is planned for level 1 only")
        return {"level": 1, "algorithm": "strassen", "kernel": f"blackwell_{dtype}_strassen_fused_presum_2sm",
                "mnk": [m, n, k],
                "launches": [{"program": "level1_strassen", "products": ["m1", "m4", "m7", "m5", "m3", "m6", "m2"],
                              "presum": "formed in shared memory by the presum warps"}]}
    if algorithm != "strassen_winograd":
        raise ValueError(f"unknown algorithm '{algorithm}'")
    labels = [s if isinstance(s, str) else next(iter(s)) for s in schedule]
    if len(labels) == 1 and labels[0].startswith("K2("):
        plan = {"level": 1, "kernel": f"blackwell_{dtype}_sw_fused_presum",
                "launches": [{"program": "level1_full_fly", "products": ["m1", "m0", "m4", "m2", "m5", "m3", "m6"],
                              "presum": "formed in shared memory by the presum warps"}]}
    else:
        plan = {"level": 1, "kernel": f"blackwell_{dtype}_sw_interleaved_presum_2sm",
                "launches": [{"program": "level1_first_early", "products": ["m0", "m1"],
                              "presum": "materialised by the presum warps of this launch"},
                             {"program": "level1_second_taps", "products": ["m4", "m2", "m5", "m3", "m6"],
                              "presum": "read from the workspace by TMA"}]}
    plan["mnk"] = [m, n, k]
    if level == 2:
        from .algos.strassen_winograd_level1 import strassen_winograd

        _, ms = strassen_winograd(4, 4, 4)
        plan["kernel"] = f"blackwell_{dtype}_sw_level2_2sm"
        plan["groups"] = [{"product": ch["name"], "a": ch["a"], "b": ch["b"],
                           "launches": [f"level2_{ch['name']}_launch1", f"level2_{ch['name']}_launch2"],
                           "outer_presum_job": {0: "A side", 1: "B side"}.get(i)}
                          for i, ch in enumerate(level2_children(ms))]
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


def generate_tables() -> str:
    """The C text the library compiles in (csrc/sw_tile_programs.inc): every tile program as the bytes of an
    `sb200_program_t`, a name index, and the seven groups of a level-2 run.  The programs are checked first."""
    from .algos.strassen_winograd_level1 import strassen_winograd

    programs = all_programs()
    verify_programs(programs)
    size = C.sizeof(tp.Program)
    out = ["/* Generated by subcuber_b200/emit.py from the algorithm DSL (subcuber_b200/algos) - do not edit.\n"
           "   Tile programs as the bytes of sb200_program_t (csrc/tile_program.h). */\n",
           f"#define SB200_EMITTED_PROGRAM_BYTES {size}\n"]
    for name in sorted(programs):
        out.append(program_to_c(name, programs[name]))
    out.append("static const struct sb200_emitted_program { const char* name; const unsigned char* bytes; } "
               "sb200_emitted_programs[] = {\n")
    for name in sorted(programs):
        out.append(f'  {{"{name}", sb200_program_{name}}},\n')
    out.append("};\n")
    out.append(f"#define SB200_NUM_EMITTED_PROGRAMS {len(programs)}\n")
    from .algos.strassen_level1 import strassen

    out.append("/* Presums of Strassen's original algorithm under its presum plan, per side (A, B) in workspace order: "
               "view slot that\n   reads the presum, then result = c0 * quadrant q0 + c1 * quadrant q1. */\n")
    out.append("static const struct sb200_presum_pair { int view, q0, c0, q1, c1; } sb200_strassen_presums[2][5] = {\n")
    table = strassen_presum_table(strassen(4, 4, 4)[1])
    for side in ("a", "b"):
        out.append("  {" + ", ".join("{%d, %d, %d, %d, %d}" % row for row in table[side]) + "},\n")
    out.append("};\n")
    _, ms = strassen_winograd(4, 4, 4)
    out.append("/* The seven level-1 groups of a level-2 run in execution order.  a, b: operand codes (0..3 raw outer "
               "quadrant, 4..7 outer presum);\n   dst, src, src2, extra_dst: outer chain buffers X0..X2 (-1 none); "
               "out_quadrant: quadrant of C written in the output type (-1 none). */\n")
    out.append("static const struct sb200_level2_child { const char* name; int a, b, dst, src, src2, extra_dst, "
               "out_quadrant; } sb200_level2_children[7] = {\n")
    for ch in level2_children(ms):
        out.append(f'  {{"{ch["name"]}", {ch["a"]}, {ch["b"]}, {ch["dst"]}, {ch["src"]}, {ch["src2"]}, {ch["extra_dst"]}, '
                   f'{ch["out_quadrant"]}}},\n')
    out.append("};\n")
    return "".join(out)


def artefacts(schedule: list, fusion: Optional[dict], plan: dict) -> Dict[str, str]:
    programs = all_programs()
    verify_programs(programs)
    used = sorted({launch["program"] for launch in plan.get("launches", [])} |
                  {name for group in plan.get("groups", []) for name in group["launches"]})
    files = {"schedule.json": json.dumps({"schedule": schedule, "fusion": fusion, "plan": plan}, indent=1, default=list)}
    files["tile_programs.json"] = json.dumps({name: program_to_dict(programs[name]) for name in used}, indent=1)
    files["sw_tile_programs.inc"] = "".join(program_to_c(name, programs[name]) for name in used)
    return files
