"""Tile programs: Python mirror of csrc/tile_program.h plus a checker.

A tile program is the per-output-tile schedule the persistent kernel interprets (product steps that
accumulate into tensor-memory slots, epilogue steps that apply the postsums).  It is the runtime form of what
the reference project expresses with compile-time schedule types (include/cutlass/gemm/device/strassen_decls.h:
RWCTypes / CUW / Plus / Neg / FusedMiGroup).  `check_program` proves two things about a table without a GPU:

  * the hand-over protocol is consistent: every slot alternates wait_free -> ... -> release and
    commit -> wait_full, both roles can run the program for several tiles in a row without blocking forever,
    and no epilogue step reads a slot while a product is still accumulating into it;
  * the algebra is right: with symbolic quadrants, the four outputs equal C0 = A0B0 + A1B2, C1 = A0B1 + A1B3,
    C2 = A2B0 + A3B2, C3 = A2B1 + A3B3 (level 1) or C = AB (level 0).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import numpy as np

MAX_TERMS = 4
MAX_PRODUCTS = 8
MAX_EPILOGUES = 12
MAX_SLOT_TERMS = 3
MAX_SRC_TERMS = 3
NUM_WS = 20
WS_OUTER_DST, WS_OUTER_SRC, WS_OUTER_SRC2, WS_EXTRA_DST = 4, 8, 12, 16

VIEW_NAMES = ["A0", "A1", "A2", "A3", "S1", "S2", "A02", "A1S2", "B0", "B1", "B2", "B3", "B10", "B31", "S3", "S3B2"]
# coefficient vectors of every view over (A0..A3) or (B0..B3):
#   src/algos/strassen_winograd_level1.py:16-25 in the reference project
VIEW_COEF = {
    "A0": (1, 0, 0, 0), "A1": (0, 1, 0, 0), "A2": (0, 0, 1, 0), "A3": (0, 0, 0, 1),
    "S1": (0, 0, 1, 1), "S2": (-1, 0, 1, 1), "A02": (1, 0, -1, 0), "A1S2": (1, 1, -1, -1),
    "B0": (1, 0, 0, 0), "B1": (0, 1, 0, 0), "B2": (0, 0, 1, 0), "B3": (0, 0, 0, 1),
    "B10": (-1, 1, 0, 0), "B31": (0, -1, 0, 1), "S3": (1, -1, 0, 1), "S3B2": (1, -1, -1, 1),
}


class Operand(C.Structure):
    _fields_ = [("nterms", C.c_int8), ("view", C.c_int8 * MAX_TERMS), ("coef", C.c_int8 * MAX_TERMS)]


class Product(C.Structure):
    _fields_ = [("a", Operand), ("b", Operand), ("slot", C.c_uint8), ("accumulate", C.c_uint8),
                ("negate", C.c_uint8), ("wait_free", C.c_uint8), ("commit", C.c_uint8), ("pad", C.c_uint8 * 3)]


class Epilogue(C.Structure):
    _fields_ = [("nslots", C.c_uint8), ("slot", C.c_uint8 * MAX_SLOT_TERMS), ("slot_sign", C.c_int8 * MAX_SLOT_TERMS),
                ("wait_full_mask", C.c_uint8), ("release_mask", C.c_uint8), ("nsrc", C.c_uint8),
                ("src", C.c_uint8 * MAX_SRC_TERMS), ("dst_kind", C.c_uint8), ("dst", C.c_uint8),
                ("pad", C.c_uint8 * 2)]


class Program(C.Structure):
    _fields_ = [("nproducts", C.c_int32), ("nepilogues", C.c_int32), ("alternate_slots", C.c_int32),
                ("needs_feed", C.c_int32), ("product", Product * MAX_PRODUCTS), ("epilogue", Epilogue * MAX_EPILOGUES),
                ("epilogue_after", C.c_uint8 * MAX_EPILOGUES)]


def from_library(which: str) -> Program:
    """The table compiled into the CUDA library under the name `which`."""
    from . import _lib

    lib = _lib.load()
    if lib.sb200_tile_program_bytes() != C.sizeof(Program):
        raise RuntimeError("tile_program.py is out of sync with csrc/tile_program.h")
    pg = Program()
    rc = lib.sb200_tile_program(which.encode(), C.byref(pg), C.sizeof(pg))
    if rc != 0:
        raise KeyError(which)
    return pg


def to_bytes(pg: Program) -> bytes:
    return bytes(memoryview(pg))


class ProgramError(ValueError):
    pass


def _operand_vector(op: Operand, view_coef: Optional[Dict[int, Sequence[int]]] = None) -> np.ndarray:
    v = np.zeros(4, dtype=np.int64)
    if not (1 <= op.nterms <= MAX_TERMS):
        raise ProgramError("operand with a bad term count")
    side = None
    for t in range(op.nterms):
        name = VIEW_NAMES[op.view[t]]
        s = "A" if op.view[t] < 8 else "B"
        if side is not None and s != side:
            raise ProgramError("operand mixes A-side and B-side views")
        side = s
        if op.coef[t] not in (1, -1):
            raise ProgramError("coefficients must be +1 or -1")
        coef = view_coef[op.view[t]] if view_coef and op.view[t] in view_coef else VIEW_COEF[name]
        v += op.coef[t] * np.array(coef, dtype=np.int64)
    if op.nterms == 1 and op.coef[0] != 1:
        raise ProgramError("a single-term operand is loaded by TMA and cannot carry a sign; use `negate`")
    return v


def check_program(pg: Program, level: int, nslots: int = 2, ws_in: Optional[Dict[int, np.ndarray]] = None,
                  expect: Optional[Sequence[int]] = None, tiles: int = 3, algebra: bool = True,
                  view_coef: Optional[Dict[int, Sequence[int]]] = None) -> Dict[str, object]:
    """Validate `pg`.  Returns {"outputs": {quadrant: 4x4 matrix}, "ws": {...}, "bubbles": n}.

    view_coef: what the views hold when that is not the Strassen-Winograd assignment of VIEW_COEF (view id ->
               coefficients over the side's four quadrants), for plans that put other presums in the view slots.

    ws_in: symbolic contents of workspace buffers written by an earlier launch.
    algebra: False checks the hand-over protocol only (programs tied into an outer recursion step do not produce
             the plain level-1 outputs).
    expect: output quadrants this program must write (default: all four at level 1, quadrant 0 at level 0).
    """
    np_, ne = pg.nproducts, pg.nepilogues
    if not (1 <= np_ <= MAX_PRODUCTS and 1 <= ne <= MAX_EPILOGUES):
        raise ProgramError("empty or oversized program")

    # ---- protocol: run MMA and epilogue roles as two agents over `tiles` tiles -------------------
    free = [1] * (2 * nslots)      # slot_free credits (one initial credit each)
    full = [0] * (2 * nslots)
    busy_until_commit = [False] * (2 * nslots)  # a product chain is accumulating and has not committed
    mma_pos, epi_pos = [0, 0], [0, 0]  # (tile, step)
    bubbles = 0
    slot_val: List[Optional[np.ndarray]] = [None] * (2 * nslots)
    ws: Dict[int, np.ndarray] = dict(ws_in or {})
    outputs: Dict[int, np.ndarray] = {}
    progress = True
    while progress:
        progress = False
        # MMA role: runs ahead as far as its credits allow
        while mma_pos[0] < tiles:
            t, s = mma_pos
            pr = pg.product[s]
            sx = (t & 1) if pg.alternate_slots else 0
            slot = pr.slot ^ sx
            if slot >= nslots:
                raise ProgramError("slot id out of range for this tile width")
            if pr.wait_free:
                if free[slot] == 0:
                    break
                free[slot] -= 1
            elif not busy_until_commit[slot]:
                raise ProgramError(f"product step {s} writes slot {slot} without owning it (needs wait_free)")
            a, b = _operand_vector(pr.a, view_coef), _operand_vector(pr.b, view_coef)
            if (pr.a.view[0] >= 8) or (pr.b.view[0] < 8):
                raise ProgramError("A operand must use A-side views and B operand B-side views")
            val = np.outer(a, b) * (-1 if pr.negate else 1)
            if pr.accumulate:
                if slot_val[slot] is None:
                    raise ProgramError("accumulating into an empty slot")
                slot_val[slot] = slot_val[slot] + val
            else:
                slot_val[slot] = val
            busy_until_commit[slot] = not pr.commit
            if pr.commit:
                full[slot] += 1
                if full[slot] > 1:
                    raise ProgramError("two commits on a slot without an epilogue wait between them")
            mma_pos = [t, s + 1] if s + 1 < np_ else [t + 1, 0]
            progress = True
        # epilogue role: one step at a time
        while epi_pos[0] < tiles:
            t, s = epi_pos
            ep = pg.epilogue[s]
            sx = (t & 1) if pg.alternate_slots else 0
            need = [sl ^ sx for sl in range(nslots) if (ep.wait_full_mask >> sl) & 1]
            if any(full[sl] == 0 for sl in need):
                break
            for sl in need:
                full[sl] -= 1
            acc = np.zeros((4, 4), dtype=np.int64)
            for i in range(ep.nslots):
                sl = ep.slot[i] ^ sx
                if slot_val[sl] is None or busy_until_commit[sl]:
                    raise ProgramError(f"epilogue step {s} reads slot {sl} that is not ready")
                acc = acc + ep.slot_sign[i] * slot_val[sl]
            for i in range(ep.nsrc):
                if ep.src[i] not in ws:
                    raise ProgramError(f"epilogue step {s} reads workspace buffer {ep.src[i]} before it is written")
                acc = acc + ws[ep.src[i]]
            if ep.dst_kind == 1:
                ws[ep.dst] = acc
            else:
                outputs[ep.dst] = acc
            for sl in range(nslots):
                if (ep.release_mask >> sl) & 1:
                    free[sl ^ sx] += 1
                    if free[sl ^ sx] > 1:
                        raise ProgramError("slot released twice without a product taking the credit")
            epi_pos = [t, s + 1] if s + 1 < ne else [t + 1, 0]
            progress = True
            # the MMA role may have been blocked on this release: count it as a bubble when it was
            if mma_pos[0] < tiles:
                pr = pg.product[mma_pos[1]]
                if pr.wait_free and (ep.release_mask >> (pr.slot)) & 1:
                    bubbles += 1
            break
    if mma_pos[0] < tiles or epi_pos[0] < tiles:
        raise ProgramError(f"deadlock: mma at {mma_pos}, epilogue at {epi_pos}")
    if any(f != 1 for f in free[:nslots]) or any(f != 0 for f in full[:nslots]):
        raise ProgramError("credits do not return to their initial state after a tile")

    if not algebra:
        return {"outputs": outputs, "ws": ws, "bubbles": bubbles // max(1, tiles)}

    # ---- algebra ---------------------------------------------------------------------------------
    want = {}
    if level == 0:
        w = np.zeros((4, 4), dtype=np.int64)
        w[0, 0] = 1
        want = {0: w}
    else:
        for q, pairs in {0: ((0, 0), (1, 2)), 1: ((0, 1), (1, 3)), 2: ((2, 0), (3, 2)), 3: ((2, 1), (3, 3))}.items():
            w = np.zeros((4, 4), dtype=np.int64)
            for (i, j) in pairs:
                w[i, j] = 1
            want[q] = w
    expect = list(want.keys()) if expect is None else list(expect)
    for q in expect:
        if q not in outputs:
            raise ProgramError(f"output quadrant {q} is never written")
        if not np.array_equal(outputs[q], want[q]):
            raise ProgramError(f"output quadrant {q} is algebraically wrong:\n{outputs[q]}")
    for q in outputs:
        if q not in expect:
            raise ProgramError(f"unexpected output quadrant {q}")
    return {"outputs": outputs, "ws": ws, "bubbles": bubbles // max(1, tiles)}
