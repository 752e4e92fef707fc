"""Tile-program tables compiled into the library: protocol and algebra, checked symbolically on the CPU."""
import ctypes as C

import pytest

from subcuber_b200 import tile_program as tp


def test_struct_mirror_matches_header(lib):
    assert lib.sb200_tile_program_bytes() == C.sizeof(tp.Program)


def test_level0(lib):
    pg = tp.from_library("level0")
    assert pg.nproducts == 1 and pg.alternate_slots == 1 and pg.needs_feed == 0
    tp.check_program(pg, level=0, nslots=2, tiles=5)
    tp.check_program(pg, level=0, nslots=4, tiles=5)


@pytest.mark.parametrize("which,feed", [("level1_full_fly", 1), ("level1_full_ws", 0)])
def test_level1_single_launch(lib, which, feed):
    pg = tp.from_library(which)
    assert pg.nproducts == 7 and pg.needs_feed == feed
    res = tp.check_program(pg, level=1, nslots=2, tiles=4)
    assert sorted(res["outputs"]) == [0, 1, 2, 3]


def test_level1_two_launches(lib):
    first = tp.from_library("level1_first")
    second = tp.from_library("level1_second")
    assert first.nproducts == 2 and second.nproducts == 5
    assert first.needs_feed == 0 and second.needs_feed == 0
    r1 = tp.check_program(first, level=1, nslots=2, expect=[0], tiles=4)
    assert 0 in r1["ws"]  # M0 handed to the second launch
    r2 = tp.check_program(second, level=1, nslots=2, ws_in=r1["ws"], expect=[1, 2, 3], tiles=4)
    assert sorted(r2["outputs"]) == [1, 2, 3]


def test_level1_second_launch_with_short_taps(lib):
    first = tp.from_library("level1_first")
    taps = tp.from_library("level1_second_taps")
    r1 = tp.check_program(first, level=1, nslots=2, expect=[0], tiles=3)
    r2 = tp.check_program(taps, level=1, nslots=2, ws_in=r1["ws"], expect=[1, 2, 3], tiles=5)
    assert sorted(r2["outputs"]) == [1, 2, 3] and sorted(r2["ws"]) == [0, 1, 2]  # U and V share buffer 2
    # every step a product waits on is a pure slot-to-hand-off copy or a final sum of one slot: none reads two slots
    assert all(taps.epilogue[i].nslots <= 1 for i in range(taps.nepilogues))


def test_second_launch_needs_the_handoff(lib):
    with pytest.raises(tp.ProgramError):
        tp.check_program(tp.from_library("level1_second"), level=1, nslots=2, expect=[1, 2, 3])


def test_checker_rejects_broken_tables(lib):
    pg = tp.from_library("level1_full_ws")
    pg.product[3].negate = 1  # flips the sign of one product
    with pytest.raises(tp.ProgramError):
        tp.check_program(pg, level=1)
    pg = tp.from_library("level1_full_ws")
    pg.product[4].wait_free = 0  # writes a slot the epilogue still owns
    with pytest.raises(tp.ProgramError):
        tp.check_program(pg, level=1)
    pg = tp.from_library("level1_full_ws")
    pg.epilogue[1].release_mask = 0  # never gives the slot back
    with pytest.raises(tp.ProgramError):
        tp.check_program(pg, level=1)


def test_the_library_runs_the_generated_tables(lib):
    """The C++ side holds no schedule of its own: every table the library reports is the front end's, byte for byte,
    and csrc/sw_programs.h only looks tables up."""
    import os

    from subcuber_b200 import emit

    programs = emit.all_programs()
    assert len(programs) >= 8 + 14
    for name, pg in programs.items():
        assert bytes(tp.to_bytes(tp.from_library(name))) == bytes(tp.to_bytes(pg)), name
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(here, "subcuber_b200", "csrc", "sw_programs.h")).read()
    assert "sw_tile_programs.inc" in text and "add_product" not in text and "add_epilogue" not in text
    # m0 comes from DRAM: the second launch reads it exactly once
    second = programs["level1_second_taps"]
    reads_m0 = sum(1 for i in range(second.nepilogues) for t in range(second.epilogue[i].nsrc)
                   if second.epilogue[i].src[t] == 0)
    assert reads_m0 == 1


def test_strassen_presum_plan_tables(lib):
    """Strassen's original algorithm on materialised presums: the generated presum table lists each two-term operand
    sum of the DSL products once, every product operand of the program is a single view, and with the views holding
    what the table says the program yields the four blocks of the product."""
    import numpy as np

    from subcuber_b200 import emit
    from subcuber_b200.algos.strassen_level1 import strassen
    from subcuber_b200.algos.strassen_winograd_level1 import strassen_winograd

    c, ms = strassen(4, 4, 4)
    table = emit.strassen_presum_table(ms)
    assert [len(table[s]) for s in ("a", "b")] == [5, 5]
    views = [row[0] for s in ("a", "b") for row in table[s]]
    assert len(set(views)) == 10 and all(v < 8 for v in views[:5]) and all(v >= 8 for v in views[5:])
    # a1 and b1 are read by no product of this algorithm on their own: their view slots carry the fifth presums
    assert 1 in views and 9 in views
    for side in ("a", "b"):
        for view, q0, c0, q1, c1 in table[side]:
            assert q0 != q1 and c0 in (1, -1) and c1 in (1, -1)
    pg = tp.from_library("level1_strassen_presum")
    assert pg.needs_feed == 0 and pg.nproducts == 7
    for i in range(pg.nproducts):
        assert pg.product[i].a.nterms == 1 and pg.product[i].b.nterms == 1
    got = tp.check_program(pg, level=1, view_coef=emit.strassen_view_coef(ms))["outputs"]
    want = {q: emit.bilinear_form(part) for q, part in enumerate(strassen_winograd(4, 4, 4)[0].parts)}
    for q in range(4):
        assert np.array_equal(got[q], want[q])
    # without the plan's view assignment the same table is not the product (views 1 and 9 would be raw quadrants)
    with pytest.raises(tp.ProgramError):
        tp.check_program(pg, level=1)
    # the table the library was built with is the generated one
    text = emit.generate_tables()
    for side in ("a", "b"):
        assert "{" + ", ".join("{%d, %d, %d, %d, %d}" % row for row in table[side]) + "}" in text
