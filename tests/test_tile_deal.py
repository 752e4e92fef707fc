"""The unit list of the persistent kernels (host arithmetic, no GPU needed): whole tiles in raster order, then two units
per tile of a last wave that is at most half full - column halves for the CTA-pair kernels, K-halves for the others."""
import ctypes as C

import numpy as np
import pytest

KERNELS = ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_cubic_2sm_256x256",
           "blackwell_f16_sw_interleaved_presum", "blackwell_f32_sw_level2_2sm"]


def _deal(lib, kernel, m, n, k, sms, **opt):
    from subcuber_b200 import _lib as L

    o = L.GemmOptions(opt.get("sm_limit", 0), opt.get("no_split", 0), 0, 0)
    units = (C.c_int * (10 * 20000))()
    workers = C.c_int(0)
    cnt = lib.sb200_gemm_deal(kernel.encode(), m, n, k, C.byref(o), sms, units, 20000, C.byref(workers))
    assert 0 <= cnt <= 20000
    return np.frombuffer(units, dtype=np.int32)[: cnt * 10].reshape(cnt, 10).copy(), workers.value


def _layout(lib, kernel, m, n, k):
    from subcuber_b200 import _lib as L

    lay = L.WorkspaceLayout()
    assert lib.sb200_gemm_workspace_layout(kernel.encode(), m, n, k, C.byref(lay)) == 0
    es = 2 if ("_f16_" in kernel or "_bf16_" in kernel) else 4
    return lay, -(-lay.kq // (128 // es))


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (16384, 16384, 16384), (2048, 16384, 16384), (4096, 8192, 16384),
                                   (2048, 2048, 2048), (512, 2560, 1024), (1001, 2568, 1160), (5120, 15360, 2048)])
@pytest.mark.parametrize("sms", [148, 146, 16, 8])
def test_every_k_step_of_every_tile_is_handed_out_once(kernel, shape, sms, lib):
    m, n, k = shape
    lay, num_k = _layout(lib, kernel, m, n, k)
    tiles = lay.tiles_m * lay.tiles_n
    units, workers = _deal(lib, kernel, m, n, k, sms)
    assert 1 <= workers <= (sms // 2 if "2sm" in kernel else sms)
    cover, slots, halves, columns = {}, set(), {}, {}
    for _, tile, part, parts, k0, k1, slot, split, col, cols in units:
        assert 0 <= tile < tiles and 0 <= k0 < k1 <= num_k and parts in (1, 2) and cols in (1, 2) and 0 <= col < cols
        assert not (parts == 2 and cols == 2), "a unit is cut along K or along the columns, not both"
        if cols == 2:
            # column halves: independent units, all of K each, the tile's own hand-off slot (each uses half of it)
            assert "2sm" in kernel and (k0, k1) == (0, num_k) and part == 0 and slot == tile
            columns.setdefault(tile, []).append(col)
            continue
        cover.setdefault(tile, []).append((k0, k1))
        assert slot not in slots, "two units share a hand-off slot"
        slots.add(slot)
        if parts == 1:
            assert (k0, k1) == (0, num_k) and part == 0 and slot == tile
        else:
            assert "2sm" not in kernel
            halves.setdefault(split, {})[part] = tile
            assert slot == (tile if part == 0 else tiles + split)
    assert not (set(cover) & set(columns))
    for tile in range(tiles):
        if tile in columns:
            assert sorted(columns[tile]) == [0, 1]
            continue
        spans = sorted(cover[tile])
        assert spans[0][0] == 0 and spans[-1][1] == num_k and len(spans) <= 2
        if len(spans) == 2:
            assert spans[0][1] == spans[1][0]
    for split, parts in halves.items():
        assert set(parts) == {0, 1} and parts[0] == parts[1]
    # the half that publishes comes before the half that waits for it
    cut = units[units[:, 3] == 2]
    assert (cut[0::2, 2] == 0).all() and (cut[1::2, 2] == 1).all() and (cut[0::2, 1] == cut[1::2, 1]).all()
    # column halves of a tile are neighbours in the list, and they come after every whole tile
    halved = units[units[:, 9] == 2]
    assert (halved[0::2, 8] == 0).all() and (halved[1::2, 8] == 1).all() and (halved[0::2, 1] == halved[1::2, 1]).all()
    if len(halved):
        assert (units[: len(units) - len(halved), 9] == 1).all()
    whole, _ = _deal(lib, kernel, m, n, k, sms, no_split=1)
    assert (whole[:, 3] == 1).all() and (whole[:, 9] == 1).all() and len(whole) == tiles


def test_which_tiles_are_cut(lib):
    """CTA pairs draw their units as they become free and cut a last wave that is at most half full into column
    halves.  The 1-CTA kernels deal round-robin and cut such a wave into K-halves."""
    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    # 8192^3: 256 tiles on 74 pairs = 3 waves + 34 tiles, cut: 222 whole tiles + 68 column halves
    units, workers = _deal(lib, kernel, 8192, 8192, 8192, 148)
    assert workers == 74 and len(units) == 222 + 68 and (units[:, 3] == 1).all()
    assert (units[:222, 9] == 1).all() and (units[222:, 9] == 2).all()
    # 16384^3: 1024 tiles = 13 waves + 62 tiles: more than half a wave, nothing is cut
    units, workers = _deal(lib, kernel, 16384, 16384, 16384, 148)
    assert workers == 74 and len(units) == 1024 and (units[:, 9] == 1).all()
    # two SMs left to the caller: 256 tiles on 73 pairs = 3 waves + 37 tiles, one too many to gain anything
    units, workers = _deal(lib, kernel, 8192, 8192, 8192, 148, sm_limit=146)
    assert workers == 73 and len(units) == 256 and (units[:, 9] == 1).all()
    # 1-CTA kernels, 8192^3: 512 tiles on 148 CTAs = 3 waves + 68: less than half a wave, cut along K
    units, workers = _deal(lib, "blackwell_f16_sw_interleaved_presum", 8192, 8192, 8192, 148)
    assert workers == 148 and len(units) == 444 + 136 and (units[:, 9] == 1).all()
    # 16384^3: 2048 tiles = 13 waves + 124: more than half a wave, nothing is cut
    units, workers = _deal(lib, "blackwell_f16_sw_interleaved_presum", 16384, 16384, 16384, 148)
    assert len(units) == 2048 and (units[:, 3] == 1).all()


def test_few_tiles_become_column_halves(lib):
    """f32 level 1 at 2048^3: 16 pair tiles on 74 pairs run as 32 column halves on 32 pairs; the one-launch and the
    fused-presum kernels are never cut."""
    units, workers = _deal(lib, "blackwell_f32_sw_interleaved_presum_2sm", 2048, 2048, 2048, 148)
    assert workers == 32 and len(units) == 32 and (units[:, 9] == 2).all() and (units[:, 3] == 1).all()
    for kernel in ("blackwell_f32_sw_merged_presum_2sm", "blackwell_f32_sw_fused_presum_2sm"):
        units, workers = _deal(lib, kernel, 2048, 2048, 2048, 148)
        assert workers == 16 and len(units) == 16 and (units[:, 9] == 1).all()
