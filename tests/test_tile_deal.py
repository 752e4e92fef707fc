"""The unit list of the persistent kernels (host arithmetic, no GPU needed): whole tiles in raster order, and two
K-halves per tile where the last wave would be at most half full or where tiles are few."""
import ctypes as C

import numpy as np
import pytest

KERNELS = ["blackwell_f16_sw_interleaved_presum_2sm", "blackwell_f16_cubic_2sm_256x256",
           "blackwell_f16_sw_interleaved_presum", "blackwell_f32_sw_level2_2sm"]


def _deal(lib, kernel, m, n, k, sms, **opt):
    from subcuber_b200 import _lib as L

    o = L.GemmOptions(opt.get("sm_limit", 0), opt.get("no_split", 0), 0, 0)
    units = (C.c_int * (8 * 20000))()
    workers = C.c_int(0)
    cnt = lib.sb200_gemm_deal(kernel.encode(), m, n, k, C.byref(o), sms, units, 20000, C.byref(workers))
    assert 0 <= cnt <= 20000
    return np.frombuffer(units, dtype=np.int32)[: cnt * 8].reshape(cnt, 8).copy(), workers.value


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
    cover, slots, halves = {}, set(), {}
    for _, tile, part, parts, k0, k1, slot, split in units:
        assert 0 <= tile < tiles and 0 <= k0 < k1 <= num_k and parts in (1, 2)
        cover.setdefault(tile, []).append((k0, k1))
        assert slot not in slots, "two units share a hand-off slot"
        slots.add(slot)
        if parts == 1:
            assert (k0, k1) == (0, num_k) and part == 0 and slot == tile
        else:
            halves.setdefault(split, {})[part] = tile
            assert slot == (tile if part == 0 else tiles + split)
    for tile in range(tiles):
        spans = sorted(cover[tile])
        assert spans[0][0] == 0 and spans[-1][1] == num_k and len(spans) <= 2
        if len(spans) == 2:
            assert spans[0][1] == spans[1][0]
    for split, parts in halves.items():
        assert set(parts) == {0, 1} and parts[0] == parts[1]
    # the half that publishes comes before the half that waits for it
    cut = units[units[:, 3] == 2]
    assert (cut[0::2, 2] == 0).all() and (cut[1::2, 2] == 1).all() and (cut[0::2, 1] == cut[1::2, 1]).all()
    whole, _ = _deal(lib, kernel, m, n, k, sms, no_split=1)
    assert (whole[:, 3] == 1).all() and len(whole) == tiles


def test_which_tiles_are_cut(lib):
    """CTA pairs with more tiles than pairs draw whole tiles as they become free: nothing is cut.  The 1-CTA kernels
    deal round-robin and cut a last wave that is at most half full."""
    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    for size, tiles in ((8192, 256), (16384, 1024)):
        units, workers = _deal(lib, kernel, size, size, size, 148)
        assert workers == 74 and len(units) == tiles and (units[:, 3] == 1).all()
    # 1-CTA kernels, 8192^3: 512 tiles on 148 CTAs = 3 waves + 68: less than half a wave, cut
    units, workers = _deal(lib, "blackwell_f16_sw_interleaved_presum", 8192, 8192, 8192, 148)
    assert workers == 148 and len(units) == 444 + 136
    # 16384^3: 2048 tiles = 13 waves + 124: more than half a wave, nothing is cut
    units, workers = _deal(lib, "blackwell_f16_sw_interleaved_presum", 16384, 16384, 16384, 148)
    assert len(units) == 2048 and (units[:, 3] == 1).all()


def test_few_tiles_are_not_cut(lib):
    """f32 level 1 at 2048^3: 16 pair tiles on 74 pairs stay whole (cutting them was measured to cost more than it
    gains)."""
    units, workers = _deal(lib, "blackwell_f32_sw_interleaved_presum_2sm", 2048, 2048, 2048, 148)
    assert workers == 16 and len(units) == 16 and (units[:, 3] == 1).all()
