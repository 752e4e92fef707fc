"""How output tiles are dealt to the workers of the persistent kernels (host arithmetic, no GPU needed): whole tiles
round-robin, two K-halves per tile when tiles are few, and an equal-share stream over the last waves otherwise."""
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


def _check(units, workers, lay, num_k):
    tiles = lay.tiles_m * lay.tiles_n
    cover = {}
    slots = set()
    cut = {}
    last_of_worker = {}
    for w, tile, part, parts, k0, k1, slot, split in units:
        assert 0 <= w < workers and 0 <= tile < tiles and 0 <= k0 < k1 <= num_k and parts in (1, 2)
        cover.setdefault(tile, []).append((k0, k1))
        assert slot not in slots, "two units share a hand-off slot"
        slots.add(slot)
        if parts == 1:
            assert (k0, k1) == (0, num_k) and part == 0 and slot == tile
        else:
            assert part in (0, 1)
            cut.setdefault(split, {})[part] = (tile, slot, w)
            assert slot == (tile if part == 0 else tiles + split)
        last_of_worker[w] = (tile, part, parts)
    for tile in range(tiles):
        spans = sorted(cover[tile])
        assert spans[0][0] == 0 and spans[-1][1] == num_k and len(spans) <= 2
        if len(spans) == 2:
            assert spans[0][1] == spans[1][0]
    for split, parts in cut.items():
        assert set(parts) == {0, 1} and parts[0][0] == parts[1][0], "a cut tile needs one publisher and one finisher"
        assert parts[0][2] != parts[1][2], "both parts of a tile on one worker"
    return cut


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (16384, 16384, 16384), (2048, 16384, 16384), (4096, 8192, 16384),
                                   (2048, 2048, 2048), (512, 2560, 1024), (1001, 2568, 1160), (5120, 15360, 2048)])
@pytest.mark.parametrize("sms", [148, 146, 16, 8])
def test_every_k_step_of_every_tile_is_dealt_once(kernel, shape, sms, lib):
    from subcuber_b200 import _lib as L

    m, n, k = shape
    lay = L.WorkspaceLayout()
    assert lib.sb200_gemm_workspace_layout(kernel.encode(), m, n, k, C.byref(lay)) == 0
    es = 2 if "_f16_" in kernel else 4
    num_k = -(-lay.kq // (128 // es))
    units, workers = _deal(lib, kernel, m, n, k, sms)
    assert 1 <= workers <= (sms // 2 if "2sm" in kernel else sms)
    _check(units, workers, lay, num_k)
    whole, _ = _deal(lib, kernel, m, n, k, sms, no_split=1)
    assert (whole[:, 3] == 1).all()


def test_stream_gives_equal_shares(lib):
    """2048 x 16384 x 16384 at level 1 on 73 pairs: 128 pair tiles, i.e. 1.75 tiles per pair instead of two waves."""
    from subcuber_b200 import _lib as L

    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    m, n, k = 2048, 16384, 16384
    units, workers = _deal(lib, kernel, m, n, k, 146)
    assert workers == 73
    lay = L.WorkspaceLayout()
    lib.sb200_gemm_workspace_layout(kernel.encode(), m, n, k, C.byref(lay))
    num_k = lay.kq // 64
    load = np.zeros(workers, dtype=np.int64)
    for w, _, _, _, k0, k1, _, _ in units:
        load[w] += k1 - k0
    assert load.sum() == 128 * num_k
    assert load.max() <= 1.87 * num_k and load.min() >= 1.63 * num_k   # 1.75 +- the snap distance on either side
    # a worker runs the part that publishes first and the part that waits for a partial sum last
    for w in range(workers):
        mine = units[units[:, 0] == w]
        cut_parts = [(i, u[2]) for i, u in enumerate(mine) if u[3] == 2]
        for i, part in cut_parts:
            assert (part == 0 and i == 0) or (part == 1 and i == len(mine) - 1)
