"""Host logic of the multi-GPU slab plan, run as 2 gloo ranks on CPU (no GPU, no NCCL)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from subcuber_b200 import multi_gpu


def test_row_shard_covers_everything():
    for rows, world in ((8192, 8), (10, 4), (7, 2), (3, 4)):
        spans = [multi_gpu.row_shard(rows, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == rows
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        multi_gpu.row_shard(8, 2, 2)


def test_plan_picks_the_cheaper_direction():
    p = multi_gpu.plan(16384, 16384, 16384, 8, esize=2, level=2)
    assert p.kind in ("row", "col") and p.local_m * p.local_n == 16384 * 16384 // 8
    assert p.exchange_bytes == 7 * 16384 * 16384 * 2 // 8
    # K-heavy rectangular config: M=16384 N=8192 K=32768 -> B (1 GiB at f32) is smaller than A (2 GiB): row slabs
    p = multi_gpu.plan(16384, 8192, 32768, 8, esize=4, level=2)
    assert p.kind == "row" and (p.local_m, p.local_n) == (2048, 8192)
    assert p.exchange_bytes == 7 * 32768 * 8192 * 4 // 8
    # wide problem: A is the smaller operand -> column slabs
    p = multi_gpu.plan(2048, 65536, 4096, 8, esize=2, level=1)
    assert p.kind == "col" and (p.local_m, p.local_n) == (2048, 8192)
    # too small to slab: replicas
    assert multi_gpu.plan(512, 512, 512, 8, esize=2, level=1).kind == "replica"
    assert multi_gpu.plan(4096, 4096, 4096, 1, esize=2).exchange_bytes == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, k, n, m_per_rank, ragged, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        b_all = torch.randint(-3, 4, (k, n), generator=g).float()
        a_all = torch.randint(-3, 4, (m_per_rank * world, k), generator=g).float()
        b0, b1 = multi_gpu.row_shard(k, world, rank)
        a_slab = a_all[rank * m_per_rank:(rank + 1) * m_per_rank].contiguous()
        calls = []

        def local_gemm(a, b):
            calls.append((tuple(a.shape), tuple(b.shape)))
            return a @ b

        c_slab = multi_gpu.slab_gemm(a_slab, b_all[b0:b1].contiguous(), k, world, rank, local_gemm)
        want = (a_all @ b_all)[rank * m_per_rank:(rank + 1) * m_per_rank]
        ok = torch.equal(c_slab, want) and calls == [((m_per_rank, k), (k, n))]
        # the gathered B must be the whole matrix on every rank
        full = torch.empty((k, n))
        multi_gpu.all_gather_rows(full, b_all[b0:b1].contiguous(), world)
        ok = ok and torch.equal(full, b_all)
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("k,ragged", [(64, False), (67, True)])
def test_slab_gemm_two_gloo_ranks(k, ragged):
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, k, 24, 16, ragged, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(out.get(timeout=10) for _ in range(world))
    assert results == {0: True, 1: True}


def _pipeline_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        k, n = 8, 6
        g = torch.Generator().manual_seed(3)
        b_all = torch.randint(-3, 4, (k, n), generator=g).float()
        b0, b1 = multi_gpu.row_shard(k, world, rank)
        shard = b_all[b0:b1].contiguous()
        pipe = multi_gpu.PipelinedGather(shard, k, world)
        seen = []
        for step in range(5):
            buf = pipe.next()
            seen.append((buf.data_ptr(), bool(torch.equal(buf, b_all))))
            shard += 1          # the next gathers must pick up the new values ...
            b_all = b_all + 1   # ... which every rank changes the same way
            pipe.done(buf)
        out.put((rank, seen))
    finally:
        dist.destroy_process_group()


def test_pipelined_gather_alternates_buffers_on_two_ranks():
    """Two gloo ranks: every step sees a fully replicated B, in alternating buffers.  (On CPU the gathers run
    synchronously, two steps ahead, so a step sees the shard values of two steps earlier.)"""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pipeline_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank in (0, 1):
        ptrs = [ptr for ptr, _ in results[rank]]
        assert ptrs[0] != ptrs[1] and ptrs[0::2] == [ptrs[0]] * 3 and ptrs[1::2] == [ptrs[1]] * 2
    assert multi_gpu.PipelinedGather.reserved_sms() == 2 * multi_gpu.PipelinedGather.NCCL_CTAS


def test_grid_plan_moves_fewer_bytes_than_slabs():
    gp = multi_gpu.grid_plan(16384, 16384, 16384, 8, esize=2, level=1)
    assert (gp.kind, gp.pr, gp.pc, gp.local_m, gp.local_n) == ("grid", 4, 2, 4096, 8192)
    assert gp.a_recv_bytes + gp.b_recv_bytes == 256 << 20          # against 448 MiB for eight row slabs
    assert gp.row_group(5) == [4, 5] and gp.col_group(5) == [1, 3, 5, 7] and gp.coords(5) == (2, 1)
    gp = multi_gpu.grid_plan(16384, 16384, 16384, 4, esize=2, level=1)
    assert (gp.pr, gp.pc) == (2, 2) and gp.a_recv_bytes == gp.b_recv_bytes == 128 << 20
    gp = multi_gpu.grid_plan(16384, 16384, 16384, 2, esize=2, level=1)
    assert (gp.pr, gp.pc, gp.a_recv_bytes) == (2, 1, 0)
    assert multi_gpu.grid_plan(16384, 16384, 16384, 1, esize=2).a_recv_bytes == 0
    assert multi_gpu.grid_plan(1000, 1000, 1000, 8, esize=2).kind == "replica"


def _grid_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 2048, 2048, 512
        gp = multi_gpu.grid_plan(m, n, k, world, esize=4, level=1)
        ex = multi_gpu.CollectiveGridExchange(gp, rank, "f32", "cpu", seed=3)
        a, b = ex.next()
        ex.done()
        want_a, want_b = multi_gpu.expected_slabs(gp, rank, "f32", "cpu", seed=3)
        ok = torch.equal(a, want_a) and torch.equal(b, want_b)
        ok = ok and tuple(a.shape) == (gp.local_m, k) and tuple(b.shape) == (k, gp.local_n)
        # the blocks of all ranks assemble to the product of the assembled operands
        i, j = gp.coords(rank)
        block = a.double() @ b.double()
        blocks = [torch.empty_like(block) for _ in range(world)]
        dist.all_gather(blocks, block)
        slabs_a = [torch.empty_like(a) for _ in range(world)]
        slabs_b = [torch.empty_like(b) for _ in range(world)]
        dist.all_gather(slabs_a, a)
        dist.all_gather(slabs_b, b)
        full_a = torch.cat([slabs_a[ii * gp.pc] for ii in range(gp.pr)])
        full_b = torch.cat([slabs_b[jj] for jj in range(gp.pc)], dim=1)
        full_c = torch.cat([torch.cat([blocks[ii * gp.pc + jj] for jj in range(gp.pc)], dim=1) for ii in range(gp.pr)])
        ok = ok and torch.allclose(full_c, full_a.double() @ full_b.double(), rtol=0, atol=1e-9)
        # ranks of one grid row hold the same A slab, ranks of one grid column the same B slab
        ok = ok and all(torch.equal(slabs_a[r], a) for r in gp.row_group(rank))
        ok = ok and all(torch.equal(slabs_b[r], b) for r in gp.col_group(rank))
        out.put((rank, bool(ok), (gp.pr, gp.pc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_grid_exchange_on_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_grid_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results)
    assert {g for _, _, g in results} == {(2, 1) if world == 2 else (2, 2)}
