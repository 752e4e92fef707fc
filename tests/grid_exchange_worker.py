"""Worker of tests/test_multi_gpu_peer.py: one rank of a torchrun launch, checks multi_gpu.GridExchange on real GPUs."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from subcuber_b200 import multi_gpu, runner

    os.environ.setdefault("NCCL_MAX_CTAS", "2")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist.init_process_group("nccl", device_id=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    opts = runner.options(sm_limit=sms - multi_gpu.GridExchange.reserved_sms())   # SMs left free for the flag kernels
    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    m = n = k = 2048
    gp = multi_gpu.grid_plan(m, n, k, world, 2, level=1)
    ex = multi_gpu.GridExchange(gp, rank, "f16", dev, seed=5)
    ws = runner.Workspace(kernel, gp.local_m, gp.local_n, k, dev, opts)
    d = torch.empty((gp.local_m, gp.local_n), dtype=torch.float16, device=dev)
    ok = True
    for step in range(5):
        a, b = ex.next()
        runner.gemm(kernel, a, b, d, workspace=ws, check=False, opts=opts)
        ex.done()
        torch.cuda.synchronize(dev)
        ok = ok and ex.verify_block(d, (a, b))
        # against the same kernel on private copies of the slabs this rank should hold
        want_a, want_b = multi_gpu.expected_slabs(gp, rank, "f16", dev, seed=5)
        ok = ok and torch.equal(d, runner.gemm(kernel, want_a, want_b, opts=opts))
    # feeding mode: every rank uploads the shards it owns from pinned host memory, new values every step (the A shards
    # scaled by a power of two, so the expected block is the same GEMM on scaled slabs, bit for bit); the two steps
    # whose pushes were already in flight still run on the old shards
    first_fed = ex.issued
    scale = lambda s: (1.0, 2.0, 0.5)[s % 3] if s >= first_fed else 1.0
    a_own, b_own = ex.shard_views(0)
    a_host = [(a_own * c).cpu().pin_memory() for c in (1.0, 2.0, 0.5)]
    b_host = b_own.cpu().pin_memory()
    ex.start_feeding()
    for step in range(5, 12):
        ex.feed(a_host[(step + ex.NBUF - 1) % 3], b_host)     # shards of the step whose pushes this `next` starts
        a, b = ex.next()
        runner.gemm(kernel, a, b, d, workspace=ws, check=False, opts=opts)
        ex.done()
        torch.cuda.synchronize(dev)
        ok = ok and torch.equal(d, runner.gemm(kernel, want_a * scale(step), want_b, opts=opts))
    ex.check_status()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("GRID_EXCHANGE_OK" if int(flag.item()) == 1 else "GRID_EXCHANGE_MISMATCH", flush=True)
    ex.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
