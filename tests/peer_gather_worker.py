"""Worker of tests/test_multi_gpu_peer.py: one rank of a torchrun launch, checks multi_gpu.PeerGather on real GPUs."""
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

    os.environ.setdefault("NCCL_MAX_CTAS", str(multi_gpu.PeerGather.NCCL_CTAS))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist.init_process_group("nccl", device_id=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    opts = runner.options(sm_limit=sms - multi_gpu.PeerGather.reserved_sms())  # SMs left free for the exchange
    kernel = "blackwell_f16_sw_interleaved_presum_2sm"
    m, n, k = 512, 1024, 1024 * world
    gen = torch.Generator(device="cpu").manual_seed(5)
    b_steps = [(torch.rand((k, n), generator=gen) * 2 - 1).to(torch.float16) for _ in range(5)]
    a = (torch.rand((m, k), generator=torch.Generator().manual_seed(9 + rank)) * 2 - 1).to(torch.float16).to(dev)
    lo, hi = multi_gpu.row_shard(k, world, rank)
    shard = b_steps[0][lo:hi].to(dev).contiguous()
    gather = multi_gpu.PeerGather(shard, k, world, rank)
    ws = runner.Workspace(kernel, m, n, k, dev, opts)
    ok = True
    for step in range(5):
        # the first call of next() starts the exchanges of steps 0 and 1, every later call the one of the step after:
        # with new shard contents handed over before each call, step s multiplies with version max(0, s - 1)
        if step > 0:
            gather.update_shard(b_steps[step][lo:hi].to(dev))
        b = gather.next()
        d = runner.gemm(kernel, a, b, workspace=ws, check=False, opts=opts)
        gather.done(b)
        want_b = b_steps[max(0, step - 1)]
        torch.cuda.synchronize(dev)
        ok = ok and torch.equal(b.cpu(), want_b)
        ref = runner.gemm(kernel, a, want_b.to(dev))
        ok = ok and torch.equal(d, ref)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PEER_GATHER_OK" if int(flag.item()) == 1 else "PEER_GATHER_MISMATCH", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
