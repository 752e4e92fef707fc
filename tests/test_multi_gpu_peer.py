"""multi_gpu.PeerGather on real GPUs (needs two; skipped on a one-GPU machine): the replicated B every rank multiplies
with equals the whole matrix and the slab GEMMs equal the single-GPU ones."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_peer_gather_on_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29571", os.path.join(here, "peer_gather_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "PEER_GATHER_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_grid_exchange_on_two_gpus():
    """multi_gpu.GridExchange on two real GPUs: the slabs every rank multiplies are the shards their owners generated,
    in place, at every step, and the block GEMMs equal the same GEMMs on private copies bit for bit."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29573", os.path.join(here, "grid_exchange_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "GRID_EXCHANGE_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


def test_two_devices_in_one_process(oracle):
    """Kernel attributes and the SM count are kept per device: one process runs a GEMM on cuda:0 and then on cuda:1
    (every launch needs more than the default dynamic shared memory, an attribute of each device's copy of a kernel)."""
    import numpy as np
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from subcuber_b200 import inputs, runner

    m, n, k = 512, 768, 384
    for kernel, dt, level in [("blackwell_f16_sw_interleaved_presum_2sm", "f16", 1),
                              ("blackwell_f16_cubic_128x256", "f16", 0), ("blackwell_f64_sw_level1", "f64", 1)]:
        a_np, b_np = inputs.operands(dt, "harness", m, n, k, seed=3)
        want = oracle.sw_gemm(dt, level, a_np, b_np)
        for dev in ("cuda:0", "cuda:1"):
            device = torch.device(dev)
            with torch.cuda.device(device):
                d = runner.gemm(kernel, torch.from_numpy(a_np).to(device), torch.from_numpy(b_np).to(device))
                torch.cuda.synchronize(device)
            assert np.array_equal(d.cpu().numpy(), want), f"{kernel} on {dev}"
