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
