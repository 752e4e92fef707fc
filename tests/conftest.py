import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle binding (test infrastructure; builds liboracle.so on first use)."""
    from oracle import binding

    binding.build(ref=True)
    return binding


@pytest.fixture(scope="session")
def lib():
    """The product library (built on first use; fails loudly when nvcc is missing)."""
    from subcuber_b200 import _lib

    return _lib.load()


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for tests marked gpu")
    return torch.device("cuda:0")
