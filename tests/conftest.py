import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "blockscaled_golden.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def cuda_lib():
    """The native library on a CUDA machine; fails loudly if it cannot be loaded."""
    import torch
    assert torch.cuda.is_available(), "a CUDA device is required for -m gpu tests"
    from cutlass_b200 import lib
    return lib.load()
