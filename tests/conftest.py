"""Shared test set-up.  GPU tests carry ``@pytest.mark.gpu``; everything else runs on a CPU-only box."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def lib():
    """The product's shared library; built on first use when missing (nvcc cross-compiles without a GPU)."""
    from candle_b200 import build, capi
    if not os.path.exists(capi.LIB_PATH):
        build.build()
    return capi.lib()


@pytest.fixture(scope="session")
def cuda_dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
