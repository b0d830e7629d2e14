import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lily():
    """The package with its CUDA library built (nvcc cross-compiles without a GPU)."""
    import lily_b200
    import lily_b200.build as build

    build.build()
    return lily_b200


@pytest.fixture(scope="session")
def cuda(lily):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch
