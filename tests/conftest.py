import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 shared by the GPU tests."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from aeon_b200.kernels import Context
    c = Context(0)
    yield c
    c.close()
