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
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def pkg():
    import importlib
    return importlib.import_module("7_b200")


@pytest.fixture(scope="session")
def wc(pkg):
    return pkg.wave_cuda


@pytest.fixture(scope="session")
def cuda(wc):
    """torch is used for device memory and streams only."""
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    wc.lib()
    return torch
