import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def ak():
    """The package (ctypes binding of the CUDA library)."""
    return entry.load_package()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (the checker)."""
    o = entry.load_oracle()
    o.lib()
    return o


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_test_math.npz"))


@pytest.fixture(scope="session")
def ctx(ak):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    c = ak.Context(0)
    yield c
    c.check_device_status()


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


def lcg(orc, n, seed):
    return orc.lcg(n, seed)
