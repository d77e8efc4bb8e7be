import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def nb():
    """The product package (its name starts with a digit, hence importlib)."""
    import importlib
    return importlib.import_module("3dmaker_b200")


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def cuda(nb):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    nb.load()  # raises if the library is not built: no fallback
    torch.cuda.set_device(0)
    return torch
