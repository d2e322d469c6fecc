import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (REPO, os.path.join(REPO, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as _o  # oracle/oracle.py — the CPU checker
    _o.lib()
    return _o


@pytest.fixture(scope="session")
def zq():
    """The product API; needs libzq.so and a GPU."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import zignn_b200
    return zignn_b200.api
