import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    import tacker_oracle

    tacker_oracle.lib()
    return tacker_oracle


@pytest.fixture(scope="session")
def cuda():
    """torch with a CUDA device and the product library loaded; fails loudly when either is missing."""
    import torch

    assert torch.cuda.is_available(), "gpu-marked test started without a CUDA device"
    import tacker_b200

    tacker_b200.lib()  # raises if libtacker_b200.so was not built: no fallback
    torch.cuda.set_device(0)
    return torch
