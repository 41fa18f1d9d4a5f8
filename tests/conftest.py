import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def be():
    """The product package (directory name has hyphens; see b200_eagle.py)."""
    import b200_eagle
    return b200_eagle


@pytest.fixture(scope="session")
def cuda(be):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    be._lib.lib()          # raises if the extension is missing: GPU tests never fall back
    return torch.device("cuda:0")
