import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    import torch

    path = os.path.join(ROOT, "tests", "golden", "golden.pt")
    return torch.load(path, weights_only=False)


@pytest.fixture(scope="session")
def sgpt_golden():
    import torch

    path = os.path.join(ROOT, "tests", "golden", "sgpt_hessian.pt")
    return torch.load(path, weights_only=False)


@pytest.fixture(scope="session")
def awq_golden():
    import torch

    path = os.path.join(ROOT, "tests", "golden", "awq.pt")
    return torch.load(path, weights_only=False)
