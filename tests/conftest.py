import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def rel_err(x, ref):
    """max|x - ref| / max|ref| per tensor, the metric the tolerances are stated in."""
    ref = ref.double()
    denom = ref.abs().max().item()
    diff = (x.detach().double().cpu() - ref.cpu()).abs().max().item()
    return diff / denom if denom > 0 else diff


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
