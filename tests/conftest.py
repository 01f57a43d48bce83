import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def tn_gpu():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import tensornet_b200 as tn

    tn.core.init()
    assert tn.core.runtime().on_gpu
    return tn


@pytest.fixture()
def status_ok(tn_gpu):
    yield
    import torch

    torch.cuda.synchronize()
    try:
        tn_gpu.core.runtime().check_status()
    except tn_gpu.core.DeviceError:
        tn_gpu.core.recover()      # a reported error is sticky: clear it so the next test starts clean
        raise
