import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with `-m gpu`")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fused_cpp_b200 import _lib

    if not _lib.device_supported():
        pytest.fail("the CUDA device is not a compute-capability-10.x GPU; the library has no other path")
    return torch.device("cuda", torch.cuda.current_device())
