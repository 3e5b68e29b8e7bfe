import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session", autouse=True)
def _native_libraries():
    """Build the in-tree native libraries once per session if they are stale or missing."""
    from kernel_align_b200 import _build

    _build.build_all()
    yield


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from kernel_align_b200 import _native

    _native.cuda()  # raises if the kernel library is missing: no silent fallback on a GPU host
    return torch.device("cuda", 0)
