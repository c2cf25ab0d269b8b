import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu and needs a CUDA device")
    from dlcompiler_b200 import _lib

    _lib.load()  # fail loudly if the extension is missing
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_guard(request):
    """After every GPU test, fail if a kernel recorded a timed-out wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        from dlcompiler_b200 import check_device_status

        check_device_status()
