import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "cute-kernels_b200"), os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    config.addinivalue_line("markers", "expects_dev_status: the test provokes and checks a device status flag itself")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel may have flagged a range / timeout / metadata problem."""
    yield
    if request.node.get_closest_marker("gpu") is not None and not request.node.get_closest_marker("expects_dev_status"):
        import torch

        if torch.cuda.is_available():
            import cute_kernels

            cute_kernels.check_device_status()
