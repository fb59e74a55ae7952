import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.join(ROOT, "flash-attention-rdna3_b200")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


@pytest.fixture(autouse=True)
def _check_kernel_status(request):
    """After every GPU test, fail if a kernel reported that one of its bounded waits ran out."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import fa_b200

        fa_b200.check_status()
