import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(autouse=True)
def _check_kernel_status(request):
    """After every GPU test, fail if a kernel recorded a timed-out wait."""
    yield
    if request.node.get_closest_marker("gpu"):
        from lingua_b200.ops import _lib

        _lib.check_status()
