import os
import sys

import pytest

# The CPU tests run tiny models in up to four gloo ranks at a time: a full thread pool per rank only
# oversubscribes the cores.  Spawned ranks and driver subprocesses inherit these.
os.environ.setdefault("OMP_NUM_THREADS", "2")
os.environ.setdefault("MKL_NUM_THREADS", "2")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(autouse=True)
def _check_device_status(request):
    """After every GPU test, fail if a kernel's bounded wait gave up."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from mist_b200.ops import native
            torch.cuda.synchronize()
            native.check_status()
