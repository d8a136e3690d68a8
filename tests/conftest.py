import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")
    config.addinivalue_line("markers", "expects_timeout: the test makes a bounded device wait run out on purpose")


@pytest.fixture(autouse=True)
def _check_device_status(request):
    """After every GPU test: no kernel may have left a timeout status behind."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    if request.node.get_closest_marker("expects_timeout") is not None:
        return
    import torch

    if torch.cuda.is_available():
        import kraken_b200

        kraken_b200.check_status()
