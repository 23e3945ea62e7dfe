import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: test needs more than one CUDA device")


def pytest_collection_modifyitems(config, items):
    import torch
    has_gpu = torch.cuda.is_available()
    skip_gpu = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords and not has_gpu:
            item.add_marker(skip_gpu)


@pytest.fixture(autouse=True)
def _kernel_status_clean(request):
    """After every GPU test, fail if a kernel reported an expired wait or a rejected index."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from ml_framework_b200 import _lib
            assert _lib.read_status(True) == 0, "a kernel left a non-zero status word"
