import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def wq():
    """The product module with its CUDA library loaded.  On a GPU box a missing library is a failure, never a skip:
    there is no other implementation to fall back to."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from wgpkernels_b200 import int8
    int8.load_library()
    torch.cuda.set_device(0)
    return int8
