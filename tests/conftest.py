import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def requested_chunk_sizes():
    """The tests ask for particular chunk geometries (chunks shorter than a tile, not a multiple of it, many short
    chunks ...): the package runs them as asked.  tests/test_gpu_auto_chunk.py switches the automatic choice on."""
    from retention_integration_b200 import retention

    old = retention.AUTO_CHUNK
    retention.AUTO_CHUNK = False
    yield
    retention.AUTO_CHUNK = old
