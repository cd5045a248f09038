import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box: pytest -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def lib():
    """The product library. Fails loudly when it is not built: the GPU tests never fall back to anything."""
    import libosmos_b200
    return libosmos_b200.load()


@pytest.fixture(scope="session")
def dev():
    import torch
    assert torch.cuda.is_available(), "a gpu-marked test ran without a CUDA device"
    torch.cuda.init()
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _release_device_tensors():
    yield
    try:
        import helpers
        helpers.release()
    except ImportError:
        pass
