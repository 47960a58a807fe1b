import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built_lib():
    """The C-ABI library, compiled for sm_100a if it is stale (nvcc needs no GPU)."""
    import kohaku_tt_b200 as ktt
    from kohaku_tt_b200 import _lib

    ktt.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def cuda(built_lib):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kohaku_tt_b200 as ktt

    ktt.install()
    return torch.device("cuda:0")
