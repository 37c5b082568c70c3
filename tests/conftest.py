import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure), built on demand."""
    from oracle import oracle

    oracle.lib()
    oracle.set_threads(min(8, oracle.hardware_threads()))
    return oracle


@pytest.fixture(scope="session")
def gpu_backend():
    """Initialised C-ABI backend on cuda:0; fails loudly when the library cannot load."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from speedycolibri_b200 import backend

    backend.init([0])
    return backend
