import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def cuda_lib():
    """The built CUDA library; GPU tests must run the native code, never a fallback."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cumm_b200 import _lib
    return _lib.load()
