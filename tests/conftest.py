import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def qgolden():
    return np.load(os.path.join(GOLDEN, "qlinear_golden.npz"))


@pytest.fixture(scope="session")
def moegolden():
    return np.load(os.path.join(GOLDEN, "moe_golden.npz"))


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and loads libb200q.so; no CUDA call is made."""
    from chadslab_b200 import build, _lib
    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def cuda_lib(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu was run without a CUDA device")
    from chadslab_b200 import _lib
    torch.cuda.set_device(0)
    return _lib.init(0)
