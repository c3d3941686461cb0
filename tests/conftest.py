import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference's Python code on small seeded inputs (tests/golden/make_golden.py)."""
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "s14_golden.npz")))


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (oracle/s14_oracle.c), built on demand with the committed Makefile."""
    from oracle import s14_oracle

    s14_oracle.build()
    return s14_oracle


@pytest.fixture(scope="session")
def cuda_lib():
    """The CUDA library, built on demand (nvcc cross-compiles without a GPU)."""
    from colormlm_b200 import build

    build.build()
    from colormlm_b200 import _lib

    return _lib.lib()
