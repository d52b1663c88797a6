import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (compute capability 10.x) GPU")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(REPO, "tests", "golden", "reference_vectors.npz"))


@pytest.fixture(scope="session")
def lib():
    from shiftaddllm_b200 import _lib, build

    if not os.path.exists(build.LIB):   # a prebuilt library (the one shipped to the GPU box) is used as it is
        build.build()
    return _lib.load()
