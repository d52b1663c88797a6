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

    # a library older than its sources would be tested silently: rebuild it (nvcc is in the image; the
    # library shipped to a GPU box is newer than the sources it was built from and is used as it is)
    if not build.up_to_date():
        build.build()
    return _lib.load()
