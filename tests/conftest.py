import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the kernels through the C-ABI)")


@pytest.fixture(scope="session", autouse=True)
def built_library():
    """The C-ABI library must exist for every test (CPU tests check its exports); build on demand."""
    from cuda_mace_b200 import build

    if not (os.path.isfile(build.LIB_PATH) and os.path.isfile(build.HOSTCHECK_PATH)):
        build.build()
    return build.LIB_PATH


@pytest.fixture(scope="session")
def U():
    from cuda_mace_b200 import cg

    return cg.u_matrices()
