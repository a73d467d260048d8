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

    if not os.path.isfile(build.LIB_PATH):
        build.build()
    return build.LIB_PATH


@pytest.fixture(scope="session")
def hostcheck_library():
    """The per-edge formulas of the kernels (csrc/edge_math.cuh, csrc/symcon_plan.hpp) compiled for the host by g++:
    test infrastructure, built next to its source under tests/hostcheck/ and never part of the product's lib/."""
    import subprocess

    here = os.path.join(ROOT, "tests", "hostcheck")
    src, out = os.path.join(here, "hostcheck.cpp"), os.path.join(here, "libcmace_hostcheck.so")
    csrc = os.path.join(ROOT, "cuda_mace_b200", "csrc")
    newest = max(os.path.getmtime(os.path.join(csrc, f)) for f in os.listdir(csrc) if f.endswith((".cuh", ".hpp", ".inc")))
    if not os.path.isfile(out) or os.path.getmtime(out) < max(os.path.getmtime(src), newest):
        r = subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I" + csrc, "-o", out, src],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    return out


@pytest.fixture(scope="session")
def U():
    from cuda_mace_b200 import cg

    return cg.u_matrices()
