import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """librode_b200.so, compiled on demand (nvcc cross-compiles without a GPU)."""
    from rode_b200 import build

    return build.build_library()


@pytest.fixture(scope="session")
def oracle_cpu():
    from oracle import cpu

    cpu.build()
    return cpu


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
