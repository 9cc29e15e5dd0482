import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_lib():
    """The CPU restatement (oracle/hkv_oracle.cpp), built on demand with g++."""
    from tests.hkv_testlib import load_oracle

    return load_oracle()


@pytest.fixture(scope="session")
def product_lib():
    """libhkv_b200.so, built on demand with nvcc (cross-compiles without a GPU)."""
    from hierarchicalkv_b200.build import build_library
    from hierarchicalkv_b200 import load_library

    build_library()
    return load_library()
