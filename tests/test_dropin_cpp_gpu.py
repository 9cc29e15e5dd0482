"""Runs the C++ client of the drop-in header (tests/cpp/dropin_test.cu): the
reference's own test invariants, written against nv::merlin::HashTable and
linked with libhkv_b200.so."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "tests", "cpp", "build", "dropin_test")


@pytest.mark.gpu
def test_cpp_client_of_the_dropin_header(product_lib):
    if not os.path.exists(BINARY):
        subprocess.run(["make", "-C", os.path.join(ROOT, "tests", "cpp")], check=True)
    r = subprocess.run([BINARY], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout


def test_cpp_client_compiles(product_lib):
    """nvcc cross-compiles the client without a GPU: the header keeps the
    reference's class, option and method names."""
    r = subprocess.run(["make", "-C", os.path.join(ROOT, "tests", "cpp")], capture_output=True,
                       text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert os.path.exists(BINARY)
