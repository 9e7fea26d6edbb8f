"""The C++ free functions with the reference's names (fastertransformer_b200/shim/decode_kernels.h):
tests/cpp/kernels_driver.cc calls each of them on seeded inputs and compares with the CPU restatement."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
DRIVER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp", "_build", "kernels_driver")


def test_cxx_free_functions_against_restatement():
    if not os.path.exists(DRIVER):
        # built binaries normally travel with the tree; build here when this one did not
        import sys
        subprocess.run([sys.executable, os.path.join(os.path.dirname(DRIVER), "..", "build_kernels_driver.py")],
                       capture_output=True, text=True, timeout=600)
    if not os.path.exists(DRIVER):
        pytest.fail("tests/cpp/_build/kernels_driver is not built: run python tests/cpp/build_kernels_driver.py")
    r = subprocess.run([DRIVER], capture_output=True, text=True, timeout=300)
    lines = [l for l in r.stdout.splitlines() if l.startswith(("PASS", "FAIL"))]
    assert r.returncode == 0, r.stdout + r.stderr
    assert len(lines) >= 20 and all(l.startswith("PASS") for l in lines), r.stdout
