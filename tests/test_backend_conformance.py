"""The C++ CudaBackend driven through the reference's own Backend interface,
launch helpers and cross-device helpers (tests/cpp/backend_conformance.cpp)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "tests", "cpp", "build", "backend_conformance")


@pytest.mark.gpu
def test_cpp_backend_conformance():
    if not os.path.exists(BINARY):
        pytest.skip("conformance driver not built (needs the reference checkout at build time)")
    run = subprocess.run([BINARY], capture_output=True, text=True, timeout=300)
    print(run.stdout[-4000:])
    print(run.stderr[-2000:])
    assert run.returncode == 0, run.stdout[-2000:]
    assert "ALL PASS" in run.stdout
    assert "FAIL " not in run.stdout
