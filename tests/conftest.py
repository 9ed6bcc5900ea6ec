import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "projection_golden.npz"))


@pytest.fixture(scope="session")
def oracle():
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference_oracle():
    from oracle.oracle import Oracle, reference_available
    if not reference_available():
        pytest.skip("oracle/_ref was not built (no reference checkout)")
    return Oracle(reference=True)


@pytest.fixture(scope="session")
def backend():
    """One CudaBackend on device 0; fails (not skips) when the library or the
    device is missing, so a silent fallback cannot pass."""
    from tessera_b200.backend import CreateBackend
    b = CreateBackend()
    b.SetDeviceIndex(0)
    b.Init()
    yield b
    b.Synchronize()
    b.close()


def rel_err(y, r):
    """max |y - r| / max |r|: the 2e-3 bound of the projection outputs is
    stated against the largest reference magnitude because single outputs of
    a signed sum can be arbitrarily close to zero."""
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(r, dtype=np.float64)
    return float(np.abs(y - r).max() / max(np.abs(r).max(), 1e-30))


def per_element_ok(y, r, tol=2e-3):
    """The per-element form of the projection bound: |y - r| <= tol*|r| + tol*rms(r) for every
    output, which also holds outputs near zero to the scale of the whole vector."""
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(r, dtype=np.float64)
    rms = float(np.sqrt(np.mean(r * r)))
    return bool(np.all(np.abs(y - r) <= tol * np.abs(r) + tol * rms))
