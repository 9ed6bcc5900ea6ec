"""Generates tests/golden/elementwise_golden.npz from the reference's own host functions
RmsNormRef, AddRef and SiluMulRef (src/core/numerics/norm.cpp of the reference, reached
through oracle/_ref/libtessera_ref.so, which oracle/Makefile builds from the reference
checkout).  Run from the repository root where the reference checkout is available:

    python tests/golden/make_elementwise_golden.py

The fixture holds small seeded inputs together with the reference's outputs; the tests compare
the C restatement (oracle/) and the CUDA kernels with it.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.oracle import Oracle  # noqa: E402


def main() -> None:
    ref = Oracle(reference=True)
    g = np.random.default_rng(20261126)
    out = {}
    x = (g.standard_normal((3, 520)) * np.float32([[0.01], [1.0], [300.0]])).astype(np.float32)
    x[0, :8] = 0.0
    w = (1.0 + 0.2 * g.standard_normal(520)).astype(np.float32)
    out["rms_x"], out["rms_w"] = x, w
    out["rms_eps"] = np.float32([1e-6, 1e-5, 0.0])
    out["rms_y"] = np.stack([ref.rmsnorm(x, w, float(e)) for e in out["rms_eps"]])
    gate = np.concatenate([np.float32([0.0, -0.0, 1.0, -1.0, 20.0, -20.0, 88.0, -88.0, 90.0, -104.0, 1e-30, -1e-30]),
                           (g.standard_normal(1000) * 5.0).astype(np.float32)])
    up = g.standard_normal(gate.size).astype(np.float32)
    out["silu_g"], out["silu_u"] = gate, up
    out["silu_o"] = ref.silu_mul(gate, up)
    a = (g.standard_normal(777) * 1e3).astype(np.float32)
    b = g.standard_normal(777).astype(np.float32)
    out["add_a"], out["add_b"], out["add_o"] = a, b, ref.add(a, b)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "elementwise_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
