"""Generates tests/golden/moe_golden.npz: a small routed-expert case (6 experts, 4 selected,
hidden 512, expert width 256; the seeded weight tensors are rebuilt by expert_tensors() and not
stored) with the outputs of the reference's own CpuMoeExpertsForward
(src/core/numerics/moe_cpu.cpp:66-131 of the reference, reached through
oracle/_ref/libtessera_ref.so).  Run from the repository root where the reference checkout is
available:

    python tests/golden/make_moe_golden.py

The tests compare the oracle's restatement of the device contracts (gate/up, then down) and
the CUDA kernels with it.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.oracle import Oracle  # noqa: E402
from tessera_b200 import synth  # noqa: E402

HIDDEN, INTER, EXPERTS, TOP_K = 512, 256, 6, 4


def expert_tensors(seed):
    """Zero-mean weights (the projection fixtures' generator has a positive mean, which would
    saturate silu): E experts, each gate/up (INTER x HIDDEN) and down (HIDDEN x INTER)."""
    gate = np.concatenate([synth.q4k_weights(INTER, HIDDEN, seed=seed + e, index=1) for e in range(EXPERTS)])
    up = np.concatenate([synth.q4k_weights(INTER, HIDDEN, seed=seed + e, index=2) for e in range(EXPERTS)])
    down4 = np.concatenate([synth.q4k_weights(HIDDEN, INTER, seed=seed + e, index=3) for e in range(EXPERTS)])
    down6 = np.concatenate([synth.q6k_weights(HIDDEN, INTER, seed=seed + e, index=4) for e in range(EXPERTS)])
    return gate, up, down4, down6


def main() -> None:
    ref = Oracle(reference=True)
    g = np.random.default_rng(20261127)
    gate, up, down4, down6 = expert_tensors(500)
    x = (g.standard_normal(HIDDEN) * 0.02).astype(np.float32)
    ids = np.array([4, 0, 5, 2], dtype=np.uint32)
    wts = g.random(TOP_K).astype(np.float32)
    wts /= wts.sum()
    acc0 = g.standard_normal(HIDDEN).astype(np.float32)
    per_gu = INTER * (HIDDEN // 256) * 144
    out = {"x": x, "ids": ids, "wts": wts, "acc0": acc0}
    out["acc_q4k"] = ref.moe_experts_forward(x, ids, wts, gate, per_gu, up, per_gu, 10, down4, HIDDEN * (INTER // 256) * 144,
                                             HIDDEN, INTER, acc0)
    out["acc_q6k"] = ref.moe_experts_forward(x, ids, wts, gate, per_gu, up, per_gu, 12, down6, HIDDEN * (INTER // 256) * 210,
                                             HIDDEN, INTER, acc0)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
