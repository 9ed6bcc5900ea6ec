"""Generates tests/golden/attention_golden.npz from the reference's own host functions AttentionRef,
AttentionRefF16, AttentionQ8Ref, AttentionQ4Ref and AttentionFp8Ref (src/core/numerics/attention.cpp of the
reference, reached through oracle/_ref/libtessera_ref.so, which oracle/Makefile builds from the reference
checkout).  Run from the repository root where the reference checkout is available:

    python tests/golden/make_attention_golden.py

The fixture holds one small seeded cache in the five formats together with the reference's outputs for a
few (q_base, window, causal) settings; the tests compare the C restatement (oracle/) and the CUDA kernels
with it.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.oracle import Oracle  # noqa: E402

# (q_base, window, causal); the last row of q_base 38 sits past the cache and is clamped to its last key
SETTINGS = [(0, 0, 1), (37, 0, 1), (38, 16, 1), (5, 0, 0)]


def caches(g, n, kv_heads, head_dim):
    """The same seeded cache as fp32, fp16 bytes, int8, packed 4-bit and FP8 bytes (+ per-row scales)."""
    row = kv_heads * head_dim
    out = {}
    for name in ("k", "v"):
        x = g.standard_normal((n, row)).astype(np.float32)
        out[name + "_f32"] = x
        out[name + "_f16"] = x.astype(np.float16).view(np.uint8)
        out[name + "_i8"] = g.integers(-127, 128, (n, row)).astype(np.int8).view(np.uint8)
        nib = g.integers(0, 16, (n, row)).astype(np.uint8)
        out[name + "_i4"] = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
        fp8 = g.integers(0, 256, (n, row)).astype(np.uint8)
        fp8[(fp8 & 0x7F) == 0x7F] = 0x3C  # no NaN codes
        out[name + "_f8"] = fp8
        out[name + "_scale"] = (0.004 + 0.01 * g.random(n)).astype(np.float32)
    return out


def main() -> None:
    ref = Oracle(reference=True)
    g = np.random.default_rng(20261127)
    m, n, heads, kv_heads, head_dim = 3, 40, 4, 2, 128
    out = {"dims": np.array([m, n, heads, kv_heads, head_dim], dtype=np.int64),
           "settings": np.array(SETTINGS, dtype=np.int64)}
    out["q"] = g.standard_normal((m, heads * head_dim)).astype(np.float32)
    out.update(caches(g, n, kv_heads, head_dim))
    for fmt, tag in enumerate(("f32", "f16", "i8", "i4", "f8")):
        for si, (q_base, window, causal) in enumerate(SETTINGS):
            if not causal and fmt != 0:
                continue  # only AttentionRef takes the flag
            out[f"out_{tag}_{si}"] = ref.attention(fmt, out["q"], out["k_" + tag], out["v_" + tag], m, n, heads, kv_heads,
                                                   head_dim, q_base, window, bool(causal), out["k_scale"], out["v_scale"])
    path = os.path.join(ROOT, "tests", "golden", "attention_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
