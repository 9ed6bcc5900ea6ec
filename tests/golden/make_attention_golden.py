"""Generates tests/golden/attention_golden.npz from the reference's own host functions AttentionRef,
AttentionRefF16, AttentionQ8Ref, AttentionQ4Ref, AttentionFp8Ref and RopeRef (src/core/numerics/attention.cpp of
the reference) the cache writers QuantizeQ8Ref and QuantizeQ4Ref (src/core/numerics/quant.cpp) and the unquantised projections
GemmF32Ref and GemmBf16Ref (src/core/numerics/gemm.cpp), reached through
oracle/_ref/libtessera_ref.so, which oracle/Makefile builds from the reference checkout.  Run from the repository root where the reference checkout is available:

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
    # rope: three rows from position 1021 on, rope_dim 48 of head_dim 64
    out["rope_io"] = g.standard_normal(3 * 2 * 64).astype(np.float32)
    out["rope_out"] = ref.rope(out["rope_io"], 3, 2, 64, 48, 1021, 1e6)
    # the int8 / 4-bit cache writers: ties (x / scale exactly .5), a zero row, values beyond the clamp cannot occur
    x = (g.standard_normal((5, 256)) * np.float32([[1.0], [1e-3], [50.0], [0.0], [1.0]])).astype(np.float32)
    x[4, :] = np.round(x[4, :] * 4) / 4
    x[4, 0] = 127.0 / 4  # amax: scale 0.25, so the row's values are exact multiples of the scale or ties
    out["kvq_in"] = x
    out["kvq8_codes"], out["kvq8_scale"] = ref.quantize_rows(0, x)
    out["kvq4_codes"], out["kvq4_scale"] = ref.quantize_rows(1, x)
    # the unquantised projections: fp32 and bf16 weights (bit patterns), k not a multiple of the vector width
    out["dense_a"] = g.standard_normal((3, 75)).astype(np.float32)
    out["dense_w32"] = g.standard_normal((9, 75)).astype(np.float32)
    out["dense_w16"] = (g.standard_normal((9, 75)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    out["dense_c32"] = ref.gemm_dense(False, out["dense_a"], out["dense_w32"], 3, 9, 75)
    out["dense_c16"] = ref.gemm_dense(True, out["dense_a"], out["dense_w16"], 3, 9, 75)
    path = os.path.join(ROOT, "tests", "golden", "attention_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
