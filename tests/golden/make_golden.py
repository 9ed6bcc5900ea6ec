"""Generates tests/golden/projection_golden.npz from the reference's own host
reference functions (oracle/_ref/libtessera_ref.so, built from the reference
checkout by oracle/Makefile).  Run from the repository root where the
reference checkout is available:

    python tests/golden/make_golden.py

The fixture holds small seeded inputs together with the reference's outputs;
the tests compare the C restatement (oracle/) and the CUDA kernels with it.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.oracle import Oracle  # noqa: E402
from tessera_b200 import synth  # noqa: E402


def main() -> None:
    ref = Oracle(reference=True)
    g = np.random.default_rng(20261125)
    out = {}

    # scalar codecs: exhaustive byte tables and a value sweep
    allb = np.arange(256)
    out["e4m3_decode"] = ref.fp8e4m3_to_float(allb)
    out["e8m0_decode"] = ref.e8m0_to_float(allb)
    out["e2m1_decode"] = ref.f4e2m1_to_float(np.arange(16))
    h = np.concatenate([g.integers(0, 65536, 500), [0, 0x3C00, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00]])
    out["fp16_bits"] = h.astype(np.uint16)
    out["fp16_decode"] = ref.fp16_to_float(h)
    edge = np.float32([0.0, -0.0, 1.0, 1.5, 448.0, 449.0, -448.0, 464.0, 1e-9, 2.0 ** -9, 2.0 ** -10,
                       0.0146, 0.0155, 0.015625, 0.0166, 0.00097, 0.000976, 0.0029296875, 240.0, 247.9,
                       248.0, 0.0625, 0.06640625, np.inf, -np.inf, np.nan])
    sweep = np.concatenate([edge, (g.standard_normal(1500) * 100).astype(np.float32),
                            (g.standard_normal(1500) * 0.02).astype(np.float32)])
    out["encode_in"] = sweep
    out["e4m3_encode"] = ref.fp32_to_fp8e4m3(sweep)
    out["e2m1_encode"] = ref.fp32_to_f4e2m1(sweep)

    # Q4_K / Q6_K: dequantised blocks and a 3-row GEMM
    n, k, m = 16, 512, 3
    a = synth.activations(m, k, seed=7)
    out["a"] = a
    w4 = synth.q4k_weights(n, k, seed=7)
    out["q4k_w"] = w4
    out["q4k_dequant"] = ref.dequant_blocks(0, w4)
    out["q4k_gemm"] = ref.gemm_q4k(a, w4, m, n, k)
    w6 = synth.q6k_weights(n, k, seed=7)
    out["q6k_w"] = w6
    out["q6k_dequant"] = ref.dequant_blocks(1, w6)
    out["q6k_gemm"] = ref.gemm_q6k(a, w6, m, n, k)

    # MXFP4 (wide scale range so the W4A8 fold reaches its subnormal tail)
    wm = synth.mxfp4_weights(n, k, seed=7, exp_lo=-18, exp_hi=0)
    out["mxfp4_w"] = wm
    out["mxfp4_gemm"] = ref.gemm_mxfp4(a, wm, m, n, k)

    # FP8 with a ragged k
    kf = 200
    af = synth.activations(2, kf, seed=8)
    wf, sf = synth.fp8_weights(n, kf, seed=8)
    out["fp8_a"], out["fp8_w"], out["fp8_s"] = af, wf, sf
    out["fp8_gemm"] = ref.gemm_fp8(af, wf, sf, 2, n, kf)

    # per-token FP8 quantisation: a normal row, a zero row, a tiny row, a row
    # with one large outlier and a NaN
    q_in = synth.activations(5, 384, seed=9)
    q_in[1] = 0.0
    q_in[2] *= np.float32(1e-7)
    q_in[3, 17] = np.float32(3.0e4)
    q_in[4, 5] = np.float32(np.nan)
    out["quant_in"] = q_in
    out["quant_qdq"], out["quant_scale"] = ref.quantize_fp8(q_in)
    out["quant_codes"], _ = ref.quantize_fp8_pack(q_in)
    out["round_bf16"] = ref.round_bf16(sweep[np.isfinite(sweep)])

    # W4A8: fold and the fp8 x fp8 GEMM
    a8, as_ = ref.quantize_fp8_pack(a)
    fold, wref = ref.fold_mxfp4_to_fp8(wm, n, k)
    out["w4a8_a8"], out["w4a8_as"] = a8, as_
    out["w4a8_fold"], out["w4a8_wref"] = fold, wref
    out["w4a8_gemm"] = ref.gemm_mxfp4_fp8(a8, as_, fold, wref, m, n, k)

    # the fold table itself: one row per relative exponent d = 0..17 with all
    # sixteen nibbles, produced through FoldMxFp4ToFp8
    rows = 18
    tw = np.zeros((rows, 64), dtype=np.uint8)  # two 32-element blocks per row
    codes16 = np.arange(16, dtype=np.uint8)
    tw[:, 16:24] = (codes16[0::2] | (codes16[1::2] << 4))  # second block holds nibbles 0..15
    ts = np.zeros((rows, 2), dtype=np.uint8)
    ts[:, 0] = 140                       # first block pins the row reference
    ts[:, 1] = 140 - np.arange(rows)     # second block sits d below it
    tpacked = np.concatenate([np.zeros((rows, 16), np.uint8), tw[:, 16:32]], axis=1)
    packed = np.concatenate([tpacked.reshape(-1), ts.reshape(-1)])
    tfold, tref = ref.fold_mxfp4_to_fp8(packed, rows, 64)
    out["fold_table"] = tfold[:, 32:48]
    out["fold_table_wref"] = tref

    path = os.path.join(ROOT, "tests", "golden", "projection_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
