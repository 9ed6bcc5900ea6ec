"""Generates tests/golden/elementwise_golden.npz from the reference's own host functions
RmsNormRef, AddRef, SiluMulRef, SigmoidGateRef, L2NormRef, RmsNormGatedRef, SsmGateRef
(src/core/numerics/norm.cpp) and QGateSplitRef, RepeatHeadsRef, MropeRef, DeltaStepHeadsRef (attention.cpp), Conv1dStepRef (conv.cpp of the
reference, reached
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
    # the steps between the projections
    out["sig_a"], out["sig_g"] = a[:500].copy(), gate[:500].copy()
    out["sig_o"] = ref.sigmoid_gate(out["sig_a"], out["sig_g"])
    out["l2_x"] = x
    out["l2_y"] = ref.l2norm(x, 1e-6, 0.0883883)
    gx = g.standard_normal((4, 384)).astype(np.float32)
    gw = (1.0 + 0.2 * g.standard_normal(384)).astype(np.float32)
    gg = (g.standard_normal((4, 384)) * 3).astype(np.float32)
    out["rg_x"], out["rg_w"], out["rg_g"] = gx, gw, gg
    out["rg_y"] = ref.rmsnorm_gated(gx, gw, gg, 1e-6)
    heads, rows = 48, 3
    out["ssm_a_log"] = (-np.exp(g.standard_normal(heads))).astype(np.float32)
    out["ssm_dt"] = g.standard_normal(heads).astype(np.float32)
    out["ssm_alpha_raw"] = (g.standard_normal((rows, heads)) * 8).astype(np.float32)
    out["ssm_alpha_raw"][0, :3] = [25.0, -40.0, 19.99]
    out["ssm_beta_raw"] = (g.standard_normal((rows, heads)) * 4).astype(np.float32)
    out["ssm_alpha"], out["ssm_beta"] = ref.ssm_gate(out["ssm_a_log"], out["ssm_dt"], out["ssm_alpha_raw"], out["ssm_beta_raw"])
    fused = g.standard_normal(2 * 6 * 2 * 32).astype(np.float32)
    out["qg_fused"] = fused
    out["qg_q"], out["qg_gate"] = ref.qgate_split(fused, 6, 32, 2)
    rin = g.standard_normal(4 * 16).astype(np.float32)
    out["rep_in"] = rin
    out["rep_out"] = ref.repeat_heads(rin, 12, 16, 3)
    io = g.standard_normal(2 * 3 * 64).astype(np.float32)
    pos = np.array([[5, 2, 9], [4096, 17, 3]], dtype=np.uint64)
    out["rope_io"], out["rope_pos"] = io, pos
    out["rope_out"] = ref.mrope(io, pos, 2, 3, 64, 48, 11, 8, 5, 1e7)
    heads, dk, dv = 3, 20, 24
    st = (g.standard_normal(heads * dk * dv) * 0.3).astype(np.float32)
    kk, qq = (g.standard_normal(heads * dk) * 0.2).astype(np.float32), g.standard_normal(heads * dk).astype(np.float32)
    vv = g.standard_normal(heads * dv).astype(np.float32)
    al, be = g.random(heads).astype(np.float32), g.random(heads).astype(np.float32)
    out["ds_s"], out["ds_k"], out["ds_v"], out["ds_q"], out["ds_alpha"], out["ds_beta"] = st, kk, vv, qq, al, be
    out["ds_s_out"], out["ds_o"] = ref.delta_step_heads(st, kk, vv, qq, al, be, heads, dk, dv)
    cx, cw = g.standard_normal(40 * 4).astype(np.float32), g.standard_normal(40 * 4).astype(np.float32)
    out["conv_x"], out["conv_w"] = cx, cw
    out["conv_y"] = ref.conv1d_step(cx, cw, 40, 4)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "elementwise_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
