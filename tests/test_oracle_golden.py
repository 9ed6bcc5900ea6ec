"""The CPU oracle against the reference's golden vectors and known answers."""
import numpy as np
import pytest

from tessera_b200 import synth


def test_known_answers(oracle):
    # values stated in the reference's own comments
    # (src/core/numerics/quant.hpp:21,94,102,109,565,573)
    assert oracle.fp16_to_float([0x3C00])[0] == 1.0
    # The usage comments at quant.hpp:94,565 pair 0x40 with 1.0; the reference's
    # compiled functions (and OCP E4M3, bias 7) pair 0x38 with 1.0 and 0x40
    # with 2.0.  The code is what the kernels must match.
    assert oracle.fp8e4m3_to_float([0x38])[0] == 1.0
    assert oracle.fp8e4m3_to_float([0x40])[0] == 2.0
    assert oracle.e8m0_to_float([127])[0] == 1.0
    assert oracle.f4e2m1_to_float([3])[0] == 1.5
    assert oracle.fp32_to_fp8e4m3([1.0])[0] == 0x38
    assert oracle.fp32_to_f4e2m1([1.5])[0] == 3
    # E2M1 magnitudes (src/backends/vulkan/kernels/gemm_mxfp4.comp:47-49)
    assert list(oracle.f4e2m1_to_float(range(8))) == [0, .5, 1, 1.5, 2, 3, 4, 6]
    assert list(oracle.f4e2m1_to_float(range(8, 16))) == [-0., -.5, -1, -1.5, -2, -3, -4, -6]


def test_codecs_match_golden(oracle, golden):
    allb = np.arange(256)
    assert np.array_equal(oracle.fp8e4m3_to_float(allb), golden["e4m3_decode"], equal_nan=True)
    assert np.array_equal(oracle.e8m0_to_float(allb), golden["e8m0_decode"])
    assert np.array_equal(oracle.f4e2m1_to_float(range(16)), golden["e2m1_decode"])
    assert np.array_equal(oracle.fp16_to_float(golden["fp16_bits"]), golden["fp16_decode"], equal_nan=True)
    assert np.array_equal(oracle.fp32_to_fp8e4m3(golden["encode_in"]), golden["e4m3_encode"])
    assert np.array_equal(oracle.fp32_to_f4e2m1(golden["encode_in"]), golden["e2m1_encode"])


def test_numpy_codec_helpers_match_golden(golden):
    assert np.array_equal(synth.e4m3_decode_table(), golden["e4m3_decode"], equal_nan=True)
    x = golden["encode_in"]
    ok = np.isfinite(x) & (np.abs(x) <= 448)
    assert np.array_equal(synth.e4m3_encode(x[ok]), golden["e4m3_encode"][ok])


def test_block_dequant_and_gemm_match_golden(oracle, golden):
    a = golden["a"]
    assert np.array_equal(oracle.dequant_blocks(0, golden["q4k_w"]), golden["q4k_dequant"])
    assert np.array_equal(oracle.dequant_blocks(1, golden["q6k_w"]), golden["q6k_dequant"])
    assert np.array_equal(oracle.gemm_q4k(a, golden["q4k_w"], 3, 16, 512), golden["q4k_gemm"])
    assert np.array_equal(oracle.gemm_q6k(a, golden["q6k_w"], 3, 16, 512), golden["q6k_gemm"])
    assert np.array_equal(oracle.gemm_mxfp4(a, golden["mxfp4_w"], 3, 16, 512), golden["mxfp4_gemm"])
    assert np.array_equal(oracle.gemm_fp8(golden["fp8_a"], golden["fp8_w"], golden["fp8_s"], 2, 16, 200),
                          golden["fp8_gemm"])


def test_threaded_gemm_is_identical(oracle, golden):
    a = golden["a"]
    assert np.array_equal(oracle.gemm_q4k(a, golden["q4k_w"], 3, 16, 512, threads=4), golden["q4k_gemm"])
    assert np.array_equal(oracle.gemm_q6k(a, golden["q6k_w"], 3, 16, 512, threads=3), golden["q6k_gemm"])
    assert np.array_equal(oracle.gemm_mxfp4(a, golden["mxfp4_w"], 3, 16, 512, threads=4), golden["mxfp4_gemm"])
    assert np.array_equal(oracle.gemm_fp8(golden["fp8_a"], golden["fp8_w"], golden["fp8_s"], 2, 16, 200, threads=2),
                          golden["fp8_gemm"])


def test_activation_quant_matches_golden(oracle, golden):
    qdq, scale = oracle.quantize_fp8(golden["quant_in"])
    assert np.array_equal(qdq, golden["quant_qdq"], equal_nan=True)
    assert np.array_equal(scale, golden["quant_scale"])
    codes, scale2 = oracle.quantize_fp8_pack(golden["quant_in"])
    assert np.array_equal(codes, golden["quant_codes"])
    assert np.array_equal(scale2, golden["quant_scale"])
    # zero row: minimum scale 1/(448*512), all-zero codes
    assert scale[1] == np.float32(1.0) / (np.float32(448.0) * np.float32(512.0))
    assert not codes[1].any()
    x = golden["encode_in"]
    assert np.array_equal(oracle.round_bf16(x[np.isfinite(x)]), golden["round_bf16"])


def test_w4a8_fold_matches_golden(oracle, golden):
    fold, wref = oracle.fold_mxfp4_to_fp8(golden["mxfp4_w"], 16, 512)
    assert np.array_equal(fold, golden["w4a8_fold"])
    assert np.array_equal(wref, golden["w4a8_wref"])
    assert np.array_equal(oracle.mxfp4_row_ref(golden["mxfp4_w"], 16, 512), golden["w4a8_wref"])
    c = oracle.gemm_mxfp4_fp8(golden["w4a8_a8"], golden["w4a8_as"], fold, wref, 3, 16, 512)
    assert np.array_equal(c, golden["w4a8_gemm"])
    # the kernel-side twin folds inside the loop and must agree with fold+gemm
    twin = oracle.gemm_mxfp4_wmma(golden["w4a8_a8"], golden["mxfp4_w"], golden["w4a8_as"], wref, 3, 16, 512, 1)[0]
    assert np.abs(twin - c).max() <= 1e-5 * np.abs(c).max()


def test_fold_table_rows(oracle, golden):
    """Every (relative exponent, nibble) entry of the fold table, d = 0..17."""
    rows = 18
    codes16 = np.arange(16, dtype=np.uint8)
    blob = np.zeros((rows, 32), dtype=np.uint8)
    blob[:, 16:24] = codes16[0::2] | (codes16[1::2] << 4)
    sc = np.zeros((rows, 2), dtype=np.uint8)
    sc[:, 0] = 140
    sc[:, 1] = 140 - np.arange(rows)
    packed = np.concatenate([blob.reshape(-1), sc.reshape(-1)])
    fold, wref = oracle.fold_mxfp4_to_fp8(packed, rows, 64)
    assert np.array_equal(fold[:, 32:48], golden["fold_table"])
    assert np.array_equal(wref, golden["fold_table_wref"])
    # the 0x4c entry for magnitude 6 at d = 0 and the flush to zero at d >= 13
    assert fold[0, 32 + 7] == 0x4C and not (fold[13:, 32:48] & 0x7F).any()


def test_split_partials_sum_to_full(oracle, golden):
    a = golden["a"]
    full = golden["q4k_gemm"]
    part = oracle.gemm_vec_split(0, a, golden["q4k_w"], 3, 16, 512, 2)
    assert part.shape == (2, 3, 16)
    red = oracle.gemm_vec_reduce(part).reshape(3, 16)
    assert np.abs(red - full).max() <= 1e-5 * np.abs(full).max()
    one = oracle.gemm_vec_split(0, a, golden["q4k_w"], 3, 16, 512, 1)[0]
    assert np.array_equal(one, full)


def test_split_rule(oracle):
    # src/core/decode_internal.hpp:866-885: n=5120,k=17408 -> 68 superblocks, split 4
    assert oracle.gemm_vec_split_rule(5120, 17408) == 4
    assert oracle.gemm_vec_split_rule(17408, 5120) == 1
    assert oracle.gemm_vec_split_rule(5120, 5120) == 4
    assert oracle.gemm_vec_split_rule(8, 256 * 7) == 7
    assert oracle.gemm_vec_split_rule(8, 256 * 11) == 1


def test_tp_reduce_order(oracle):
    g = np.random.default_rng(5)
    parts = [g.standard_normal(64).astype(np.float32) * 10 ** i for i in range(4)]
    out = oracle.tp_reduce(parts)
    exp = parts[0].copy()
    for p in parts[1:]:
        exp = exp + p
    assert np.array_equal(out, exp)


def test_oracle_equals_reference_build(oracle, reference_oracle):
    """Fresh random inputs: the restatement and the reference's compiled host
    functions agree bit for bit."""
    n, k, m = 24, 768, 4
    a = synth.activations(m, k, seed=11)
    w4, w6 = synth.q4k_weights(n, k, seed=11), synth.q6k_weights(n, k, seed=11)
    wm = synth.mxfp4_weights(n, k, seed=11)
    wf, sf = synth.fp8_weights(n, k, seed=11)
    assert np.array_equal(oracle.gemm_q4k(a, w4, m, n, k), reference_oracle.gemm_q4k(a, w4, m, n, k))
    assert np.array_equal(oracle.gemm_q6k(a, w6, m, n, k), reference_oracle.gemm_q6k(a, w6, m, n, k))
    assert np.array_equal(oracle.gemm_mxfp4(a, wm, m, n, k), reference_oracle.gemm_mxfp4(a, wm, m, n, k))
    assert np.array_equal(oracle.gemm_fp8(a, wf, sf, m, n, k), reference_oracle.gemm_fp8(a, wf, sf, m, n, k))
    q1, s1 = oracle.quantize_fp8(a)
    q2, s2 = reference_oracle.quantize_fp8(a)
    assert np.array_equal(q1, q2) and np.array_equal(s1, s2)


def test_elementwise_steps_match_golden(oracle):
    """RmsNormRef, SiluMulRef, AddRef (src/core/numerics/norm.cpp of the reference)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "elementwise_golden.npz"))
    for i, eps in enumerate(g["rms_eps"]):
        assert np.array_equal(oracle.rmsnorm(g["rms_x"], g["rms_w"], float(eps)), g["rms_y"][i])
    assert np.array_equal(oracle.silu_mul(g["silu_g"], g["silu_u"]), g["silu_o"], equal_nan=True)
    assert np.array_equal(oracle.add(g["add_a"], g["add_b"]), g["add_o"])


def test_steps_between_the_projections_match_golden(oracle):
    """SigmoidGateRef, L2NormRef, RmsNormGatedRef, SsmGateRef (norm.cpp), QGateSplitRef, RepeatHeadsRef
    (attention.cpp) of the reference."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "elementwise_golden.npz"))
    assert np.array_equal(oracle.sigmoid_gate(g["sig_a"], g["sig_g"]), g["sig_o"])
    assert np.array_equal(oracle.l2norm(g["l2_x"], 1e-6, 0.0883883), g["l2_y"])
    assert np.array_equal(oracle.rmsnorm_gated(g["rg_x"], g["rg_w"], g["rg_g"], 1e-6), g["rg_y"])
    alpha, beta = oracle.ssm_gate(g["ssm_a_log"], g["ssm_dt"], g["ssm_alpha_raw"], g["ssm_beta_raw"])
    assert np.array_equal(alpha, g["ssm_alpha"]) and np.array_equal(beta, g["ssm_beta"])
    q, gate = oracle.qgate_split(g["qg_fused"], 6, 32, 2)
    assert np.array_equal(q, g["qg_q"]) and np.array_equal(gate, g["qg_gate"])
    assert np.array_equal(oracle.repeat_heads(g["rep_in"], 12, 16, 3), g["rep_out"])


def test_rope_and_delta_rule_match_golden(oracle):
    """MropeRef and DeltaStepHeadsRef (src/core/numerics/attention.cpp of the reference)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "elementwise_golden.npz"))
    assert np.array_equal(oracle.mrope(g["rope_io"], g["rope_pos"], 2, 3, 64, 48, 11, 8, 5, 1e7), g["rope_out"])
    s, o = oracle.delta_step_heads(g["ds_s"], g["ds_k"], g["ds_v"], g["ds_q"], g["ds_alpha"], g["ds_beta"], 3, 20, 24)
    assert np.array_equal(s, g["ds_s_out"]) and np.array_equal(o, g["ds_o"])


def test_conv_step_matches_golden_and_underlies_conv1d_state(oracle):
    """Conv1dStepRef (src/core/numerics/conv.cpp of the reference); the device-only conv1d_state contract
    is that convolution over [current, history] with the taps reversed, then SiLU and the split."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "elementwise_golden.npz"))
    assert np.array_equal(oracle.conv1d_step(g["conv_x"], g["conv_w"], 40, 4), g["conv_y"])
    rng = np.random.default_rng(3)
    c, w_, kd = 40, 4, 10
    hist = rng.standard_normal(c * (w_ - 1)).astype(np.float32)
    qkv = rng.standard_normal(c).astype(np.float32)
    q, k, v, hist2, _ = oracle.conv1d_state(qkv, g["conv_w"], hist, c, w_, kd, 0, 1)
    xs = np.concatenate([qkv[:, None], hist.reshape(c, w_ - 1)], axis=1).reshape(-1)
    wr = g["conv_w"].reshape(c, w_)[:, ::-1].copy().reshape(-1)
    acc = oracle.conv1d_step(xs, wr, c, w_).astype(np.float64)
    want = (acc / (1 + np.exp(-acc))).astype(np.float32)
    assert np.abs(np.concatenate([q, k, v]) - want).max() <= 1e-6
    assert np.array_equal(hist2.reshape(c, w_ - 1)[:, 0], qkv) and np.array_equal(hist2.reshape(c, w_ - 1)[:, 1:], hist.reshape(c, w_ - 1)[:, :-1])


ATTENTION_TAGS = ("f32", "f16", "i8", "i4", "f8")


def test_attention_matches_golden(oracle):
    """AttentionRef and its cache-decoding wrappers (src/core/numerics/attention.cpp:45-214 of the reference):
    every cache format, the causal prefix, a query row past the cache, a sliding window, the non-causal form."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    m, n, heads, kv_heads, head_dim = (int(x) for x in g["dims"])
    checked = 0
    for fmt, tag in enumerate(ATTENTION_TAGS):
        for si, (q_base, window, causal) in enumerate(g["settings"]):
            key = f"out_{tag}_{si}"
            if key not in g:
                continue
            y = oracle.attention(fmt, g["q"], g["k_" + tag], g["v_" + tag], m, n, heads, kv_heads, head_dim, int(q_base),
                                 int(window), bool(causal), g["k_scale"], g["v_scale"])
            assert np.array_equal(y, g[key]), key
            checked += 1
    assert checked == 16


def test_rope_and_cache_writers_match_golden(oracle):
    """RopeRef (src/core/numerics/attention.cpp:11-43) and QuantizeQ8Ref / QuantizeQ4Ref (quant.cpp:123-181)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    assert np.array_equal(oracle.rope(g["rope_io"], 3, 2, 64, 48, 1021, 1e6), g["rope_out"])
    for kind, tag in ((0, "kvq8"), (1, "kvq4")):
        codes, scale = oracle.quantize_rows(kind, g["kvq_in"])
        assert np.array_equal(codes, g[tag + "_codes"]) and np.array_equal(scale, g[tag + "_scale"])
    assert g["kvq8_scale"][3] == 1.0 and not g["kvq8_codes"][3].any()  # the zero row


def test_dense_projections_match_golden(oracle):
    """GemmF32Ref / GemmBf16Ref (src/core/numerics/gemm.cpp:205-252 of the reference)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    assert np.array_equal(oracle.gemm_dense(False, g["dense_a"], g["dense_w32"], 3, 9, 75), g["dense_c32"])
    assert np.array_equal(oracle.gemm_dense(True, g["dense_a"], g["dense_w16"], 3, 9, 75), g["dense_c16"])
