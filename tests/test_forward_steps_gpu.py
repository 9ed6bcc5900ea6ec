"""The elementwise and row-wise steps between the projections on the GPU against the CPU
oracle (bit-equal to the reference's *Ref functions, tests/test_oracle_golden.py): same
formulas; sums of squares are added as a tree on the device, so norms agree to rounding."""
import numpy as np
import pytest

from tessera_b200 import capi
from tessera_b200.backend import KernelLaunch

pytestmark = pytest.mark.gpu


def bits(x):
    return int(np.float32(x).view(np.uint32))


def close(y, r, tol):
    return bool(np.all(np.abs(y - r) <= tol * np.abs(r) + 1e-30))


def run(backend, name, buffers, scalars):
    backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=buffers, scalars=scalars))


def test_sigmoid_gate(backend, oracle):
    g = np.random.default_rng(1)
    n = 6144 + 3
    a = g.standard_normal(n).astype(np.float32)
    gate = (g.standard_normal(n) * 6).astype(np.float32)
    gate[:3] = [0.0, 95.0, -95.0]
    out = backend.AllocateBuffer(n * 4)
    run(backend, "sigmoid_gate", [backend.upload(a), backend.upload(gate), out], [n])
    assert close(backend.download(out, np.float32, n), oracle.sigmoid_gate(a, gate), 4e-7)


@pytest.mark.parametrize("rows,cols", [(48, 128), (3, 1000), (1, 17)])
def test_l2norm(backend, oracle, rows, cols):
    g = np.random.default_rng(rows + cols)
    x = (g.standard_normal((rows, cols)) * 5).astype(np.float32)
    out = backend.AllocateBuffer(x.nbytes)
    run(backend, "l2norm", [backend.upload(x), out], [rows, cols, bits(1e-6), bits(0.088388)])
    assert close(backend.download(out, np.float32, x.size).reshape(rows, cols), oracle.l2norm(x, 1e-6, np.float32(0.088388)), 2e-6)


def test_rmsnorm_gated_with_bases(backend, oracle):
    """The gate is read and the output written at element bases inside larger buffers (one
    token's slice of a batched buffer)."""
    g = np.random.default_rng(5)
    rows, cols, gbase, ybase = 48, 128, 6144, 2 * 6144
    x = g.standard_normal((rows, cols)).astype(np.float32)
    w = (1 + 0.1 * g.standard_normal(cols)).astype(np.float32)
    gate_all = (g.standard_normal(gbase + rows * cols + 64) * 3).astype(np.float32)
    canary = np.float32(9.5e9)
    y_all = np.full(ybase + rows * cols + 64, canary, dtype=np.float32)
    yb = backend.upload(y_all)
    run(backend, "rmsnorm_gated", [backend.upload(x), backend.upload(w), backend.upload(gate_all), yb],
        [rows, cols, bits(1e-6), gbase, ybase])
    got = backend.download(yb, np.float32, y_all.size)
    assert np.all(got[:ybase] == canary) and np.all(got[ybase + rows * cols:] == canary)
    want = oracle.rmsnorm_gated(x, w, gate_all[gbase:gbase + rows * cols].reshape(rows, cols), 1e-6)
    assert close(got[ybase:ybase + rows * cols].reshape(rows, cols), want, 3e-6)


def test_ssm_gate(backend, oracle):
    g = np.random.default_rng(6)
    heads, rows = 48, 5
    a_log = (-np.exp(g.standard_normal(heads))).astype(np.float32)
    dt = g.standard_normal(heads).astype(np.float32)
    alpha_raw = (g.standard_normal((rows, heads)) * 8).astype(np.float32)
    alpha_raw[0, :3] = [25.0, -40.0, 19.99]
    beta_raw = (g.standard_normal((rows, heads)) * 4).astype(np.float32)
    ab, bb = backend.AllocateBuffer(rows * heads * 4), backend.AllocateBuffer(rows * heads * 4)
    run(backend, "ssm_gate", [backend.upload(a_log), backend.upload(dt), backend.upload(alpha_raw), backend.upload(beta_raw), ab, bb],
        [heads, rows])
    alpha, beta = oracle.ssm_gate(a_log, dt, alpha_raw, beta_raw)
    assert close(backend.download(ab, np.float32, rows * heads).reshape(rows, heads), alpha, 2e-6)
    assert close(backend.download(bb, np.float32, rows * heads).reshape(rows, heads), beta, 4e-7)


def test_qgate_split_and_repeat_heads_are_exact(backend, oracle):
    g = np.random.default_rng(7)
    heads, dim, rows = 24, 256, 3
    fused = g.standard_normal(rows * heads * 2 * dim).astype(np.float32)
    qb, gb = backend.AllocateBuffer(fused.nbytes // 2), backend.AllocateBuffer(fused.nbytes // 2)
    run(backend, "qgate_split", [backend.upload(fused), qb, gb], [heads, dim, rows])
    q, gate = oracle.qgate_split(fused, heads, dim, rows)
    assert np.array_equal(backend.download(qb, np.float32, q.size), q)
    assert np.array_equal(backend.download(gb, np.float32, gate.size), gate)
    vh, kd, factor, rows = 48, 128, 3, 2
    x = g.standard_normal(rows * (vh // factor) * kd).astype(np.float32)
    ob = backend.AllocateBuffer(rows * vh * kd * 4)
    run(backend, "repeat_heads", [backend.upload(x), ob], [vh, kd, factor, rows])
    want = np.concatenate([oracle.repeat_heads(x.reshape(rows, -1)[r], vh, kd, factor) for r in range(rows)])
    assert np.array_equal(backend.download(ob, np.float32, want.size), want)


def test_steps_check_their_arguments(backend):
    buf = backend.AllocateBuffer(1024)
    for name, buffers, scalars in [
        ("sigmoid_gate", [buf, buf, buf], [1024]),                              # 4096 bytes needed
        ("l2norm", [buf, buf], [2, 256, bits(-1.0), bits(1.0)]),                 # eps < 0
        ("rmsnorm_gated", [buf, buf, buf, buf], [1, 128, bits(1e-6), 200, 0]),   # gate base beyond the buffer
        ("ssm_gate", [buf, buf, buf, buf, buf, buf], [300, 1]),                  # heads beyond the buffers
        ("qgate_split", [buf, buf, buf], [4, 64, 1]),                            # fused too small
        ("repeat_heads", [buf, buf], [12, 16, 5, 1]),                            # heads not divisible
    ]:
        with pytest.raises(capi.StatusError):
            run(backend, name, buffers, scalars)
    backend.Synchronize()


@pytest.mark.parametrize("kind", ["f32", "bf16", "q4k"])
def test_embedding_rows_are_exact(backend, oracle, kind):
    """out[row] = table[ids[row]] as fp32, a zero row for an id beyond the table; the Q4_K table
    is decoded with the reference's rounding sequence (bit-equal to DequantizeQ4K)."""
    from tessera_b200 import synth
    g = np.random.default_rng(8)
    vocab, cols = 50, 512
    ids = np.array([3, 49, 0, 50, 7, 4000000000], dtype=np.uint32)   # two ids outside the table
    if kind == "f32":
        table = g.standard_normal((vocab, cols)).astype(np.float32)
        dense = table
    elif kind == "bf16":
        dense = (g.standard_normal((vocab, cols)).astype(np.float32).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
        table = (dense.view(np.uint32) >> 16).astype(np.uint16)
    else:
        table = synth.q4k_weights(vocab, cols, seed=8)
        dense = oracle.dequant_blocks(0, table).reshape(vocab, cols)
    out = backend.upload(np.full(ids.size * cols, np.float32(7.0)))
    run(backend, f"embedding_{kind}", [backend.upload(ids), backend.upload(table), out], [ids.size, cols, vocab])
    got = backend.download(out, np.float32, ids.size * cols).reshape(ids.size, cols)
    want = np.stack([dense[i] if i < vocab else np.zeros(cols, dtype=np.float32) for i in ids])
    assert np.array_equal(got, want)


def test_mrope(backend, oracle):
    """Positions in the thousands: the angle is formed in double precision on both sides; the
    device's double sine and cosine may differ from the host's in the last bit, which shows as
    one ulp of an fp32 factor."""
    g = np.random.default_rng(9)
    rows, heads, dim, rdim = 3, 24, 256, 64
    io = g.standard_normal(rows * heads * dim).astype(np.float32)
    pos = np.array([[7, 7, 7], [4095, 12, 300], [100000, 0, 1]], dtype=np.uint64)
    buf = backend.upload(io)
    run(backend, "mrope", [buf, backend.upload(pos)], [rows, heads, dim, rdim, bits(1e7), 11, 11, 10])
    got = backend.download(buf, np.float32, io.size)
    want = oracle.mrope(io, pos, rows, heads, dim, rdim, 11, 11, 10, float(np.float32(1e7)))
    assert np.all(np.abs(got - want) <= 3e-7 * (np.abs(want) + np.abs(io)))
    untouched = np.arange(io.size) % dim >= rdim
    assert np.array_equal(got[untouched], io[untouched])


def test_cast_f32_f16_rounds_to_nearest_even(backend):
    g = np.random.default_rng(10)
    x = np.concatenate([np.float32([0.0, -0.0, 1.0, 65504.0, 65520.0, 1e-8, 6.1e-5, 5.96e-8, 2049.0, 2051.0, -3.3, 1e9]),
                        (g.standard_normal(1012) * 50).astype(np.float32)])
    out = backend.AllocateBuffer(x.size * 2)
    run(backend, "cast_f32_f16", [backend.upload(x), out], [x.size])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    assert np.array_equal(backend.download(out, np.uint16, x.size), want.view(np.uint16))


@pytest.mark.parametrize("heads,dk,dv,rows,history", [(48, 128, 128, 1, False), (6, 128, 128, 3, True), (3, 20, 24, 2, False),
                                                      (2, 256, 40, 1, False)])
def test_delta_step_heads(backend, oracle, heads, dk, dv, rows, history):
    """rows steps in turn; with history every step's state goes to its own slot after the input
    state (slot t + 1), otherwise the state advances in place.  alpha and beta are read at an
    element base."""
    g = np.random.default_rng(heads + dk)
    state = (g.standard_normal(heads * dk * dv) * 0.3).astype(np.float32)
    k = (g.standard_normal((rows, heads * dk)) * 0.1).astype(np.float32)
    q = g.standard_normal((rows, heads * dk)).astype(np.float32)
    v = g.standard_normal((rows, heads * dv)).astype(np.float32)
    abase = 5
    alpha = g.random(abase + rows * heads).astype(np.float32)
    beta = g.random(abase + rows * heads).astype(np.float32)
    sbase = 16
    stride = heads * dk * dv if history else 0
    slots = rows + 1 if history else 1
    s_all = np.full(sbase + slots * heads * dk * dv + 8, np.float32(-7e7), dtype=np.float32)
    s_all[sbase:sbase + state.size] = state
    sb = backend.upload(s_all)
    ob = backend.AllocateBuffer(rows * heads * dv * 4)
    run(backend, "delta_step_heads", [sb, backend.upload(k), backend.upload(v), backend.upload(q), ob, backend.upload(alpha),
                                      backend.upload(beta)], [heads, dk, dv, rows, sbase, stride, abase])
    got_s = backend.download(sb, np.float32, s_all.size)
    got_o = backend.download(ob, np.float32, rows * heads * dv).reshape(rows, heads * dv)
    cur = state
    for t in range(rows):
        a_t = alpha[abase + t * heads:abase + (t + 1) * heads]
        b_t = beta[abase + t * heads:abase + (t + 1) * heads]
        cur, o = oracle.delta_step_heads(cur, k[t], v[t], q[t], a_t, b_t, heads, dk, dv)
        assert np.abs(got_o[t] - o).max() <= 2e-5 * max(np.abs(o).max(), 1e-6), t
        if history:
            slot = got_s[sbase + (t + 1) * stride:sbase + (t + 2) * stride]
            assert np.abs(slot - cur).max() <= 2e-6 * np.abs(cur).max(), t
    if history:
        assert np.array_equal(got_s[sbase:sbase + state.size], state)          # the input state stays
    else:
        assert np.abs(got_s[sbase:sbase + state.size] - cur).max() <= 2e-6 * np.abs(cur).max()
    assert np.all(got_s[:sbase] == np.float32(-7e7)) and np.all(got_s[sbase + slots * state.size:] == np.float32(-7e7))


@pytest.mark.parametrize("rows,history", [(1, False), (3, True)])
def test_conv1d_state(backend, oracle, rows, history):
    g = np.random.default_rng(11 + rows)
    conv_dim, width, key_dim, offset = 10240, 4, 2048, 64
    qkv = g.standard_normal(offset + rows * conv_dim).astype(np.float32)
    w = g.standard_normal(conv_dim * width).astype(np.float32)
    hist = g.standard_normal(conv_dim * (width - 1)).astype(np.float32)
    stride = conv_dim * (width - 1) if history else 0
    hh = np.zeros((rows + 1) * conv_dim * (width - 1) if history else 4, dtype=np.float32)
    hb, hhb = backend.upload(hist), backend.upload(hh)
    vd = conv_dim - 2 * key_dim
    qb, kb, vb = backend.AllocateBuffer(rows * key_dim * 4), backend.AllocateBuffer(rows * key_dim * 4), backend.AllocateBuffer(rows * vd * 4)
    run(backend, "conv1d_state", [backend.upload(qkv), backend.upload(w), hb, qb, kb, vb, hhb],
        [conv_dim, width, key_dim, offset, rows, stride])
    q, k, v, hist2, hh2 = oracle.conv1d_state(qkv, w, hist, conv_dim, width, key_dim, offset, rows, stride, hh if history else None)
    for buf, want in ((qb, q), (kb, k), (vb, v)):
        assert close(backend.download(buf, np.float32, want.size), want, 2e-6)
    assert np.array_equal(backend.download(hb, np.float32, hist.size), hist2)
    if history:
        assert np.array_equal(backend.download(hhb, np.float32, hh.size), hh2)


def test_top_k_rows(backend, oracle):
    g = np.random.default_rng(13)
    rows, vocab, top_k, base = 3, 5000, 8, 2
    logits = g.standard_normal((base + rows) * vocab).astype(np.float32)
    logits[base * vocab + 17] = logits[base * vocab + 4000] = 9.0      # a tie: the lower index comes first
    ib, vb = backend.AllocateBuffer(rows * top_k * 4), backend.AllocateBuffer(rows * top_k * 4)
    run(backend, "top_k_rows", [backend.upload(logits), ib, vb], [rows, vocab, top_k, base])
    ids, vals = oracle.top_k_rows(logits, rows, vocab, top_k, base)
    got_i = backend.download(ib, np.uint32, rows * top_k).reshape(rows, top_k)
    got_v = backend.download(vb, np.float32, rows * top_k).reshape(rows, top_k)
    assert np.array_equal(got_i, ids) and np.array_equal(got_v, vals)
    assert list(got_i[0][:2]) == [17, 4000]
    full = logits.reshape(base + rows, vocab)[base:]
    assert np.array_equal(np.sort(full, axis=1)[:, ::-1][:, :top_k], got_v)
    # routing shape of the MoE configuration: 256 experts, 8 selected
    lg = g.standard_normal(256).astype(np.float32)
    run(backend, "top_k_rows", [backend.upload(lg), ib, vb], [1, 256, 8, 0])
    assert np.array_equal(backend.download(ib, np.uint32, 8), np.argsort(-lg, kind="stable")[:8].astype(np.uint32))
