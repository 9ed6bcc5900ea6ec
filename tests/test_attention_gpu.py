"""Attention over the key / value cache on the GPU (ids attention, attention_q8 / _q4 / _fp8, their split
halves and attention_combine) against the CPU oracle, which is bit-equal to the reference's AttentionRef
family (tests/test_oracle_golden.py).  The device adds the keys' contributions in a different order (lanes
split head_dim, warps split the keys, chunks merge at the end), so results agree to fp32 rounding."""
import os

import numpy as np
import pytest

from tessera_b200 import capi
from tessera_b200.backend import KernelLaunch

pytestmark = pytest.mark.gpu

TAGS = ("f32", "f16", "i8", "i4", "f8")
QUANT_ID = {2: "attention_q8", 3: "attention_q4", 4: "attention_fp8"}
QUANT_KIND = {2: 0, 3: 1, 4: 2}
TOL = 2e-5  # of the largest output magnitude


def run(backend, name, buffers, scalars):
    backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=buffers, scalars=scalars))


def near(y, r):
    return float(np.max(np.abs(y - r))) <= TOL * float(np.max(np.abs(r)))


def device_attention(backend, fmt, q, k, v, ks, vs, m, n, heads, kv_heads, head_dim, q_base, window, causal, row_base=0):
    width = heads * head_dim
    qfull = np.zeros((row_base + m, width), np.float32)
    qfull[row_base:] = q.reshape(m, width)
    out = backend.AllocateBuffer((row_base + m) * width * 4)
    if fmt < 2:
        run(backend, "attention", [backend.upload(qfull), backend.upload(k), backend.upload(v), out],
            [m, n, heads, kv_heads, head_dim, q_base, row_base, window, fmt, 1 if causal else 0])
    else:
        run(backend, QUANT_ID[fmt],
            [backend.upload(qfull), backend.upload(k), backend.upload(v), backend.upload(ks), backend.upload(vs), out],
            [m, n, heads, kv_heads, head_dim, q_base, row_base, window, QUANT_KIND[fmt]])
    return backend.download(out, np.float32, (row_base + m) * width).reshape(row_base + m, width)[row_base:]


def make_cache(g, fmt, n, row):
    """(k, v, k_scale, v_scale) of a seeded cache in the format."""
    ks = (0.004 + 0.01 * g.random(n)).astype(np.float32)
    vs = (0.004 + 0.01 * g.random(n)).astype(np.float32)

    def one():
        if fmt == 0:
            return g.standard_normal((n, row)).astype(np.float32)
        if fmt == 1:
            return g.standard_normal((n, row)).astype(np.float16).view(np.uint8)
        if fmt == 2:
            return g.integers(-127, 128, (n, row)).astype(np.int8).view(np.uint8)
        if fmt == 3:
            nib = g.integers(0, 16, (n, row)).astype(np.uint8)
            return (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
        b = g.integers(0, 256, (n, row)).astype(np.uint8)
        b[(b & 0x7F) == 0x7F] = 0x3C
        return b
    return one(), one(), ks, vs


def test_golden_cases_every_format(backend):
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    m, n, heads, kv_heads, head_dim = (int(x) for x in g["dims"])
    checked = 0
    for fmt, tag in enumerate(TAGS):
        for si, (q_base, window, causal) in enumerate(g["settings"]):
            key = f"out_{tag}_{si}"
            if key not in g:
                continue
            y = device_attention(backend, fmt, g["q"], g["k_" + tag], g["v_" + tag], g["k_scale"], g["v_scale"], m, n, heads,
                                 kv_heads, head_dim, int(q_base), int(window), bool(causal))
            assert near(y, g[key]), key
            checked += 1
    assert checked == 16


@pytest.mark.parametrize("fmt", [0, 1, 2, 3, 4])
def test_decode_row_over_a_long_cache(backend, oracle, fmt):
    """One query row, 24 heads over 4 kv heads of 256, 4096 keys: the key range is cut into 32 chunks."""
    g = np.random.default_rng(10 + fmt)
    n, heads, kv_heads, head_dim = 4096, 24, 4, 256
    q = g.standard_normal((1, heads * head_dim)).astype(np.float32)
    k, v, ks, vs = make_cache(g, fmt, n, kv_heads * head_dim)
    y = device_attention(backend, fmt, q, k, v, ks, vs, 1, n, heads, kv_heads, head_dim, n - 1, 0, True)
    r = oracle.attention(fmt, q, k, v, 1, n, heads, kv_heads, head_dim, n - 1, 0, True, ks, vs)
    assert near(y, r)


@pytest.mark.parametrize("fmt,window", [(0, 0), (1, 300), (4, 1000)])
def test_verify_rows_with_row_base_and_window(backend, oracle, fmt, window):
    """Five query rows at the end of a 1500-key cache, written at rows 2..6 of a shared batch buffer."""
    g = np.random.default_rng(20 + fmt)
    m, n, heads, kv_heads, head_dim = 5, 1500, 16, 2, 128
    q = g.standard_normal((m, heads * head_dim)).astype(np.float32)
    k, v, ks, vs = make_cache(g, fmt, n, kv_heads * head_dim)
    y = device_attention(backend, fmt, q, k, v, ks, vs, m, n, heads, kv_heads, head_dim, n - m, window, True, row_base=2)
    r = oracle.attention(fmt, q, k, v, m, n, heads, kv_heads, head_dim, n - m, window, True, ks, vs)
    assert near(y, r)


@pytest.mark.parametrize("fmt", [0, 1, 2, 4])
@pytest.mark.parametrize("q_base,split", [(2047, 16), (5, 16), (2047, 64)])
def test_split_and_combine_ids(backend, oracle, fmt, q_base, split):
    """The caller's chunk count and partial buffers (the reference's single-token path): partials in the reference's
    layout, empty chunks as the null partial (0, -1e30, 0), attention_combine merges them."""
    g = np.random.default_rng(30 + fmt)
    n, heads, kv_heads, head_dim = 2048, 8, 2, 256
    q = g.standard_normal((1, heads * head_dim)).astype(np.float32)
    k, v, ks, vs = make_cache(g, fmt, n, kv_heads * head_dim)
    parts = heads * split
    pacc, pmax, psum = (backend.AllocateBuffer(parts * c * 4) for c in (head_dim, 1, 1))
    out = backend.AllocateBuffer(heads * head_dim * 4)
    if fmt < 2:
        for name in ("attention_split", "attention_split_gqa"):
            run(backend, name, [backend.upload(q), backend.upload(k), backend.upload(v), pacc, pmax, psum],
                [1, n, heads, kv_heads, head_dim, q_base, 0, fmt, 1, split])
    else:
        run(backend, QUANT_ID[fmt] + "_split",
            [backend.upload(q), backend.upload(k), backend.upload(v), backend.upload(ks), backend.upload(vs), pacc, pmax, psum],
            [1, n, heads, kv_heads, head_dim, q_base, 0, QUANT_KIND[fmt], split])
    run(backend, "attention_combine", [pacc, pmax, psum, out], [1, heads, head_dim, split])
    y = backend.download(out, np.float32, heads * head_dim).reshape(1, -1)
    r = oracle.attention(fmt, q, k, v, 1, n, heads, kv_heads, head_dim, q_base, 0, True, ks, vs)
    assert near(y, r)
    mx = backend.download(pmax, np.float32, parts).reshape(heads, split)
    sm = backend.download(psum, np.float32, parts).reshape(heads, split)
    acc = backend.download(pacc, np.float32, parts * head_dim).reshape(heads, split, head_dim)
    span = q_base + 1
    chunk = (span + split - 1) // split
    for s in range(split):
        if s * chunk >= span:
            assert np.all(mx[:, s] == np.float32(-1e30)) and np.all(sm[:, s] == 0) and np.all(acc[:, s] == 0)
        else:
            assert np.all(mx[:, s] > -1e29) and np.all(sm[:, s] >= 1.0)  # the chunk's own max contributes exp(0)


def test_rejects_what_it_does_not_serve(backend):
    buf = backend.AllocateBuffer(1 << 20)
    cases = [
        ("attention", [buf] * 4, [1, 16, 4, 2, 64, 15, 0, 0, 0, 1], capi.StatusCode.UnsupportedFeature),      # head_dim 64
        ("attention", [buf] * 4, [1, 16, 32, 2, 128, 15, 0, 0, 0, 1], capi.StatusCode.UnsupportedFeature),    # 16 heads per kv head
        ("attention", [buf] * 4, [1, 16, 6, 4, 128, 15, 0, 0, 0, 1], capi.StatusCode.InvalidArgument),        # heads % kv_heads
        ("attention", [buf] * 4, [1, 4096, 8, 8, 256, 15, 0, 0, 0, 1], capi.StatusCode.InvalidArgument),      # cache beyond the buffer
        ("attention_q8", [buf] * 6, [1, 16, 4, 2, 128, 15, 0, 0, 2], capi.StatusCode.InvalidArgument),        # kind of another id
        ("attention_split", [buf] * 6, [1, 16, 4, 2, 128, 15, 0, 0, 1, 65], capi.StatusCode.InvalidArgument),  # more than 64 chunks
        ("attention_combine", [buf] * 4, [1, 4, 128, 0], capi.StatusCode.InvalidArgument),
    ]
    for name, buffers, scalars, code in cases:
        with pytest.raises(capi.StatusError) as e:
            run(backend, name, buffers, scalars)
        assert e.value.code == code, name
    backend.Synchronize()


def bits(x):
    return int(np.float32(x).view(np.uint32))


def test_rope_against_golden_and_oracle(backend, oracle):
    """The angle is formed in double precision on both sides; the device's double sine and cosine may differ from
    the host's in the last bit, which shows as one ulp of an fp32 factor."""
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    buf = backend.upload(g["rope_io"])
    run(backend, "rope", [buf], [3, 2, 64, 48, 1021, bits(1e6)])
    got = backend.download(buf, np.float32, g["rope_io"].size)
    assert np.all(np.abs(got - g["rope_out"]) <= 3e-7 * (np.abs(g["rope_out"]) + np.abs(g["rope_io"])))
    untouched = np.arange(got.size) % 64 >= 48
    assert np.array_equal(got[untouched], g["rope_io"][untouched])
    rng = np.random.default_rng(41)
    rows, heads, dim, rdim = 5, 24, 256, 64
    io = rng.standard_normal(rows * heads * dim).astype(np.float32)
    buf = backend.upload(io)
    run(backend, "rope", [buf], [rows, heads, dim, rdim, 100000, bits(1e7)])
    want = oracle.rope(io, rows, heads, dim, rdim, 100000, float(np.float32(1e7)))
    assert np.all(np.abs(backend.download(buf, np.float32, io.size) - want) <= 3e-7 * (np.abs(want) + np.abs(io)))


@pytest.mark.parametrize("kind,name", [(0, "quantize_q8"), (1, "quantize_q4")])
def test_cache_writers_are_bit_equal(backend, oracle, kind, name):
    """quantize_q8 / quantize_q4 (the int8 / 4-bit cache rows): golden cases with ties and a zero row, then
    a cache-sized row; the row maximum is exact in any order, so codes and scales are bit-equal."""
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    tag = "kvq8" if kind == 0 else "kvq4"
    rng = np.random.default_rng(43 + kind)
    big = (rng.standard_normal((7, 1024)) * 3).astype(np.float32)
    for x, want in ((g["kvq_in"], (g[tag + "_codes"], g[tag + "_scale"])), (big, oracle.quantize_rows(kind, big))):
        rows, cols = x.shape
        nbytes = rows * cols if kind == 0 else rows * cols // 2
        codes, scale = backend.AllocateBuffer(nbytes), backend.AllocateBuffer(rows * 4)
        run(backend, name, [backend.upload(x), codes, scale], [rows, cols])
        assert np.array_equal(backend.download(codes, np.uint8, nbytes).reshape(want[0].shape), want[0])
        assert np.array_equal(backend.download(scale, np.float32, rows), want[1])
    buf = backend.AllocateBuffer(4096)
    with pytest.raises(capi.StatusError):
        run(backend, name, [buf, buf, buf], [1, 1020 if kind == 1 else 1022])  # cols not a multiple of 8 / 4
    backend.Synchronize()


def test_written_cache_feeds_attention(backend, oracle):
    """quantize_q8 rows written by the device, read back by attention_q8: the pair the int8 cache path runs."""
    rng = np.random.default_rng(47)
    n, heads, kv_heads, head_dim = 300, 8, 2, 128
    row = kv_heads * head_dim
    kf, vf = (rng.standard_normal((n, row)).astype(np.float32) for _ in range(2))
    q = rng.standard_normal((1, heads * head_dim)).astype(np.float32)
    bufs = []
    for x in (kf, vf):
        codes, scale = backend.AllocateBuffer(n * row), backend.AllocateBuffer(n * 4)
        run(backend, "quantize_q8", [backend.upload(x), codes, scale], [n, row])
        bufs += [codes, scale]
    out = backend.AllocateBuffer(heads * head_dim * 4)
    run(backend, "attention_q8", [backend.upload(q), bufs[0], bufs[2], bufs[1], bufs[3], out],
        [1, n, heads, kv_heads, head_dim, n - 1, 0, 0, 0])
    (kc, ks), (vc, vs) = oracle.quantize_rows(0, kf), oracle.quantize_rows(0, vf)
    want = oracle.attention(2, q, kc, vc, 1, n, heads, kv_heads, head_dim, n - 1, 0, True, ks, vs)
    assert near(backend.download(out, np.float32, heads * head_dim).reshape(1, -1), want)
