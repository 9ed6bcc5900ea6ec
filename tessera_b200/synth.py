"""Seeded synthetic inputs in the reference's on-device layouts.

The reference is measured on private model checkpoints; these generators
produce tensors with the same layouts, sizes and value distributions (numpy
PCG64, one generator per tensor).  Layout facts:

* Q4_K: 144-byte super-blocks of 256 values: fp16 d and dmin, twelve bytes of
  packed 6-bit (scale, min) pairs, 128 nibble bytes
  (src/core/numerics/quant.cpp:58-70,656-675 of the reference).
* Q6_K: 210 bytes: ql[128], qh[64], int8 scales[16], fp16 d (quant.cpp:421-449).
* MXFP4: n*k/2 nibble bytes (low nibble = even element) followed by n*k/32
  E8M0 scale bytes (include/tessera/backend.hpp:195-201).
* FP8: n*k E4M3 bytes plus one fp32 scale per row (backend.hpp:190-194).
"""
from __future__ import annotations

import numpy as np


def rng(seed: int, index: int = 0) -> np.random.Generator:
    return np.random.default_rng(seed * 1000 + index)


def pack_q4k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """(…, 8) 6-bit scales and mins -> (…, 12) bytes, inverse of GetScaleMin."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return out


def q4k_weights(n: int, k: int, seed: int = 0, index: int = 0) -> np.ndarray:
    """n rows of k/256 Q4_K blocks: d, dmin ~ U[1e-3, 4e-3] (fp16), scales and
    mins ~ U{0..63}, nibbles ~ U{0..15}.  Returns uint8 of n*(k/256)*144 bytes."""
    assert k % 256 == 0
    g = rng(seed, index)
    nb = n * (k // 256)
    blocks = np.empty((nb, 144), dtype=np.uint8)
    d = g.uniform(1e-3, 4e-3, size=nb).astype(np.float16)
    dmin = g.uniform(1e-3, 4e-3, size=nb).astype(np.float16)
    blocks[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    blocks[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    sc = g.integers(0, 64, size=(nb, 8), dtype=np.uint8)
    mn = g.integers(0, 64, size=(nb, 8), dtype=np.uint8)
    blocks[:, 4:16] = pack_q4k_scales(sc, mn)
    blocks[:, 16:144] = g.integers(0, 256, size=(nb, 128), dtype=np.uint8)
    return blocks.reshape(-1)


def q6k_weights(n: int, k: int, seed: int = 0, index: int = 0) -> np.ndarray:
    """n rows of k/256 Q6_K blocks: d ~ U[1e-4, 4e-4] (fp16), int8 scales ~
    U{-64..63}, 6-bit quants uniform."""
    assert k % 256 == 0
    g = rng(seed, index)
    nb = n * (k // 256)
    blocks = np.empty((nb, 210), dtype=np.uint8)
    blocks[:, 0:192] = g.integers(0, 256, size=(nb, 192), dtype=np.uint8)
    blocks[:, 192:208] = g.integers(-64, 64, size=(nb, 16), dtype=np.int8).view(np.uint8)
    d = g.uniform(1e-4, 4e-4, size=nb).astype(np.float16)
    blocks[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    return blocks.reshape(-1)


def mxfp4_weights(n: int, k: int, seed: int = 0, index: int = 0, exp_lo: int = -8, exp_hi: int = 0) -> np.ndarray:
    """Packed MXFP4: E2M1 codes uniform over all 16 values, one E8M0 byte per
    32 elements with exponent uniform in [exp_lo, exp_hi]."""
    assert k % 32 == 0
    g = rng(seed, index)
    blob = g.integers(0, 256, size=n * k // 2, dtype=np.uint8)
    scales = (127 + g.integers(exp_lo, exp_hi + 1, size=n * k // 32)).astype(np.uint8)
    return np.concatenate([blob, scales])


E4M3_MAX = 448.0


def e4m3_decode_table() -> np.ndarray:
    """fp32 value of each E4M3 byte (OCP: bias 7, 0x7F/0xFF NaN)."""
    b = np.arange(256, dtype=np.uint32)
    e = (b >> 3) & 15
    m = (b & 7).astype(np.float32)
    val = np.where(e == 0, m * np.float32(2.0 ** -9),
                   (1.0 + m / 8.0) * np.exp2(e.astype(np.float32) - 7.0)).astype(np.float32)
    val = np.where((b & 0x7F) == 0x7F, np.nan, val).astype(np.float32)
    return np.where(b & 0x80, -val, val).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even E4M3 codes of finite fp32 values in [-448, 448],
    with the reference's subnormal rule (mantissa clamped at 7)."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x)
    fr, ex = np.frexp(mag)
    field = ex.astype(np.int64) + 6
    sub = field < 1
    man_sub = np.minimum(np.rint(mag * np.float32(512.0)), 7).astype(np.int64)
    man = np.rint((fr * np.float32(2.0) - np.float32(1.0)) * np.float32(8.0)).astype(np.int64)
    carry = man == 8
    man = np.where(carry, 0, man)
    field = np.where(carry, field + 1, field)
    field = np.minimum(field, 15)
    man = np.where((field == 15) & (man > 6), 6, man)
    code = np.where(sub, man_sub, (field << 3) | man)
    code = np.where(mag == 0, 0, code)
    code = np.where(mag > E4M3_MAX, 0x7F, code)
    return (code | np.where(np.signbit(x), 0x80, 0)).astype(np.uint8)


def fp8_weights(n: int, k: int, seed: int = 0, index: int = 0, std: float = 0.02):
    """w ~ N(0, std) quantised per output row: s = amax/448 (fp32), codes =
    E4M3(w / s).  Returns (codes uint8 n*k, scales float32 n)."""
    g = rng(seed, index)
    w = (g.standard_normal((n, k), dtype=np.float32) * np.float32(std)).astype(np.float32)
    amax = np.abs(w).max(axis=1)
    s = (amax / np.float32(E4M3_MAX)).astype(np.float32)
    s = np.where(s > 0, s, np.float32(1.0)).astype(np.float32)
    q = np.clip(w / s[:, None], -E4M3_MAX, E4M3_MAX).astype(np.float32)
    return e4m3_encode(q).reshape(-1), s


def activations(m: int, k: int, seed: int = 0, index: int = 99, bf16: bool = False) -> np.ndarray:
    """fp32 N(0,1); with bf16=True the values are rounded to bfloat16 (kept
    in fp32 storage), the activation type the measurement configs name."""
    a = rng(seed, index).standard_normal((m, k), dtype=np.float32)
    if bf16:
        u = a.view(np.uint32)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & np.uint32(0xFFFF0000)
        a = u.view(np.float32)
    return np.ascontiguousarray(a)


def slice_rows_by_block(w: np.ndarray, n: int, k: int, block_bytes: int, rank: int, world: int,
                        unit: int = 256) -> np.ndarray:
    """Row-parallel (K) shard of a block-quantised matrix at block boundaries,
    repacked contiguous, as the reference's SliceTensor2D does
    (src/core/loaders/tensor_slice.cpp:130-158)."""
    nb = k // unit
    assert nb % world == 0, "K shard must fall on block boundaries"
    per = nb // world
    rows = w.reshape(n, nb, block_bytes)
    return np.ascontiguousarray(rows[:, rank * per:(rank + 1) * per, :]).reshape(-1)


def slice_mxfp4_cols(w: np.ndarray, n: int, k: int, rank: int, world: int) -> np.ndarray:
    """Row-parallel shard of a packed MXFP4 matrix: nibble blob and scales are
    sliced together (tensor_slice.cpp:79-100)."""
    assert (k // 32) % world == 0
    kp = k // world
    blob = w[: n * k // 2].reshape(n, k // 2)[:, rank * kp // 2:(rank + 1) * kp // 2]
    sc = w[n * k // 2:].reshape(n, k // 32)[:, rank * kp // 32:(rank + 1) * kp // 32]
    return np.concatenate([np.ascontiguousarray(blob).reshape(-1), np.ascontiguousarray(sc).reshape(-1)])
