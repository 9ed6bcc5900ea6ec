"""ctypes front-end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

``Oracle()`` loads ``oracle/liboracle.so`` (the plain-C restatement);
``Oracle(reference=True)`` loads ``oracle/_ref/libtessera_ref.so`` (the
reference's own host functions) when it was built.  Both expose the same
numpy-level calls, so either can check a CUDA result or be timed as the CPU
baseline.  Only tests, the smoke check and the benchmark's CPU-baseline leg
import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libtessera_ref.so")

_sz = C.c_size_t
_p = C.c_void_p


def build(reference_root: str | None = None) -> None:
    """Runs the Makefile beside this file; `reference_root` overrides its default
    location of the reference checkout."""
    cmd = ["make", "-C", _HERE] + ([f"REFERENCE={reference_root}"] if reference_root else [])
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def reference_available() -> bool:
    return os.path.exists(REF_SO)


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_p)


class Oracle:
    def __init__(self, reference: bool = False):
        self.reference = reference
        path = REF_SO if reference else ORACLE_SO
        if not os.path.exists(path):
            if reference:
                raise FileNotFoundError(path)
            build()
        self.lib = C.CDLL(path)
        self.pre = "ref_" if reference else "orc_"

    def _fn(self, name, restype, argtypes):
        fn = getattr(self.lib, self.pre + name)
        fn.restype, fn.argtypes = restype, argtypes
        return fn

    def slice_tensor2d(self, dtype: int, rows: int, cols: int, kind: int, rank: int, world: int, src: np.ndarray):
        """The reference's SliceTensor2D (reference build only).  dtype is the reference's DType
        value (F4E2M1 6, Q4K 10, Q6K 12, F8E4M3 3).  Returns (bytes, rows, cols) or the negative
        status code the reference answered with."""
        assert self.reference
        fn = self.lib.ref_slice_tensor2d
        fn.restype = C.c_longlong
        fn.argtypes = [C.c_int, _sz, _sz, C.c_int, C.c_int, C.c_int, _p, _sz, _p, _sz, C.POINTER(_sz), C.POINTER(_sz)]
        src = np.ascontiguousarray(src.reshape(-1).view(np.uint8))
        dst = np.empty(src.nbytes, dtype=np.uint8)
        r, c = _sz(), _sz()
        n = fn(dtype, rows, cols, kind, rank, world, _ptr(src), src.nbytes, _ptr(dst), dst.nbytes, C.byref(r), C.byref(c))
        if n < 0:
            return int(n)
        return dst[:n].copy(), r.value, c.value

    # ---- scalar codecs (vectorised by looping in Python: small inputs only)
    def _map(self, name, restype, argtype, values, out_dtype):
        fn = self._fn(name, restype, [argtype])
        return np.array([fn(v) for v in values], dtype=out_dtype)

    def fp16_to_float(self, h):
        return self._map("fp16_to_float", C.c_float, C.c_uint16, [int(x) for x in h], np.float32)

    def fp8e4m3_to_float(self, b):
        return self._map("fp8e4m3_to_float", C.c_float, C.c_uint8, [int(x) for x in b], np.float32)

    def e8m0_to_float(self, b):
        return self._map("e8m0_to_float", C.c_float, C.c_uint8, [int(x) for x in b], np.float32)

    def f4e2m1_to_float(self, b):
        return self._map("f4e2m1_to_float", C.c_float, C.c_uint8, [int(x) for x in b], np.float32)

    def fp32_to_fp8e4m3(self, v):
        return self._map("fp32_to_fp8e4m3", C.c_uint8, C.c_float, [float(x) for x in v], np.uint8)

    def fp32_to_f4e2m1(self, v):
        return self._map("fp32_to_f4e2m1", C.c_uint8, C.c_float, [float(x) for x in v], np.uint8)

    # ---- blocks
    def dequant_blocks(self, fmt: int, w: np.ndarray) -> np.ndarray:
        bb = 144 if fmt == 0 else 210
        nb = w.size // bb
        out = np.empty(nb * 256, dtype=np.float32)
        fn = self._fn("dequant_blocks", C.c_int, [C.c_int, _p, _sz, _p])
        assert fn(fmt, _ptr(w), nb, _ptr(out)) == 0
        return out

    # ---- GEMMs
    def _gemm3(self, name, a, w, m, n, k, threads=0):
        c = np.empty((m, n), dtype=np.float32)
        if threads and not self.reference:
            fn = self._fn(name + "_mt", C.c_int, [_p, _p, _p, _sz, _sz, _sz, C.c_int])
            rc = fn(_ptr(a), _ptr(w), _ptr(c), m, n, k, threads)
        else:
            fn = self._fn(name, C.c_int, [_p, _p, _p, _sz, _sz, _sz])
            rc = fn(_ptr(a), _ptr(w), _ptr(c), m, n, k)
        assert rc == 0, rc
        return c

    def gemm_q4k(self, a, w, m, n, k, threads=0):
        return self._gemm3("gemm_q4k", a, w, m, n, k, threads)

    def gemm_q6k(self, a, w, m, n, k, threads=0):
        return self._gemm3("gemm_q6k", a, w, m, n, k, threads)

    def gemm_mxfp4(self, a, w_packed, m, n, k, threads=0):
        """w_packed is the device layout blob||scales."""
        blob = np.ascontiguousarray(w_packed[: n * k // 2])
        sc = np.ascontiguousarray(w_packed[n * k // 2:])
        c = np.empty((m, n), dtype=np.float32)
        if threads and not self.reference:
            fn = self._fn("gemm_mxfp4_mt", C.c_int, [_p, _p, _p, _p, _sz, _sz, _sz, C.c_int])
            rc = fn(_ptr(a), _ptr(blob), _ptr(sc), _ptr(c), m, n, k, threads)
        else:
            fn = self._fn("gemm_mxfp4", C.c_int, [_p, _p, _p, _p, _sz, _sz, _sz])
            rc = fn(_ptr(a), _ptr(blob), _ptr(sc), _ptr(c), m, n, k)
        assert rc == 0, rc
        return c

    def gemm_fp8(self, a, w, s, m, n, k, threads=0):
        c = np.empty((m, n), dtype=np.float32)
        if threads and not self.reference:
            fn = self._fn("gemm_fp8_mt", C.c_int, [_p, _p, _p, _p, _sz, _sz, _sz, C.c_int])
            rc = fn(_ptr(a), _ptr(w), _ptr(s), _ptr(c), m, n, k, threads)
        else:
            fn = self._fn("gemm_fp8", C.c_int, [_p, _p, _p, _p, _sz, _sz, _sz])
            rc = fn(_ptr(a), _ptr(w), _ptr(s), _ptr(c), m, n, k)
        assert rc == 0, rc
        return c

    # ---- activation quantisation
    def quantize_fp8(self, data: np.ndarray):
        rows, cols = data.shape
        out = np.ascontiguousarray(data, dtype=np.float32).copy()
        scale = np.empty(rows, dtype=np.float32)
        fn = self._fn("quantize_fp8", C.c_int, [_p, _p, _sz, _sz])
        assert fn(_ptr(out), _ptr(scale), rows, cols) == 0
        return out, scale

    def quantize_fp8_pack(self, data: np.ndarray):
        rows, cols = data.shape
        codes = np.empty((rows, cols), dtype=np.uint8)
        scale = np.empty(rows, dtype=np.float32)
        fn = self._fn("quantize_fp8_pack", C.c_int, [_p, _p, _p, _sz, _sz])
        assert fn(_ptr(np.ascontiguousarray(data, dtype=np.float32)), _ptr(codes), _ptr(scale), rows, cols) == 0
        return codes, scale

    def rmsnorm(self, x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
        rows, cols = x.shape
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        y = np.empty_like(x)
        fn = self._fn("rmsnorm", C.c_int, [_p, _p, _p, _sz, _sz, C.c_float])
        assert fn(_ptr(x), _ptr(w), _ptr(y), rows, cols, eps) == 0
        return y

    def add(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        o = np.empty_like(a)
        fn = self._fn("add", C.c_int, [_p, _p, _p, _sz])
        assert fn(_ptr(a), _ptr(b), _ptr(o), a.size) == 0
        return o

    def silu_mul(self, g: np.ndarray, u: np.ndarray) -> np.ndarray:
        g = np.ascontiguousarray(g, dtype=np.float32)
        u = np.ascontiguousarray(u, dtype=np.float32)
        o = np.empty_like(g)
        fn = self._fn("silu_mul", C.c_int, [_p, _p, _p, _sz])
        assert fn(_ptr(g), _ptr(u), _ptr(o), g.size) == 0
        return o

    # ---- steps between the projections (both builds)
    def sigmoid_gate(self, a, g):
        a, g = (np.ascontiguousarray(v, dtype=np.float32) for v in (a, g))
        o = np.empty_like(a)
        assert self._fn("sigmoid_gate", C.c_int, [_p, _p, _p, _sz])(_ptr(a), _ptr(g), _ptr(o), a.size) == 0
        return o

    def l2norm(self, x, eps, scale):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        fn = self._fn("l2norm", C.c_int, [_p, _p, _sz, _sz, C.c_float, C.c_float])
        assert fn(_ptr(x), _ptr(y), x.shape[0], x.shape[1], eps, scale) == 0
        return y

    def rmsnorm_gated(self, x, w, gate, eps):
        x, w, gate = (np.ascontiguousarray(v, dtype=np.float32) for v in (x, w, gate))
        y = np.empty_like(x)
        fn = self._fn("rmsnorm_gated", C.c_int, [_p, _p, _p, _p, _sz, _sz, C.c_float])
        assert fn(_ptr(x), _ptr(w), _ptr(gate), _ptr(y), x.shape[0], x.shape[1], eps) == 0
        return y

    def ssm_gate(self, a_log, dt, alpha_raw, beta_raw):
        a_log, dt, alpha_raw, beta_raw = (np.ascontiguousarray(v, dtype=np.float32) for v in (a_log, dt, alpha_raw, beta_raw))
        alpha, beta = np.empty_like(alpha_raw), np.empty_like(beta_raw)
        fn = self._fn("ssm_gate", C.c_int, [_p, _p, _p, _p, _p, _p, _sz, _sz])
        assert fn(_ptr(a_log), _ptr(dt), _ptr(alpha_raw), _ptr(beta_raw), _ptr(alpha), _ptr(beta), a_log.size,
                  alpha_raw.shape[0]) == 0
        return alpha, beta

    def qgate_split(self, fused, heads, head_dim, rows):
        fused = np.ascontiguousarray(fused, dtype=np.float32)
        q = np.empty(rows * heads * head_dim, dtype=np.float32)
        gate = np.empty_like(q)
        fn = self._fn("qgate_split", C.c_int, [_p, _p, _p, _sz, _sz, _sz])
        assert fn(_ptr(fused), _ptr(q), _ptr(gate), heads, head_dim, rows) == 0
        return q, gate

    def repeat_heads(self, x, num_v_heads, head_k_dim, factor):
        """One row (the reference's function takes one; the built-in repeats it per row)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(num_v_heads * head_k_dim, dtype=np.float32)
        fn = self._fn("repeat_heads", C.c_int, [_p, _p, _sz, _sz, _sz])
        assert fn(_ptr(x), _ptr(out), num_v_heads, head_k_dim, factor) == 0
        return out

    def mrope(self, io, pos, rows, heads, head_dim, rope_dim, sec_t, sec_h, sec_w, theta):
        io = np.ascontiguousarray(io, dtype=np.float32).copy()
        pos = np.ascontiguousarray(pos, dtype=np.uint64)
        fn = self._fn("mrope", C.c_int, [_p, _p, _sz, _sz, _sz, _sz, _sz, _sz, _sz, C.c_double])
        assert fn(_ptr(io), _ptr(pos), rows, heads, head_dim, rope_dim, sec_t, sec_h, sec_w, theta) == 0
        return io

    def gemm_dense(self, bf16, a, w, m, n, k):
        """w: fp32 (n x k) or bf16 bit patterns as uint16 (n x k)."""
        a = np.ascontiguousarray(a, dtype=np.float32)
        w = np.ascontiguousarray(w)
        c = np.empty((m, n), dtype=np.float32)
        fn = self._fn("gemm_dense", C.c_int, [C.c_int, _p, _p, _p, _sz, _sz, _sz])
        assert fn(1 if bf16 else 0, _ptr(a), _ptr(w), _ptr(c), m, n, k) == 0
        return c

    def rope(self, io, rows, heads, head_dim, rope_dim, pos_base, theta):
        io = np.ascontiguousarray(io, dtype=np.float32).copy()
        fn = self._fn("rope", C.c_int, [_p, _sz, _sz, _sz, _sz, C.c_uint64, C.c_double])
        assert fn(_ptr(io), rows, heads, head_dim, rope_dim, pos_base, theta) == 0
        return io

    def quantize_rows(self, kind, data):
        """kind 0: int8 codes (rows x cols bytes); 1: 4-bit codes (rows x cols / 2 bytes).  Returns (codes, scale)."""
        rows, cols = data.shape
        codes = np.zeros((rows, cols if kind == 0 else cols // 2), dtype=np.uint8)
        scale = np.empty(rows, dtype=np.float32)
        fn = self._fn("quantize_rows", C.c_int, [C.c_int, _p, _p, _p, _sz, _sz])
        assert fn(kind, _ptr(np.ascontiguousarray(data, dtype=np.float32)), _ptr(codes), _ptr(scale), rows, cols) == 0
        return codes, scale

    def delta_step_heads(self, s, k, v, q, alpha, beta, heads, dk, dv):
        """One step; returns (new state, o)."""
        s = np.ascontiguousarray(s, dtype=np.float32).copy()
        k, v, q, alpha, beta = (np.ascontiguousarray(x, dtype=np.float32) for x in (k, v, q, alpha, beta))
        o = np.empty(heads * dv, dtype=np.float32)
        fn = self._fn("delta_step_heads", C.c_int, [_p, _p, _p, _p, _p, _p, _p, _sz, _sz, _sz])
        assert fn(_ptr(s), _ptr(k), _ptr(v), _ptr(q), _ptr(o), _ptr(alpha), _ptr(beta), heads, dk, dv) == 0
        return s, o

    def conv1d_step(self, x, w, channels, width):
        x, w = (np.ascontiguousarray(t, dtype=np.float32) for t in (x, w))
        y = np.empty(channels, dtype=np.float32)
        assert self._fn("conv1d_step", C.c_int, [_p, _p, _p, _sz, _sz])(_ptr(x), _ptr(w), _ptr(y), channels, width) == 0
        return y

    def attention(self, kv_format, q, k, v, m, n, heads, kv_heads, head_dim, q_base=0, window=0, causal=True,
                  k_scale=None, v_scale=None):
        """kv_format 0 fp32, 1 fp16, 2 int8, 3 4-bit, 4 FP8 (k, v: arrays of the cache's bytes or floats)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
        ks = np.zeros(1, np.float32) if k_scale is None else np.ascontiguousarray(k_scale, dtype=np.float32)
        vs = np.zeros(1, np.float32) if v_scale is None else np.ascontiguousarray(v_scale, dtype=np.float32)
        out = np.empty(m * heads * head_dim, dtype=np.float32)
        fn = self._fn("attention", C.c_int, [C.c_int, _p, _p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, C.c_uint64, _sz, C.c_int])
        assert fn(kv_format, _ptr(q), _ptr(k), _ptr(v), _ptr(ks), _ptr(vs), _ptr(out), m, n, heads, kv_heads, head_dim,
                  q_base, window, 1 if causal else 0) == 0
        return out.reshape(m, heads * head_dim)

    def conv1d_state(self, qkv, w, hist, conv_dim, width, key_dim, qkv_offset, rows, hist_stride=0, hist_hist=None):
        """Device contract (C restatement only).  Returns (q, k, v, hist, hist_hist)."""
        assert not self.reference
        qkv, w = (np.ascontiguousarray(t, dtype=np.float32) for t in (qkv, w))
        hist = np.ascontiguousarray(hist, dtype=np.float32).copy()
        hh = np.zeros(1, dtype=np.float32) if hist_hist is None else np.ascontiguousarray(hist_hist, dtype=np.float32).copy()
        q = np.empty(rows * key_dim, dtype=np.float32)
        k = np.empty(rows * key_dim, dtype=np.float32)
        v = np.empty(rows * (conv_dim - 2 * key_dim), dtype=np.float32)
        fn = self._fn("conv1d_state", C.c_int, [_p, _p, _p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz])
        assert fn(_ptr(qkv), _ptr(w), _ptr(hist), _ptr(q), _ptr(k), _ptr(v), _ptr(hh), conv_dim, width, key_dim, qkv_offset,
                  rows, hist_stride) == 0
        return q, k, v, hist, hh

    def top_k_rows(self, logits, rows, vocab, top_k, row_base=0):
        assert not self.reference
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        ids = np.zeros(rows * top_k, dtype=np.uint32)
        vals = np.zeros(rows * top_k, dtype=np.float32)
        fn = self._fn("top_k_rows", C.c_int, [_p, _p, _p, _sz, _sz, _sz, _sz])
        assert fn(_ptr(logits), _ptr(ids), _ptr(vals), rows, vocab, top_k, row_base) == 0
        return ids.reshape(rows, top_k), vals.reshape(rows, top_k)

    # ---- routed experts (device-only contracts; C restatement only)
    def moe_gate(self, vals, x, w):
        assert not self.reference
        vals, x, w = (np.ascontiguousarray(v, dtype=np.float32) for v in (vals, x, w))
        wts, sig = np.empty(vals.size, dtype=np.float32), np.empty(1, dtype=np.float32)
        fn = self._fn("moe_gate", C.c_int, [_p, _p, _p, _p, _p, _sz, _sz])
        assert fn(_ptr(vals), _ptr(x), _ptr(w), _ptr(wts), _ptr(sig), vals.size, x.size) == 0
        return wts, sig

    def moe_scale_add(self, a, b, f, idx):
        assert not self.reference
        a, b, f = (np.ascontiguousarray(v, dtype=np.float32) for v in (a, b, f))
        o = np.empty_like(a)
        fn = self._fn("moe_scale_add", C.c_int, [_p, _p, _p, _p, _sz, _sz])
        assert fn(_ptr(a), _ptr(b), _ptr(f), _ptr(o), a.size, idx) == 0
        return o

    def moe_experts_gate_up_q4k(self, x, gate, up, ids, hidden, inter, gate_stride, up_stride):
        assert not self.reference
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        phi = np.empty((ids.size, inter), dtype=np.float32)
        fn = self._fn("moe_experts_gate_up_q4k", C.c_int, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz])
        assert fn(_ptr(x), _ptr(gate), _ptr(up), _ptr(ids), _ptr(phi), hidden, inter, ids.size, gate_stride, up_stride) == 0
        return phi

    def moe_experts_down(self, fmt, phi, down, ids, wts, hidden, inter, down_stride, out=None):
        assert not self.reference
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        wts = np.ascontiguousarray(wts, dtype=np.float32)
        acc = out is not None
        res = np.ascontiguousarray(out, dtype=np.float32).copy() if acc else np.empty(hidden, dtype=np.float32)
        fn = self._fn("moe_experts_down", C.c_int, [C.c_int, _p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, C.c_int])
        assert fn(fmt, _ptr(phi), _ptr(down), _ptr(ids), _ptr(wts), _ptr(res), hidden, inter, ids.size, down_stride, int(acc)) == 0
        return res

    def moe_experts_forward(self, x, experts, wts, gate, gate_per, up, up_per, down_dtype, down, down_per, hidden, inter, acc):
        """The reference's CpuMoeExpertsForward (reference build only): acc + sum_c wts[c] * expert_c(x).
        Gate and up are Q4_K; down_dtype is the reference's DType value (Q4K 10, Q6K 12)."""
        assert self.reference
        experts = np.ascontiguousarray(experts, dtype=np.uint32)
        wts = np.ascontiguousarray(wts, dtype=np.float32)
        out = np.ascontiguousarray(acc, dtype=np.float32).copy()
        fn = self.lib.ref_moe_experts_forward
        fn.restype = C.c_int
        fn.argtypes = [_p, _p, _p, _sz, C.c_int, _p, _sz, _sz, C.c_int, _p, _sz, _sz, C.c_int, _p, _sz, _sz, _sz, _sz, _p]
        rc = fn(_ptr(x), _ptr(experts), _ptr(wts), experts.size, 10, _ptr(gate), gate.nbytes, gate_per, 10, _ptr(up), up.nbytes,
                up_per, down_dtype, _ptr(down), down.nbytes, down_per, hidden, inter, _ptr(out))
        assert rc == 0, rc
        return out

    def round_bf16(self, x: np.ndarray) -> np.ndarray:
        out = np.ascontiguousarray(x, dtype=np.float32).copy()
        fn = self._fn("round_bf16", C.c_int, [_p, _sz])
        assert fn(_ptr(out), out.size) == 0
        return out

    # ---- W4A8
    def fold_mxfp4_to_fp8(self, w_packed, rows, cols):
        blob = np.ascontiguousarray(w_packed[: rows * cols // 2])
        sc = np.ascontiguousarray(w_packed[rows * cols // 2:])
        out = np.empty((rows, cols), dtype=np.uint8)
        wref = np.empty(rows, dtype=np.uint8)
        fn = self._fn("fold_mxfp4_to_fp8", C.c_int, [_p, _p, _p, _p, _sz, _sz])
        assert fn(_ptr(blob), _ptr(sc), _ptr(out), _ptr(wref), rows, cols) == 0
        return out, wref

    def gemm_mxfp4_fp8(self, a8, as_, w8, wref, m, n, k):
        c = np.empty((m, n), dtype=np.float32)
        fn = self._fn("gemm_mxfp4_fp8", C.c_int, [_p, _p, _p, _p, _p, _sz, _sz, _sz])
        assert fn(_ptr(a8), _ptr(as_), _ptr(w8), _ptr(wref), _ptr(c), m, n, k) == 0
        return c

    # ---- restatement-only entry points (device contracts with no host ref)
    def gemm_vec_split(self, fmt, a, w, m, n, k, split):
        assert not self.reference
        part = np.empty((split, m, n), dtype=np.float32)
        fn = self._fn("gemm_vec_split", C.c_int, [C.c_int, _p, _p, _p, _sz, _sz, _sz, _sz])
        assert fn(fmt, _ptr(a), _ptr(w), _ptr(part), m, n, k, split) == 0
        return part

    def gemm_vec_reduce(self, part):
        assert not self.reference
        split = part.shape[0]
        total = part.size // split
        c = np.empty(total, dtype=np.float32)
        fn = self._fn("gemm_vec_reduce", C.c_int, [_p, _p, _sz, _sz])
        assert fn(_ptr(part), _ptr(c), total, split) == 0
        return c

    def gemm_vec_split_rule(self, outputs, k, target=2048):
        fn = self._fn("gemm_vec_split_rule", _sz, [_sz, _sz, _sz])
        return fn(outputs, k, target)

    def mxfp4_row_ref(self, w_packed, rows, cols):
        assert not self.reference
        sc = np.ascontiguousarray(w_packed[rows * cols // 2:])
        wref = np.empty(rows, dtype=np.uint8)
        fn = self._fn("mxfp4_row_ref", C.c_int, [_p, _p, _sz, _sz])
        assert fn(_ptr(sc), _ptr(wref), rows, cols) == 0
        return wref

    def gemm_mxfp4_wmma(self, a8, w_packed, as_, wref, m, n, k, split):
        assert not self.reference
        c = np.empty((split, m, n), dtype=np.float32)
        fn = self._fn("gemm_mxfp4_wmma", C.c_int, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _sz])
        assert fn(_ptr(a8), _ptr(w_packed), _ptr(as_), _ptr(wref), _ptr(c), m, n, k, split) == 0
        return c

    def tp_reduce(self, partials):
        assert not self.reference
        world = len(partials)
        count = partials[0].size
        arr = (C.c_void_p * world)(*[p.ctypes.data for p in partials])
        out = np.empty(count, dtype=np.float32)
        fn = self._fn("tp_reduce", C.c_int, [_p, _sz, _sz, _p])
        assert fn(arr, world, count, _ptr(out)) == 0
        return out.reshape(partials[0].shape)
