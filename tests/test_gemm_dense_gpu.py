"""Projections over unquantised weights (ids gemm_f32*, gemm_bf16*) on the GPU against the CPU oracle, which
is bit-equal to the reference's GemmF32Ref / GemmBf16Ref (tests/test_oracle_golden.py).  Same products; the
device adds them lane by lane and then as a tree, so sums agree to fp32 rounding."""
import os

import numpy as np
import pytest

from tessera_b200 import capi
from tessera_b200.backend import KernelLaunch

pytestmark = pytest.mark.gpu

TOL = 1e-5  # of the largest output magnitude


def run(backend, name, buffers, scalars):
    backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=buffers, scalars=scalars))


def project(backend, name, a, w, m, n, k):
    c = backend.AllocateBuffer(m * n * 4)
    run(backend, name, [backend.upload(a), backend.upload(w), c], [m, n, k])
    return backend.download(c, np.float32, m * n).reshape(m, n)


def near(y, r):
    return float(np.max(np.abs(y - r))) <= TOL * float(np.max(np.abs(r)))


def bf16_bits(x):
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def test_golden_cases(backend):
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz"))
    assert near(project(backend, "gemm_f32", g["dense_a"], g["dense_w32"], 3, 9, 75), g["dense_c32"])
    assert near(project(backend, "gemm_bf16", g["dense_a"], g["dense_w16"], 3, 9, 75), g["dense_c16"])


@pytest.mark.parametrize("name,bf16", [("gemm_f32", False), ("gemm_f32_batched", False), ("gemm_bf16", True),
                                       ("gemm_bf16_batched", True), ("gemm_bf16_wmma", True), ("gemm_bf16_rows", True)])
@pytest.mark.parametrize("m,n,k", [(1, 256, 2048), (5, 1003, 5120), (19, 64, 520), (1, 4099, 1024), (5, 4099, 1024), (2, 2049, 264),
                                   (11, 2051, 75)])
def test_against_the_oracle(backend, oracle, name, bf16, m, n, k):
    """A router gate (256 experts over hidden 2048), a ragged verify batch, more rows than one pass serves; then
    many weight rows: one activation row, batches (four weight rows per warp, ragged at the end), odd k."""
    g = np.random.default_rng(m * 1000 + n)
    a = g.standard_normal((m, k)).astype(np.float32)
    w = g.standard_normal((n, k)).astype(np.float32)
    if bf16:
        w = bf16_bits(w)
    assert near(project(backend, name, a, w, m, n, k), oracle.gemm_dense(bf16, a, w, m, n, k))


def test_contract_errors(backend):
    buf = backend.AllocateBuffer(4096)
    for scalars in ([1, 64, 32, 1], [0, 64, 16], [1, 64, 32]):  # a fourth scalar; m = 0; W (8 KB) beyond the buffer
        with pytest.raises(capi.StatusError):
            run(backend, "gemm_f32", [buf, buf, buf], scalars)
    backend.Synchronize()
