"""The allocation-free split-K Q4_K projection against the ordinary entry point.

Some callers of the library cannot allocate device memory while they run (all
of it was handed out at load time, or a cudaMalloc would stall their decode
loop), so `tsr_gemm_q4k_noalloc` keeps its split-K partial sums in a fixed
array inside the library.  This file is collected last on purpose: a run that
stops at the first failure has then already been through every other test.
"""
import numpy as np
import pytest

from tessera_b200 import capi, synth

from conftest import rel_err


@pytest.mark.gpu
def test_noalloc_projection_matches_the_ordinary_one_twice(backend, oracle):
    lib = capi.load_library()
    st = backend.stream()
    for call, (m, n, k) in enumerate([(1, 520, 2048), (3, 96, 1024)]):
        a = synth.activations(m, k, seed=90 + call)
        w = synth.q4k_weights(n, k, seed=91 + call)
        ab, wb = backend.upload(a), backend.upload(w)
        want = backend.AllocateBuffer(m * n * 4)
        got = backend.AllocateBuffer(m * n * 4)
        assert lib.tsr_gemm_q4k(ab.Handle(), wb.Handle(), want.Handle(), m, n, k, 1, st) == 0
        assert lib.tsr_gemm_q4k_noalloc(ab.Handle(), wb.Handle(), got.Handle(), m, n, k, st) == 0
        y = backend.download(got, np.float32, m * n).reshape(m, n)
        r = backend.download(want, np.float32, m * n).reshape(m, n)
        assert rel_err(y, r) < 1e-4                                   # same tolerance as the parity tests
        assert rel_err(y, oracle.gemm_q4k(a, w, m, n, k)) < 2e-3      # and the contract bound


@pytest.mark.gpu
def test_noalloc_refuses_shapes_beyond_its_scratch(backend):
    lib = capi.load_library()
    limit = lib.tsr_gemm_q4k_noalloc_max_outputs()
    assert limit == 1 << 20
    buf = backend.AllocateBuffer(4096)
    rc = lib.tsr_gemm_q4k_noalloc(buf.Handle(), buf.Handle(), buf.Handle(), 2, limit, 256, backend.stream())
    assert rc == capi.StatusCode.InvalidArgument
