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
@pytest.mark.parametrize("m,n,k", [(64, 16384, 2048), (12, 16384, 2816), (32, 4096, 2816)])
def test_noalloc_batches_without_a_usable_split_do_not_allocate(backend, m, n, k):
    """Batches whose block count has no divisor that fits the scratch run unsplit, through the
    batched tile; that tile must then do without its activation scratch.  Free device memory
    is read before and after a call on a stream the library has not seen (after one warm-up
    call elsewhere, which loads the kernels)."""
    import ctypes as C
    import torch
    lib = capi.load_library()
    a = synth.activations(m, k, seed=93)
    w = synth.q4k_weights(n, k, seed=94)
    ab, wb = backend.upload(a), backend.upload(w)
    want = backend.AllocateBuffer(m * n * 4)
    got = backend.AllocateBuffer(m * n * 4)
    assert lib.tsr_gemm_q4k(ab.Handle(), wb.Handle(), want.Handle(), m, n, k, 1, backend.stream()) == 0
    assert lib.tsr_gemm_q4k_noalloc(ab.Handle(), wb.Handle(), got.Handle(), m, n, k, backend.stream()) == 0
    backend.Synchronize()
    fresh = torch.cuda.Stream()
    fresh.synchronize()
    _, free_before = backend.MemoryInfo()
    assert lib.tsr_gemm_q4k_noalloc(ab.Handle(), wb.Handle(), got.Handle(), m, n, k,
                                    C.c_void_p(fresh.cuda_stream)) == 0
    fresh.synchronize()
    _, free_after = backend.MemoryInfo()
    assert free_after >= free_before, (free_before, free_after)
    y = backend.download(got, np.float32, m * n).reshape(m, n)
    r = backend.download(want, np.float32, m * n).reshape(m, n)
    assert rel_err(y, r) < 1e-3   # the batched tile's bound in the parity tests


@pytest.mark.gpu
def test_noalloc_refuses_shapes_beyond_its_scratch(backend):
    lib = capi.load_library()
    limit = lib.tsr_gemm_q4k_noalloc_max_outputs()
    assert limit == 1 << 20
    buf = backend.AllocateBuffer(4096)
    rc = lib.tsr_gemm_q4k_noalloc(buf.Handle(), buf.Handle(), buf.Handle(), 2, limit, 256, backend.stream())
    assert rc == capi.StatusCode.InvalidArgument
