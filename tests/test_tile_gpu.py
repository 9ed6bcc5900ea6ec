"""The tcgen05 tiles that read the weights straight from shared memory (FP8: kind::f8f6f4;
MXFP4: kind::mxf8f6f4 with the weights' own E8M0 scales), the W4A8 contract on them, and the
prefill-sized batches of the older binary16 tile, against the CPU oracle."""
import numpy as np
import pytest

from tessera_b200 import synth
from tessera_b200.backend import KernelLaunch
from tessera_b200.project import F4E2M1, Q4K, Projector

from conftest import per_element_ok, rel_err

pytestmark = pytest.mark.gpu

CANARY = np.float32(-3.5e12)
PAD = 64


def launch(backend, name, buffers, scalars, grid_y=1):
    backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(grid_y=grid_y, buffers=buffers, scalars=scalars))


def padded_output(backend, count):
    return backend.upload(np.full(count + 2 * PAD, CANARY, dtype=np.float32))


def read_padded(backend, buf, count):
    got = backend.download(buf, np.float32, count + 2 * PAD)
    return got[:count], got[count:]


@pytest.mark.parametrize("m", [2, 5, 16, 21])
@pytest.mark.parametrize("n,k", [(128, 256), (136, 640), (1000, 2048), (264, 5120)])
def test_fp8_tile(backend, oracle, m, n, k):
    a = synth.activations(m, k, seed=m)
    w, s = synth.fp8_weights(n, k, seed=m + 1)
    out = padded_output(backend, m * n)   # the output first, the canary words behind it
    launch(backend, "gemm_fp8", [backend.upload(a), backend.upload(w), backend.upload(s), out], [m, n, k])
    got, tail = read_padded(backend, out, m * n)
    assert np.all(tail == CANARY)
    ref = oracle.gemm_fp8(a, w, s, m, n, k)
    assert rel_err(got.reshape(m, n), ref) < 5e-5
    assert per_element_ok(got.reshape(m, n), ref)


@pytest.mark.parametrize("m", [2, 5, 16, 21])
@pytest.mark.parametrize("n,k,exp", [(128, 256, (-8, 0)), (136, 640, (-8, 0)), (1000, 2048, (-40, 30)), (264, 5120, (-14, 2))])
def test_mxfp4_block_scaled_tile(backend, oracle, m, n, k, exp):
    a = synth.activations(m, k, seed=10 + m)
    w = synth.mxfp4_weights(n, k, seed=11 + m, exp_lo=exp[0], exp_hi=exp[1])
    out = padded_output(backend, m * n)
    launch(backend, "gemm_mxfp4_rows" if m <= 16 else "gemm_mxfp4_batched", [backend.upload(a), backend.upload(w), out], [m, n, k])
    got, tail = read_padded(backend, out, m * n)
    assert np.all(tail == CANARY)
    ref = oracle.gemm_mxfp4(a, w, m, n, k)
    assert rel_err(got.reshape(m, n), ref) < 5e-5
    assert per_element_ok(got.reshape(m, n), ref)


@pytest.mark.parametrize("m", [1, 4, 16, 33])
@pytest.mark.parametrize("n,k", [(200, 2048), (136, 640)])
def test_w4a8_unsplit_on_the_tile(backend, oracle, m, n, k):
    """quantize_fp8_pack_rows + mxfp4_row_ref + gemm_mxfp4_wmma with split 1 (ProjectWmma,
    src/models/qwen3_5/project.cpp:92-231): E4M3 activation codes against the MXFP4 nibbles with
    their own scales.  Scales within 2^8 of a row's largest: the reference's fold is exact there,
    so the folded oracle and the tile agree to fp32 summation order."""
    a = synth.activations(m, k, seed=20 + m)
    w = synth.mxfp4_weights(n, k, seed=21 + m, exp_lo=-8, exp_hi=0)
    a8_ref, as_ref = oracle.quantize_fp8_pack(a)
    fold, wref_ref = oracle.fold_mxfp4_to_fp8(w, n, k)
    ref = oracle.gemm_mxfp4_fp8(a8_ref, as_ref, fold, wref_ref, m, n, k)
    ab, wb = backend.upload(a), backend.upload(w)
    a8, as_, wref = backend.AllocateBuffer(m * k), backend.AllocateBuffer(m * 4), backend.AllocateBuffer(n)
    launch(backend, "mxfp4_row_ref", [wb, wref], [n, k])
    launch(backend, "quantize_fp8_pack_rows", [ab, a8, as_], [m, k])
    out = padded_output(backend, m * n)
    launch(backend, "gemm_mxfp4_wmma", [a8, wb, as_, wref, out], [m, n, k, 1, 0])
    got, tail = read_padded(backend, out, m * n)
    assert np.all(tail == CANARY)
    assert rel_err(got.reshape(m, n), ref) < 2e-6


@pytest.mark.parametrize("fmt,n,k", [("mxfp4", 5120, 5120), ("mxfp4", 17408, 5120), ("mxfp4", 5120, 17408),
                                     ("fp8", 5120, 17408)])
@pytest.mark.parametrize("m", [4, 16])
def test_full_size_tiles_on_sampled_rows(backend, oracle, fmt, m, n, k):
    """The measured shapes whole on the GPU; about a hundred weight rows (random ones and tile
    edges) against the oracle run on those rows."""
    a = synth.activations(m, k, seed=30, bf16=True)
    rows = np.unique(np.concatenate([np.random.default_rng(2).integers(0, n, 90), [0, 127, 128, n - 129, n - 128, n - 1]]))
    out = backend.AllocateBuffer(m * n * 4)
    if fmt == "mxfp4":
        w = synth.mxfp4_weights(n, k, seed=31)
        launch(backend, "gemm_mxfp4_rows", [backend.upload(a), backend.upload(w), out], [m, n, k])
        blob, sc = w[: n * k // 2].reshape(n, k // 2), w[n * k // 2:].reshape(n, k // 32)
        sub = np.concatenate([np.ascontiguousarray(blob[rows]).reshape(-1), np.ascontiguousarray(sc[rows]).reshape(-1)])
        ref = oracle.gemm_mxfp4(a, sub, m, len(rows), k)
    else:
        w, s = synth.fp8_weights(n, k, seed=31)
        launch(backend, "gemm_fp8", [backend.upload(a), backend.upload(w), backend.upload(s), out], [m, n, k])
        sub = np.ascontiguousarray(w.reshape(n, k)[rows]).reshape(-1)
        ref = oracle.gemm_fp8(a, sub, np.ascontiguousarray(s[rows]), m, len(rows), k)
    got = backend.download(out, np.float32, m * n).reshape(m, n)
    assert np.isfinite(got).all()
    assert rel_err(got[:, rows], ref) < 5e-5


@pytest.mark.parametrize("m", [100, 256, 300, 512, 700])
def test_prefill_sized_batches(backend, oracle, m):
    """Chunked-prefill batches through the ids ProjectBatch picks for them (gemm_q4k_wmma,
    gemm_mxfp4_batched): the binary16 tcgen05 tile with one binary16 term per activation: 128, 256 or 512
    activation rows per CTA (ragged last chunks included)."""
    n, k = 264, 1024
    a = synth.activations(m, k, seed=40)
    for dtype, w, ref_fn in ((Q4K, synth.q4k_weights(n, k, seed=41), oracle.gemm_q4k),
                             (F4E2M1, synth.mxfp4_weights(n, k, seed=42), oracle.gemm_mxfp4)):
        proj = Projector(backend)
        out = backend.AllocateBuffer(m * n * 4)
        proj.ProjectBatch(dtype, backend.upload(a), backend.upload(w), out, m, n, k)
        got = backend.download(out, np.float32, m * n).reshape(m, n)
        ref = ref_fn(a, w, m, n, k)
        assert rel_err(got, ref) < 1e-3, (dtype, proj.last_kernel)
        # both operands of every product are rounded to binary16 here (as in the reference's own tile): single
        # outputs near zero reach 2.1e-3 of the vector's rms, measured; the max-relative form above is at 4e-4
        assert per_element_ok(got, ref, tol=3e-3)
