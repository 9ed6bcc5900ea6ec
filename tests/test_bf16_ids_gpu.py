"""The bf16-in / bf16-out projection ids against RoundBf16Ref(Gemm*Ref(A)) of the CPU oracle
on bf16-representable activations.  A sum that lies near a rounding boundary of bf16 may land
on the neighbouring value when the fp32 sum differs in its last bits, so the outputs are
compared in bf16 steps: equal for nearly all, one step apart at most where the value is not
small against the row's largest."""
import numpy as np
import pytest

from tessera_b200 import synth
from tessera_b200.backend import KernelLaunch

pytestmark = pytest.mark.gpu


def to_bf16_bits(x):
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def check(got_bits, want):
    got = from_bf16_bits(got_bits).astype(np.float64)
    want = want.astype(np.float64)
    top = np.abs(want).max()
    step = np.maximum(np.abs(want), 1e-30) * 2.0 ** -7          # one bf16 step is at most 2^-7 of the value
    big = np.abs(want) > 0.02 * top
    assert np.all(np.abs(got - want)[big] <= step[big] * 1.001)
    assert np.all(np.abs(got - want)[~big] <= 2e-3 * top)
    assert np.mean(got == want) > 0.9


@pytest.mark.parametrize("fmt,m,n,k", [
    ("q4k", 1, 640, 2048), ("q4k", 2, 1000, 5120), ("q4k", 5, 136, 4096), ("q4k", 8, 72, 1024),
    ("q6k", 1, 130, 2048), ("q6k", 4, 520, 4096),
    ("q4k", 16, 256, 1024), ("q6k", 12, 96, 1024),            # beyond the staged kernels: fp32 copies around the fp32 id
    ("mxfp4", 1, 520, 1024), ("mxfp4", 16, 256, 2048), ("fp8", 1, 264, 1024), ("fp8", 3, 128, 2048),
])
def test_bf16_projection_ids(backend, oracle, fmt, m, n, k):
    a = synth.activations(m, k, seed=m * 7 + n, bf16=True)
    bufs = [backend.upload(to_bf16_bits(a))]
    if fmt == "q4k":
        w = synth.q4k_weights(n, k, seed=n)
        ref = oracle.gemm_q4k(a, w, m, n, k)
        bufs.append(backend.upload(w))
    elif fmt == "q6k":
        w = synth.q6k_weights(n, k, seed=n)
        ref = oracle.gemm_q6k(a, w, m, n, k)
        bufs.append(backend.upload(w))
    elif fmt == "mxfp4":
        w = synth.mxfp4_weights(n, k, seed=n)
        ref = oracle.gemm_mxfp4(a, w, m, n, k)
        bufs.append(backend.upload(w))
    else:
        w, s = synth.fp8_weights(n, k, seed=n)
        ref = oracle.gemm_fp8(a, w, s, m, n, k)
        bufs += [backend.upload(w), backend.upload(s)]
    canary = np.full(m * n + 64, 0x7FC1, dtype=np.uint16)
    out = backend.upload(canary)
    bufs.append(out)
    kern = backend.LoadKernel(f"gemm_{fmt}_bf16")
    for _ in range(2):
        backend.LaunchKernel(kern, KernelLaunch(buffers=bufs, scalars=[m, n, k]))
    got = backend.download(out, np.uint16, m * n + 64)
    assert np.all(got[m * n:] == 0x7FC1)                      # nothing stored beyond the m x n bf16 values
    check(got[:m * n], oracle.round_bf16(ref.reshape(-1).copy()))


def test_bf16_ids_check_their_arguments(backend):
    from tessera_b200 import capi
    small = backend.AllocateBuffer(1024)
    big = backend.AllocateBuffer(1 << 20)
    with pytest.raises(capi.StatusError):   # A holds fewer than m*k bf16 values
        backend.LaunchKernel(backend.LoadKernel("gemm_q4k_bf16"), KernelLaunch(buffers=[small, big, big], scalars=[1, 16, 2048]))
    with pytest.raises(capi.StatusError):   # k not whole blocks
        backend.LaunchKernel(backend.LoadKernel("gemm_q6k_bf16"), KernelLaunch(buffers=[big, big, big], scalars=[1, 16, 250]))
    with pytest.raises(capi.StatusError):   # fp8 needs the scale buffer
        backend.LaunchKernel(backend.LoadKernel("gemm_fp8_bf16"), KernelLaunch(buffers=[big, big, big], scalars=[1, 16, 256]))
    backend.Synchronize()
