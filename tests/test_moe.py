"""Routed-expert kernels: the oracle's restatement of the device contracts pinned to the
reference's CpuMoeExpertsForward (CPU), and the CUDA kernels against the oracle (GPU)."""
import importlib.util
import os

import numpy as np
import pytest

from tessera_b200 import synth
from tessera_b200.backend import KernelLaunch

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_moe_golden", os.path.join(HERE, "golden", "make_moe_golden.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)


def golden_case():
    g = np.load(os.path.join(HERE, "golden", "moe_golden.npz"))
    gate, up, down4, down6 = gen.expert_tensors(500)
    return g, gate, up, down4, down6


def test_oracle_chain_equals_the_reference_cpu_experts(oracle):
    """gate/up -> silu product -> weighted down accumulation, as the device contracts split it,
    against the reference's one-call host forward (sums associate differently: 2e-6)."""
    g, gate, up, down4, down6 = golden_case()
    h, i = gen.HIDDEN, gen.INTER
    per = i * (h // 256) * 144
    phi = oracle.moe_experts_gate_up_q4k(g["x"], gate, up, g["ids"], h, i, per, per)
    for fmt, down, bb, key in ((0, down4, 144, "acc_q4k"), (1, down6, 210, "acc_q6k")):
        out = oracle.moe_experts_down(fmt, phi, down, g["ids"], g["wts"], h, i, h * (i // 256) * bb, out=g["acc0"])
        assert np.abs(out - g[key]).max() <= 2e-6 * np.abs(g[key]).max()


def test_reference_build_still_gives_the_fixture(reference_oracle):
    g, gate, up, down4, down6 = golden_case()
    h, i = gen.HIDDEN, gen.INTER
    per = i * (h // 256) * 144
    out = reference_oracle.moe_experts_forward(g["x"], g["ids"], g["wts"], gate, per, up, per, 10, down4,
                                               h * (i // 256) * 144, h, i, g["acc0"])
    assert np.array_equal(out, g["acc_q4k"])


def moe_case(hidden, inter, experts, top_k, seed, q6_down):
    g = np.random.default_rng(seed)
    gate = np.concatenate([synth.q4k_weights(inter, hidden, seed=seed + e, index=1) for e in range(experts)])
    up = np.concatenate([synth.q4k_weights(inter, hidden, seed=seed + e, index=2) for e in range(experts)])
    mk = synth.q6k_weights if q6_down else synth.q4k_weights
    down = np.concatenate([mk(hidden, inter, seed=seed + e, index=3) for e in range(experts)])
    x = (g.standard_normal(hidden) * 0.02).astype(np.float32)
    ids = g.choice(experts, size=top_k, replace=False).astype(np.uint32)
    return gate, up, down, x, ids


@pytest.mark.gpu
@pytest.mark.parametrize("hidden,inter,experts,top_k,q6", [(512, 256, 6, 4, False), (2048, 512, 16, 8, False),
                                                           (2048, 512, 16, 8, True), (1024, 768, 5, 1, True)])
def test_expert_kernels_match_the_oracle(backend, oracle, hidden, inter, experts, top_k, q6):
    gate, up, down, x, ids = moe_case(hidden, inter, experts, top_k, 900 + hidden + inter, q6)
    per_gu = inter * (hidden // 256) * 144
    per_d = hidden * (inter // 256) * (210 if q6 else 144)
    g = np.random.default_rng(3)
    logits = g.standard_normal(top_k).astype(np.float32) * 3
    shared_w = g.standard_normal(hidden).astype(np.float32)
    bx, bg, bu, bd, bi = (backend.upload(v) for v in (x, gate, up, down, ids))
    # moe_gate
    bl, bsw = backend.upload(logits), backend.upload(shared_w)
    bw, bs = backend.AllocateBuffer(top_k * 4), backend.AllocateBuffer(4)
    backend.LaunchKernel(backend.LoadKernel("moe_gate"), KernelLaunch(buffers=[bl, bx, bsw, bw, bs], scalars=[top_k, hidden]))
    wts = backend.download(bw, np.float32, top_k)
    sig = backend.download(bs, np.float32, 1)
    want_w, want_s = oracle.moe_gate(logits, x, shared_w)
    assert np.allclose(wts, want_w, rtol=2e-6, atol=1e-7) and np.allclose(sig, want_s, rtol=2e-6)
    # gate/up with the silu product
    canary = np.float32(-3.5e9)
    bphi = backend.upload(np.full(top_k * inter + 32, canary, dtype=np.float32))
    backend.LaunchKernel(backend.LoadKernel("moe_experts_gate_up_q4k"),
                         KernelLaunch(buffers=[bx, bg, bu, bi, bphi], scalars=[hidden, inter, top_k, per_gu, per_gu]))
    phi = backend.download(bphi, np.float32, top_k * inter + 32)
    assert np.all(phi[top_k * inter:] == canary)
    phi = phi[:top_k * inter].reshape(top_k, inter)
    want_phi = oracle.moe_experts_gate_up_q4k(x, gate, up, ids, hidden, inter, per_gu, per_gu)
    assert np.abs(phi - want_phi).max() <= 2e-5 * np.abs(want_phi).max()
    # weighted down accumulation, written and accumulated
    bphi2 = backend.upload(want_phi.reshape(-1))
    base = g.standard_normal(hidden).astype(np.float32)
    for accumulate in (0, 1):
        bout = backend.upload(base)
        backend.LaunchKernel(backend.LoadKernel("moe_experts_down_q6k" if q6 else "moe_experts_down_q4k"),
                             KernelLaunch(buffers=[bphi2, bd, bi, bw, bout], scalars=[hidden, inter, top_k, per_d, accumulate]))
        got = backend.download(bout, np.float32, hidden)
        want = oracle.moe_experts_down(1 if q6 else 0, want_phi, down, ids, wts, hidden, inter, per_d,
                                       out=base if accumulate else None)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max(), accumulate
    # moe_scale_add
    a, b = g.standard_normal(hidden).astype(np.float32), g.standard_normal(hidden).astype(np.float32)
    bo = backend.AllocateBuffer(hidden * 4)
    backend.LaunchKernel(backend.LoadKernel("moe_scale_add"),
                         KernelLaunch(buffers=[backend.upload(a), backend.upload(b), bw, bo], scalars=[hidden, top_k - 1]))
    assert np.array_equal(backend.download(bo, np.float32, hidden), oracle.moe_scale_add(a, b, wts, top_k - 1))


@pytest.mark.gpu
def test_expert_ids_beyond_the_tensors_are_refused_or_ignored(backend):
    from tessera_b200 import capi
    hidden, inter, experts, top_k = 512, 256, 3, 2
    gate, up, down, x, _ = moe_case(hidden, inter, experts, top_k, 77, False)
    per = inter * (hidden // 256) * 144
    ids = np.array([1, 9], dtype=np.uint32)    # 9 is not an expert of these tensors
    bphi = backend.AllocateBuffer(top_k * inter * 4)
    backend.LaunchKernel(backend.LoadKernel("moe_experts_gate_up_q4k"),
                         KernelLaunch(buffers=[backend.upload(x), backend.upload(gate), backend.upload(up), backend.upload(ids), bphi],
                                      scalars=[hidden, inter, top_k, per, per]))
    phi = backend.download(bphi, np.float32, top_k * inter).reshape(top_k, inter)
    assert np.all(phi[1] == 0.0) and np.any(phi[0] != 0.0)
    small = backend.AllocateBuffer(64)
    with pytest.raises(capi.StatusError):     # gate tensor smaller than one expert
        backend.LaunchKernel(backend.LoadKernel("moe_experts_gate_up_q4k"),
                             KernelLaunch(buffers=[backend.upload(x), small, backend.upload(up), backend.upload(ids), bphi],
                                          scalars=[hidden, inter, top_k, per, per]))
    backend.Synchronize()
