"""rmsnorm, silu_mul and add on the GPU: as kernels of their own, and folded by the deferred
queue into the projection that follows (rmsnorm, silu_mul) or precedes (add) them.  Every
buffer the reference's launch sequence writes must hold what the CPU oracle computes for that
sequence, whether or not the steps were folded."""
import numpy as np
import pytest

from tessera_b200 import synth
from tessera_b200.backend import KernelLaunch
from tessera_b200.project import Q4K, Q6K, Projector

from conftest import per_element_ok, rel_err

pytestmark = pytest.mark.gpu

EPS = 1e-6


def bits(x):
    return int(np.float32(x).view(np.uint32))


def close(y, r, tol):
    return float(np.abs(y - r).max()) <= tol * float(np.abs(r).max())


@pytest.mark.parametrize("rows,cols", [(1, 5120), (3, 1000), (8, 17408), (2, 17)])
def test_rmsnorm_kernel(backend, oracle, rows, cols):
    g = np.random.default_rng(rows * 31 + cols)
    x = g.standard_normal((rows, cols)).astype(np.float32) * 3.0
    w = (1.0 + 0.1 * g.standard_normal(cols)).astype(np.float32)
    xb, wb = backend.upload(x), backend.upload(w)
    yb = backend.AllocateBuffer(x.nbytes)
    backend.LaunchKernel(backend.LoadKernel("rmsnorm"), KernelLaunch(buffers=[xb, wb, yb], scalars=[rows, cols, bits(EPS)]))
    got = backend.download(yb, np.float32, x.size).reshape(rows, cols)
    assert close(got, oracle.rmsnorm(x, w, EPS), 2e-6)


def test_silu_mul_kernel(backend, oracle):
    g = np.random.default_rng(7)
    n = 17408 + 5
    gate = (g.standard_normal(n) * 4.0).astype(np.float32)
    gate[:4] = [0.0, -90.0, 90.0, -1e-30]
    up = g.standard_normal(n).astype(np.float32)
    ob = backend.AllocateBuffer(n * 4)
    backend.LaunchKernel(backend.LoadKernel("silu_mul"), KernelLaunch(buffers=[backend.upload(gate), backend.upload(up), ob], scalars=[n]))
    got = backend.download(ob, np.float32, n)
    want = oracle.silu_mul(gate, up)
    assert np.all(np.abs(got - want) <= 4e-7 * np.abs(want) + 1e-37)


def test_elementwise_ids_check_their_arguments(backend):
    from tessera_b200 import capi
    buf = backend.AllocateBuffer(4096)
    with pytest.raises(capi.StatusError):
        backend.LaunchKernel(backend.LoadKernel("rmsnorm"), KernelLaunch(buffers=[buf, buf, buf], scalars=[1, 4096, bits(EPS)]))  # X too small
    with pytest.raises(capi.StatusError):
        backend.LaunchKernel(backend.LoadKernel("rmsnorm"), KernelLaunch(buffers=[buf, buf, buf], scalars=[1, 16, bits(-1.0)]))   # eps < 0
    with pytest.raises(capi.StatusError):
        backend.LaunchKernel(backend.LoadKernel("silu_mul"), KernelLaunch(buffers=[buf, buf, buf], scalars=[0]))
    backend.Synchronize()


class Block:
    """One FFN block as the reference's forward issues it: rmsnorm, gate and up projections,
    silu_mul, down projection, residual add (src/models/qwen3_5/trunk.cpp:440-470)."""

    def __init__(self, backend, oracle, m, hidden, ffn, down_fmt, seed, in_place_residual):
        g = np.random.default_rng(seed)
        self.m, self.hidden, self.ffn, self.down_fmt = m, hidden, ffn, down_fmt
        self.x = g.standard_normal((m, hidden)).astype(np.float32)
        self.nw = (1.0 + 0.1 * g.standard_normal(hidden)).astype(np.float32)
        self.wg = synth.q4k_weights(ffn, hidden, seed=seed + 1)
        self.wu = synth.q4k_weights(ffn, hidden, seed=seed + 2)
        self.wd = synth.q4k_weights(hidden, ffn, seed=seed + 3) if down_fmt == Q4K else synth.q6k_weights(hidden, ffn, seed=seed + 3)
        # expected contents of every buffer of the sequence
        y = oracle.rmsnorm(self.x, self.nw, EPS)
        self.want = {"y": y}
        gate = oracle.gemm_q4k(y, self.wg, m, ffn, hidden)
        up = oracle.gemm_q4k(y, self.wu, m, ffn, hidden)
        act = oracle.silu_mul(gate.reshape(-1), up.reshape(-1)).reshape(m, ffn)
        down = (oracle.gemm_q4k if down_fmt == Q4K else oracle.gemm_q6k)(act, self.wd, m, hidden, ffn)
        self.want.update(gate=gate, up=up, act=act, down=down, out=oracle.add(self.x.reshape(-1), down.reshape(-1)).reshape(m, hidden))
        b = backend
        self.b = {
            "x": b.upload(self.x), "nw": b.upload(self.nw), "wg": b.upload(self.wg), "wu": b.upload(self.wu),
            "wd": b.upload(self.wd), "y": b.AllocateBuffer(m * hidden * 4), "gate": b.AllocateBuffer(m * ffn * 4),
            "up": b.AllocateBuffer(m * ffn * 4), "act": b.AllocateBuffer(m * ffn * 4),
            "down": b.AllocateBuffer(m * hidden * 4),
        }
        self.b["out"] = self.b["x"] if in_place_residual else b.AllocateBuffer(m * hidden * 4)
        self.in_place = in_place_residual

    def issue(self, backend, proj):
        b, m, hidden, ffn = self.b, self.m, self.hidden, self.ffn
        backend.LaunchKernel(backend.LoadKernel("rmsnorm"), KernelLaunch(buffers=[b["x"], b["nw"], b["y"]], scalars=[m, hidden, bits(EPS)]))
        proj.ProjectBatch(Q4K, b["y"], b["wg"], b["gate"], m, ffn, hidden)
        proj.ProjectBatch(Q4K, b["y"], b["wu"], b["up"], m, ffn, hidden)
        backend.LaunchKernel(backend.LoadKernel("silu_mul"), KernelLaunch(buffers=[b["gate"], b["up"], b["act"]], scalars=[m * ffn]))
        proj.ProjectBatch(self.down_fmt, b["act"], b["wd"], b["down"], m, hidden, ffn)
        backend.LaunchKernel(backend.LoadKernel("add"), KernelLaunch(buffers=[b["x"], b["down"], b["out"]], scalars=[m * hidden]))

    def check(self, backend):
        m, hidden, ffn = self.m, self.hidden, self.ffn
        get = lambda name, n: backend.download(self.b[name], np.float32, m * n).reshape(m, n)
        assert close(get("y", hidden), self.want["y"], 2e-6)
        bound = 2e-5 if m <= 2 else 1e-4
        for name in ("gate", "up"):
            assert rel_err(get(name, ffn), self.want[name]) < bound, name
        # silu_mul and the down projection amplify the projections' rounding: compare with the
        # oracle chain at the projection bound scaled by the chain's depth
        assert rel_err(get("act", ffn), self.want["act"]) < 4 * bound
        down = get("down", hidden)
        assert rel_err(down, self.want["down"]) < 8 * bound
        assert per_element_ok(down, self.want["down"])
        assert rel_err(get("out", hidden), self.want["out"]) < 8 * bound


@pytest.mark.parametrize("m,down_fmt,in_place", [(1, Q4K, False), (1, Q6K, True), (4, Q4K, True), (8, Q6K, False)])
def test_ffn_block_through_the_deferred_queue(backend, oracle, m, down_fmt, in_place):
    """Eight launches of the reference's sequence (rmsnorm, 2 x (vec [+ reduce]), silu_mul,
    vec + reduce, add) leave the queue as two kernels: [rmsnorm + gate + up] and
    [silu_mul + down + add] (three when silu_mul stays a kernel of its own: m = 8 here)."""
    hidden, ffn = 2048, 4096
    blk = Block(backend, oracle, m, hidden, ffn, down_fmt, seed=200 + m, in_place_residual=in_place)
    proj = Projector(backend)
    backend.Synchronize()
    backend.SetDeferred(1)
    try:
        for rep in range(4):
            if in_place:
                backend.CopyH2D(blk.b["x"], blk.x)
                backend.Synchronize()
            api0, dev0, graphs0 = backend.LaunchStats()
            blk.issue(backend, proj)
            backend.Synchronize()
            api1, dev1, graphs1 = backend.LaunchStats()
            # silu_mul is folded only while the work every CTA repeats stays small (row tiles x m x k)
            folded_silu = ((hidden + 47) // 48) * m * ffn <= 1000000
            assert dev1 - dev0 == (2 if folded_silu else 3), dev1 - dev0
            if rep >= 2 and api1 - api0 >= 8:   # queues of eight launches or more are replayed as graphs
                assert graphs1 - graphs0 == 1
            blk.check(backend)
    finally:
        backend.SetDeferred(0)


def test_ffn_block_launch_by_launch_gives_the_same_buffers(backend, oracle):
    """Without the queue every id runs as a kernel of its own."""
    blk = Block(backend, oracle, 2, 2048, 4096, Q4K, seed=300, in_place_residual=False)
    backend.Synchronize()
    _, dev0, _ = backend.LaunchStats()
    blk.issue(backend, Projector(backend))
    backend.Synchronize()
    _, dev1, _ = backend.LaunchStats()
    assert dev1 - dev0 >= 6
    blk.check(backend)


def test_steps_that_would_race_are_not_folded(backend, oracle):
    """rmsnorm in place (Y = X) cannot run inside the projection's CTAs, which all read X;
    an add whose output overlaps the projection's activations cannot either."""
    m, hidden, n = 1, 2048, 512
    g = np.random.default_rng(11)
    x = g.standard_normal((m, hidden)).astype(np.float32)
    nw = (1.0 + 0.1 * g.standard_normal(hidden)).astype(np.float32)
    w = synth.q4k_weights(n, hidden, seed=12)
    w2 = synth.q4k_weights(hidden, hidden, seed=13)
    y = oracle.rmsnorm(x, nw, EPS)
    want = oracle.gemm_q4k(y, w, m, n, hidden)
    want2 = oracle.gemm_q4k(y, w2, m, hidden, hidden)
    xb, nwb, wb, w2b = backend.upload(x), backend.upload(nw), backend.upload(w), backend.upload(w2)
    out, out2 = backend.AllocateBuffer(m * n * 4), backend.AllocateBuffer(m * hidden * 4)
    proj = Projector(backend)
    backend.Synchronize()
    backend.SetDeferred(1)
    try:
        _, dev0, _ = backend.LaunchStats()
        backend.LaunchKernel(backend.LoadKernel("rmsnorm"), KernelLaunch(buffers=[xb, nwb, xb], scalars=[m, hidden, bits(EPS)]))
        proj.ProjectBatch(Q4K, xb, wb, out, m, n, hidden)
        backend.Synchronize()
        _, dev1, _ = backend.LaunchStats()
        assert dev1 - dev0 == 2
        assert close(backend.download(xb, np.float32, hidden).reshape(m, hidden), y, 2e-6)
        assert rel_err(backend.download(out, np.float32, n).reshape(m, n), want) < 2e-5
        # xb now holds y: y2 = y . W2^T, then add(y, y2) written over the activations
        proj.ProjectBatch(Q4K, xb, w2b, out2, m, hidden, hidden)
        backend.LaunchKernel(backend.LoadKernel("add"), KernelLaunch(buffers=[xb, out2, xb], scalars=[hidden]))
        backend.Synchronize()
        _, dev2, _ = backend.LaunchStats()
        assert dev2 - dev1 == 2
        assert rel_err(backend.download(out2, np.float32, hidden).reshape(m, hidden), want2) < 2e-5
        assert rel_err(backend.download(xb, np.float32, hidden).reshape(m, hidden), oracle.add(y.reshape(-1), want2.reshape(-1)).reshape(m, hidden)) < 2e-5
    finally:
        backend.SetDeferred(0)
