"""Merged launches on the GPU: several weight tensors per launch, the split of k and its
sum inside the launch, the tile loop of a small grid, and the deferred queue with its CUDA
graph replay, each against the CPU oracle.  Outputs sit between canary words so that a
store outside the output range of a ragged shape is seen."""
import ctypes as C

import numpy as np
import pytest

from tessera_b200 import capi, synth
from tessera_b200.backend import KernelLaunch
from tessera_b200.project import Q4K, Q6K, Projector

from conftest import per_element_ok, rel_err

pytestmark = pytest.mark.gpu

CANARY = np.float32(-7.25e11)
PAD = 64  # floats before and after every output


def weights(fmt, n, k, seed):
    return synth.q4k_weights(n, k, seed=seed) if fmt == 0 else synth.q6k_weights(n, k, seed=seed)


def oracle_gemm(oracle, fmt, a, w, m, n, k):
    return oracle.gemm_q4k(a, w, m, n, k) if fmt == 0 else oracle.gemm_q6k(a, w, m, n, k)


def run_group(backend, oracle, fmt, m, ns, k, seed, bound):
    lib = capi.load_library()
    a = synth.activations(m, k, seed=seed)
    ab = backend.upload(a)
    ws = [weights(fmt, n, k, seed + 1 + i) for i, n in enumerate(ns)]
    wbs = [backend.upload(w) for w in ws]
    outs = []
    for n in ns:
        host = np.full(m * n + 2 * PAD, CANARY, dtype=np.float32)
        outs.append(backend.upload(host))
    count = len(ns)
    wp = (C.c_void_p * count)(*[b.Handle() for b in wbs])
    cp = (C.c_void_p * count)(*[b.Handle() + PAD * 4 for b in outs])
    np_ = (C.c_uint64 * count)(*ns)
    capi.check(lib.tsr_gemv_group(backend._ctx, fmt, ab.Handle(), wp, cp, np_, count, m, k), "tsr_gemv_group")
    backend.Synchronize()
    for n, w, out in zip(ns, ws, outs):
        got = backend.download(out, np.float32, m * n + 2 * PAD)
        assert np.all(got[:PAD] == CANARY) and np.all(got[PAD + m * n:] == CANARY), ("canary", n)
        y = got[PAD:PAD + m * n].reshape(m, n)
        r = oracle_gemm(oracle, fmt, a, w, m, n, k)
        assert rel_err(y, r) < bound, (fmt, m, n, k, rel_err(y, r))
        assert per_element_ok(y, r)


@pytest.mark.parametrize("m", [1, 2, 3, 8])
def test_q4k_group_of_four_weights(backend, oracle, m):
    run_group(backend, oracle, 0, m, [520, 96, 48, 17], 2048, seed=40 + m, bound=2e-5 if m <= 2 else 1e-4)


@pytest.mark.parametrize("m", [1, 4])
def test_q6k_group_of_three_weights(backend, oracle, m):
    run_group(backend, oracle, 1, m, [130, 48, 6], 2048, seed=50 + m, bound=2e-5 if m <= 2 else 1e-4)


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("cluster", [1, 0])
@pytest.mark.parametrize("split,grid,rgs", [(2, 0, 0), (4, 3, 1), (1, 2, 2), (8, 1, 4), (4, 0, 3), (8, 0, 2)])
def test_split_inside_the_launch_and_tile_loop(backend, oracle, monkeypatch, fmt, cluster, split, grid, rgs):
    """Forces the number of k chunks, a grid smaller than the tile list (every CTA then works
    through several tiles) and the tile height; the plan picks them by itself otherwise.  The
    chunks of a tile meet in the shared memory of a thread-block cluster where a CTA has at most
    two tiles, else (and with cluster = 0 always) through tickets in global memory."""
    monkeypatch.setenv("TSR_CLUSTER", str(cluster))
    monkeypatch.setenv("TSR_SPLIT", str(split))
    if grid:
        monkeypatch.setenv("TSR_GRID", str(grid))
    if rgs:
        monkeypatch.setenv("TSR_RGS", str(rgs))
    run_group(backend, oracle, fmt, 1, [200, 72], 4096, seed=60 + split, bound=2e-5)
    run_group(backend, oracle, fmt, 5, [136], 4096, seed=70 + split, bound=1e-4)


def test_full_size_group_on_sampled_rows(backend, oracle):
    """ffn_gate + ffn_up of the 27B-class layer as one launch, checked on sampled rows."""
    lib = capi.load_library()
    n, k, m = 17408, 5120, 1
    a = synth.activations(m, k, seed=80)
    ab = backend.upload(a)
    ws = [synth.q4k_weights(n, k, seed=81 + i) for i in range(2)]
    wbs = [backend.upload(w) for w in ws]
    outs = [backend.AllocateBuffer(m * n * 4) for _ in range(2)]
    wp = (C.c_void_p * 2)(*[b.Handle() for b in wbs])
    cp = (C.c_void_p * 2)(*[b.Handle() for b in outs])
    np_ = (C.c_uint64 * 2)(n, n)
    capi.check(lib.tsr_gemv_group(backend._ctx, 0, ab.Handle(), wp, cp, np_, 2, m, k))
    backend.Synchronize()
    rows = np.unique(np.concatenate([np.random.default_rng(1).integers(0, n, 90), [0, 63, 64, n - 65, n - 64, n - 1]]))
    rb = (k // 256) * 144
    for w, out in zip(ws, outs):
        got = backend.download(out, np.float32, m * n).reshape(m, n)[:, rows]
        sub = np.concatenate([w[r * rb:(r + 1) * rb] for r in rows])
        ref = oracle.gemm_q4k(a, sub, m, len(rows), k)
        assert rel_err(got, ref) < 2e-5


def test_deferred_queue_merges_and_replays_as_a_graph(backend, oracle):
    """Three split projections that share their activations plus a fourth with its own: the
    reference's launch sequence (gemm_*_vec + gemm_vec_reduce each) goes into the queue, comes
    out as fewer kernels, and from the second repetition on as one CUDA graph launch."""
    proj = Projector(backend)
    k, m = 5120, 1
    ns = [1024, 768, 48]
    a = synth.activations(m, k, seed=90)
    a2 = synth.activations(m, 2048, seed=91)
    ab, a2b = backend.upload(a), backend.upload(a2)
    ws = [synth.q4k_weights(n, k, seed=92 + i) for i, n in enumerate(ns)]
    w2 = synth.q6k_weights(520, 2048, seed=99)
    wbs = [backend.upload(w) for w in ws]
    w2b = backend.upload(w2)
    outs = [backend.AllocateBuffer(m * n * 4) for n in ns]
    out2 = backend.AllocateBuffer(520 * 4)
    refs = [oracle.gemm_q4k(a, w, m, n, k) for w, n in zip(ws, ns)]
    ref2 = oracle.gemm_q6k(a2, w2, m, 520, 2048)
    backend.Synchronize()
    backend.SetDeferred(1)
    try:
        first = None
        for rep in range(4):
            api0, dev0, graphs0 = backend.LaunchStats()
            for wb, out, n in zip(wbs, outs, ns):
                proj.ProjectBatch(Q4K, ab, wb, out, m, n, k)
            proj.ProjectBatch(Q6K, a2b, w2b, out2, m, 520, 2048)
            backend.Synchronize()
            api1, dev1, graphs1 = backend.LaunchStats()
            assert api1 - api0 == 8            # four projections, each gemm_*_vec + gemm_vec_reduce
            assert dev1 - dev0 == 2, dev1 - dev0  # one launch for the three that share a, one for the other
            got = [backend.download(o, np.float32, m * n).reshape(m, n) for o, n in zip(outs, ns)]
            got2 = backend.download(out2, np.float32, 520).reshape(1, 520)
            for y, r in zip(got, refs):
                assert rel_err(y, r) < 2e-5
            assert rel_err(got2, ref2) < 2e-5
            if first is None:
                first = got
            else:
                assert all(np.array_equal(x, y) for x, y in zip(first, got))  # replays repeat the bits
            if rep >= 2:
                assert graphs1 - graphs0 == 1
    finally:
        backend.SetDeferred(0)


@pytest.mark.parametrize("m", [11, 16])
def test_deferred_queue_merges_verify_batches_as_two_passes(backend, oracle, m):
    """Nine to sixteen rows (a speculative-verify step): projections that share their activations leave the
    queue as the merged launch run twice, eight rows and the rest; a single projection over a long k (which
    one staged pass cannot hold in shared memory) the same way with k cut inside the launch."""
    proj = Projector(backend)
    k, ns = 5120, [1024, 768, 48]
    a = synth.activations(m, k, seed=190)
    ab = backend.upload(a)
    ws = [synth.q4k_weights(n, k, seed=192 + i) for i, n in enumerate(ns)]
    wbs = [backend.upload(w) for w in ws]
    k2, n2 = 17408, 264
    a2 = synth.activations(m, k2, seed=191)
    w2 = synth.q6k_weights(n2, k2, seed=199)
    a2b, w2b = backend.upload(a2), backend.upload(w2)
    outs = [backend.AllocateBuffer(m * n * 4) for n in ns + [n2]]
    refs = [oracle.gemm_q4k(a, w, m, n, k) for w, n in zip(ws, ns)] + [oracle.gemm_q6k(a2, w2, m, n2, k2)]
    backend.Synchronize()
    backend.SetDeferred(1)
    try:
        for rep in range(3):
            _, dev0, _ = backend.LaunchStats()
            for wb, out, n in zip(wbs, outs, ns):
                proj.ProjectBatch(Q4K, ab, wb, out, m, n, k)
            proj.ProjectBatch(Q6K, a2b, w2b, outs[3], m, n2, k2)
            backend.Synchronize()
            _, dev1, _ = backend.LaunchStats()
            assert dev1 - dev0 == 4, dev1 - dev0   # two passes for the three that share a, two for the long one
            for out, n, r in zip(outs, ns + [n2], refs):
                y = backend.download(out, np.float32, m * n).reshape(m, n)
                assert rel_err(y, r) < 2e-4 and per_element_ok(y, r)
    finally:
        backend.SetDeferred(0)


def test_deferred_launch_still_checks_its_arguments_at_once(backend):
    backend.SetDeferred(1)
    try:
        buf = backend.AllocateBuffer(4096)
        kern = backend.LoadKernel("gemm_q4k_vec")
        with pytest.raises(capi.StatusError) as e:
            backend.LaunchKernel(kern, KernelLaunch(buffers=[buf, buf, buf], scalars=[1, 4096, 4096, 1]))
        assert e.value.code == capi.StatusCode.InvalidArgument   # buffers too small for the shape
        with pytest.raises(capi.StatusError):
            backend.LaunchKernel(kern, KernelLaunch(buffers=[buf, buf, buf], scalars=[1, 8, 250, 1]))  # k not whole blocks
        backend.Synchronize()
    finally:
        backend.SetDeferred(0)


def test_deferred_queue_keeps_the_order_of_unmerged_launches(backend):
    """fill -> add -> add on the same buffer must see each other's results."""
    backend.SetDeferred(1)
    try:
        n = 4096
        x = backend.AllocateBuffer(n * 4)
        y = backend.upload(np.full(n, 2.0, dtype=np.float32))
        fill, add = backend.LoadKernel("fill"), backend.LoadKernel("add")
        one = int(np.float32(1.0).view(np.uint32))
        for _ in range(3):
            backend.LaunchKernel(fill, KernelLaunch(buffers=[x], scalars=[one, n]))
            for _ in range(9):
                backend.LaunchKernel(add, KernelLaunch(buffers=[x, y, x], scalars=[n]))
            got = backend.download(x, np.float32, n)
            assert np.all(got == 19.0)
    finally:
        backend.SetDeferred(0)


@pytest.mark.parametrize("name,fmt", [("gemm_q4k_vec_allreduce", 0), ("gemm_q6k_vec_allreduce", 1)])
def test_allreduce_ids_on_a_single_rank_are_the_projection(backend, oracle, name, fmt):
    from tessera_b200.tp import TpComm
    m, n, k = 1, 640, 2048
    a = synth.activations(m, k, seed=33)
    w = weights(fmt, n, k, 34)
    ab, wb = backend.upload(a), backend.upload(w)
    out = backend.AllocateBuffer(m * n * 4)
    kern = backend.LoadKernel(name)
    ref = oracle_gemm(oracle, fmt, a, w, m, n, k)
    backend.LaunchKernel(kern, KernelLaunch(buffers=[ab, wb, out], scalars=[m, n, k]))   # nothing bound
    assert rel_err(backend.download(out, np.float32, n).reshape(1, n), ref) < 2e-5
    comm = TpComm(0, 0, 1, 8 * 5120)
    backend.BindTensorParallel(comm)
    try:
        backend.LaunchKernel(kern, KernelLaunch(buffers=[ab, wb, out], scalars=[m, n, k]))
        assert rel_err(backend.download(out, np.float32, n).reshape(1, n), ref) < 2e-5
        x = np.random.default_rng(5).standard_normal(2 * 5120).astype(np.float32)
        xb = backend.upload(x)
        backend.LaunchKernel(backend.LoadKernel("allreduce_sum"), KernelLaunch(buffers=[xb], scalars=[2, 5120]))
        assert np.array_equal(backend.download(xb, np.float32, x.size), x)
        assert comm.error_count() == 0
    finally:
        backend.BindTensorParallel(None)
        backend.Synchronize()
        comm.close()
