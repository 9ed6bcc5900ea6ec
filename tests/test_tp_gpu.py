"""The peer-memory all-reduce on GPUs: one rank, two ranks in one process
(the reference's thread-per-rank layout), graph replay, and the bounded wait."""
import ctypes as C

import numpy as np
import pytest

from tessera_b200 import capi
from tessera_b200.backend import CreateBackend
from tessera_b200.tp import TpComm, rank_order_sum

pytestmark = pytest.mark.gpu


def device_count():
    n = C.c_int()
    capi.load_library().tsr_device_count(C.byref(n))
    return n.value


def make_backend(index):
    b = CreateBackend()
    b.SetDeviceIndex(index)
    b.Init()
    return b


def test_single_rank_is_the_identity(backend):
    comm = TpComm(0, 0, 1, 5120)
    x = np.random.default_rng(0).standard_normal(5120).astype(np.float32)
    buf = backend.upload(x)
    for _ in range(3):
        comm.allreduce(buf.Handle(), 5120, backend.stream())
    assert np.array_equal(backend.download(buf, np.float32, 5120), x)
    assert comm.error_count() == 0
    odd = backend.upload(x[:4099])
    comm.allreduce(odd.Handle(), 4099, backend.stream())         # any count up to the capacity
    assert np.array_equal(backend.download(odd, np.float32, 4099), x[:4099])
    with pytest.raises(capi.StatusError):
        comm.allreduce(buf.Handle(), 1 << 20, backend.stream())  # beyond the capacity
    backend.Synchronize()
    comm.close()


@pytest.mark.parametrize("split", [1, 4, 5])
def test_fused_split_reduce_on_one_rank_equals_vec_reduce(backend, oracle, split):
    """tsr_tp_reduce_allreduce at world 1 is gemm_vec_reduce: same order, same bits."""
    comm = TpComm(0, 0, 1, 5120)
    parts = np.random.default_rng(split).standard_normal((split, 5120)).astype(np.float32)
    src = backend.upload(parts.reshape(-1))
    out = backend.AllocateBuffer(5120 * 4)
    comm.reduce_allreduce(src.Handle(), split, out.Handle(), 5120, backend.stream())
    got = backend.download(out, np.float32, 5120)
    want = oracle.gemm_vec_reduce(parts) if split > 1 else parts[0]
    assert np.array_equal(got, want)
    assert comm.error_count() == 0
    comm.close()


def test_wait_for_a_silent_peer_gives_up_with_a_status(backend):
    """Rank 1 never launches: rank 0's wait runs out, the kernel returns and
    the communicator reports it; the context stays usable."""
    c0 = TpComm(0, 0, 2, 1024)
    c1 = TpComm(0, 1, 2, 1024)
    c0.attach_local(c1)
    x = np.ones(1024, dtype=np.float32)
    buf = backend.upload(x)
    c0.allreduce(buf.Handle(), 1024, backend.stream())
    backend.Synchronize()
    assert c0.error_count() >= 1
    buf2 = backend.upload(x)
    assert np.array_equal(backend.download(buf2, np.float32, 1024), x)
    c0.close()
    c1.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_in_one_process(world):
    if device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    backends = [make_backend(i) for i in range(world)]
    count = 16 * 5120
    comms = [TpComm(i, i, world, count) for i in range(world)]
    for a in comms:
        for b in comms:
            if a is not b:
                a.attach_local(b)
    g = np.random.default_rng(3)
    for it in range(4):
        n = 5120 if it % 2 == 0 else count
        parts = [(g.standard_normal(n) * 10.0 ** r).astype(np.float32) for r in range(world)]
        bufs = [backends[r].upload(parts[r]) for r in range(world)]
        for r in range(world):
            comms[r].allreduce(bufs[r].Handle(), n, backends[r].stream())
        want = rank_order_sum(parts)
        for r in range(world):
            got = backends[r].download(bufs[r], np.float32, n)
            assert np.array_equal(got, want), (it, r)
    # every device of the process runs the staged kernels (their shared-memory limit is a
    # per-device attribute): the same small projection on each rank's backend
    from oracle.oracle import Oracle
    from tessera_b200 import synth
    from tessera_b200.project import Projector, Q4K
    a = synth.activations(1, 1024, seed=9)
    w = synth.q4k_weights(96, 1024, seed=9)
    ref = Oracle().gemm_q4k(a, w, 1, 96, 1024)
    for r in range(world):
        out = backends[r].AllocateBuffer(96 * 4)
        Projector(backends[r]).ProjectBatch(Q4K, backends[r].upload(a), backends[r].upload(w), out, 1, 96, 1024)
        got = backends[r].download(out, np.float32, 96).reshape(1, 96)
        assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-5, r
    # fused split-K reduce + all-reduce: region-order sums per rank, then the rank-order sum
    split = 4
    regions = [(g.standard_normal((split, 5120))).astype(np.float32) for _ in range(world)]
    srcs = [backends[r].upload(regions[r].reshape(-1)) for r in range(world)]
    outs = [backends[r].AllocateBuffer(5120 * 4) for r in range(world)]
    for r in range(world):
        comms[r].reduce_allreduce(srcs[r].Handle(), split, outs[r].Handle(), 5120, backends[r].stream())
    local = []
    for r in range(world):
        acc = np.zeros(5120, dtype=np.float32)
        for s_ in range(split):
            acc = acc + regions[r][s_]
        local.append(acc)
    want = rank_order_sum(local)
    for r in range(world):
        assert np.array_equal(backends[r].download(outs[r], np.float32, 5120), want), r
    assert all(c.error_count() == 0 for c in comms)
    for b in backends:
        b.Synchronize()
    for c in comms:
        c.close()
    for b in backends:
        b.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fmt,m", [("q4k", 1), ("q4k", 16), ("q6k", 1), ("q6k", 4), ("mxfp4", 1), ("mxfp4", 16)])
def test_row_parallel_projection_matches_the_unsharded_one(world, fmt, m):
    """The down projection's shape in k (17408: 68 blocks, uneven on 8 ranks), cut for every rank
    by the library's slicer from one full tensor, projected per rank and summed over ranks by the
    launch itself (Q4_K, Q6_K at m <= 8) or by allreduce_sum: within 2e-3 of the un-sharded CPU
    reference, and the same bits on every rank."""
    if device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from oracle.oracle import Oracle
    from tessera_b200 import tp_check
    n, k = 640, 17408
    case = tp_check.make_case(fmt, m, n, k, seed=21)
    oracle = Oracle()
    ref = {"q4k": oracle.gemm_q4k, "q6k": oracle.gemm_q6k, "mxfp4": oracle.gemm_mxfp4}[fmt](
        case.activations, case.weight, m, n, k)
    backends = [make_backend(i) for i in range(world)]
    comms = [TpComm(i, i, world, 16 * 5120) for i in range(world)]
    for a in comms:
        for b in comms:
            if a is not b:
                a.attach_local(b)
    outs = []
    for r in range(world):
        backends[r].BindTensorParallel(comms[r])
        a, w, k_local = tp_check.rank_inputs(case, r, world)
        ab, wb = backends[r].upload(a), backends[r].upload(w)
        out = backends[r].AllocateBuffer(m * n * 4)
        outs.append((ab, wb, out, k_local))
    for rep in range(2):
        for r in range(world):   # nothing here blocks: the kernels of all ranks meet on the GPUs
            ab, wb, out, k_local = outs[r]
            tp_check.launch_rank(backends[r], case, ab, wb, out, k_local)
        got = [backends[r].download(outs[r][2], np.float32, m * n).reshape(m, n) for r in range(world)]
        for r in range(world):
            assert tp_check.max_rel_err(got[r], ref) < 2e-3, (rep, r, tp_check.max_rel_err(got[r], ref))
            assert np.array_equal(got[r], got[0]), (rep, r)
    assert all(c.error_count() == 0 for c in comms)
    for r in range(world):
        backends[r].BindTensorParallel(None)
        backends[r].Synchronize()
    for c in comms:
        c.close()
    for b in backends:
        b.close()


def test_peer_with_another_capacity_is_refused(backend):
    """Every rank computes its peers' offsets from its own capacity: a block made with another
    one must not be attached."""
    c0 = TpComm(0, 0, 2, 1024)
    c1 = TpComm(0, 1, 2, 4096)
    with pytest.raises(capi.StatusError) as e:
        c0.attach_local(c1)
    assert e.value.code == capi.StatusCode.InvalidArgument
    c0.close()
    c1.close()
