"""One CPU rank of the tensor-parallel host-logic test (launched by
tests/test_tp_host.py with the gloo backend)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle.oracle import Oracle  # noqa: E402
from tessera_b200 import synth, workload  # noqa: E402
from tessera_b200.tp import rank_order_sum  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    oracle = Oracle()
    n, k, m = 48, 2048, 2
    a = synth.activations(m, k, seed=70)
    ok = True
    for dtype, bb, gen, gemm in (("q4k", 144, synth.q4k_weights, oracle.gemm_q4k),
                                 ("q6k", 210, synth.q6k_weights, oracle.gemm_q6k)):
        w = gen(n, k, seed=71)
        full = gemm(a, w, m, n, k)
        # row-parallel: this rank's block range of k, repacked contiguous
        w_r = synth.slice_rows_by_block(w, n, k, bb, rank, world)
        kp = k // world
        a_r = np.ascontiguousarray(a[:, rank * kp:(rank + 1) * kp])
        part = gemm(a_r, w_r, m, n, kp)
        gathered = [torch.zeros(m, n) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(part))
        total = rank_order_sum([g.numpy() for g in gathered])
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        err = np.abs(total - full).max() / np.abs(full).max()
        ok &= bool(err < 2e-3)
        ok &= bool(np.abs(t.numpy() - total).max() <= 1e-5 * np.abs(total).max())
        # column-parallel: a contiguous row range needs no reduce
        rows = n // world
        w_c = w.reshape(n, -1)[rank * rows:(rank + 1) * rows].reshape(-1)
        col = gemm(a, np.ascontiguousarray(w_c), m, rows, k)
        ok &= bool(np.array_equal(col, full[:, rank * rows:(rank + 1) * rows]))
    # every projection of the decode step is covered exactly once by the shards
    for p in workload.decode_projections()[:16]:
        ns = [workload.shard(p, r, world) for r in range(world)]
        if p.kind == workload.COLUMN:
            ok &= sum(x[0] for x in ns) == p.n and all(x[1] == p.k for x in ns)
        else:
            ok &= sum(x[1] for x in ns) == p.k and all(x[0] == p.n and x[1] % 256 == 0 for x in ns)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
