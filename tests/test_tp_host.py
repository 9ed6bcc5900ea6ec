"""Tensor-parallel host logic on CPU ranks (gloo, world size 2) and the shard maps."""
import os
import subprocess
import sys

import numpy as np

from tessera_b200 import synth, workload
from tessera_b200.tp import rank_order_sum

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_cpu_ranks_match_the_unsharded_projection():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29531", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29531",
           os.path.join(ROOT, "tests", "tp_gloo_worker.py")]
    run = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]


def test_shards_cover_every_projection_at_every_world_size():
    for world in (1, 2, 4, 8):
        total = 0
        for p in workload.decode_projections():
            shards = [workload.shard(p, r, world) for r in range(world)]
            if p.kind == workload.COLUMN:
                assert sum(s[0] for s in shards) == p.n
                assert all(s[1] == p.k for s in shards)
            else:
                assert sum(s[1] for s in shards) == p.k
                assert all(s[0] == p.n and s[1] % 256 == 0 and s[1] > 0 for s in shards)
        for r in range(world):
            total += workload.total_weight_bytes(r, world)
        assert total == workload.total_weight_bytes(0, 1)
    # the 17408-wide down projection has 68 blocks: at 8 ranks four take 9 and four take 8 (Q4_K);
    # a Q6_K one is cut in units of four blocks (8-byte aligned rows): seven ranks of 8, one of 12
    downs = [p for p in workload.decode_projections() if p.name == "ffn_down"]
    q4 = next(p for p in downs if p.dtype == "q4k")
    q6 = next(p for p in downs if p.dtype == "q6k")
    assert sorted(workload.shard(q4, r, 8)[1] // 256 for r in range(8)) == [8] * 4 + [9] * 4
    assert sorted(workload.shard(q6, r, 8)[1] // 256 for r in range(8)) == [8] * 7 + [12]
    # gate and up of a layer produce exactly the slice of the FFN activation its down projection reads
    for world in (2, 4, 8):
        for layer in (0, 1):
            gate = next(p for p in workload.decode_projections() if p.name == "ffn_gate" and p.layer == layer)
            down = next(p for p in downs if p.layer == layer)
            for r in range(world):
                assert workload.shard(gate, r, world)[0] == workload.shard(down, r, world)[1]


def test_slice_helpers_match_column_ranges():
    n, k = 8, 1024
    w = synth.q4k_weights(n, k, seed=1).reshape(n, 4, 144)
    for rank in range(2):
        part = synth.slice_rows_by_block(w.reshape(-1), n, k, 144, rank, 2).reshape(n, 2, 144)
        assert np.array_equal(part, w[:, 2 * rank:2 * rank + 2])
    wm = synth.mxfp4_weights(n, k, seed=2)
    half = synth.slice_mxfp4_cols(wm, n, k, 1, 2)
    assert half.size == n * k // 4 + n * k // 64
    assert np.array_equal(half[: n * k // 4].reshape(n, -1), wm[: n * k // 2].reshape(n, -1)[:, k // 4:])


def test_rank_order_sum_is_left_to_right():
    parts = [np.float32([1e8]), np.float32([1.0]), np.float32([-1e8]), np.float32([1.0])]
    assert rank_order_sum(parts)[0] == np.float32(np.float32(np.float32(1e8 + 1.0) - 1e8) + 1.0)
