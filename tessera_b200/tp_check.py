"""Row-parallel projection cases for checking the tensor-parallel path: a full seeded weight
tensor is cut for every rank by the library's own slicer (tsr_slice_tensor, the rule of the
reference's SliceTensor2D, src/core/loaders/tensor_slice.cpp:105-159, extended to uneven
block ranges), each rank projects its k range and the ranks' partial sums are added by the
library's collective.  The un-sharded result to compare with is the caller's business: the
tests use the CPU reference functions, the benchmark the same GPU with the whole tensor.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import synth
from .backend import Buffer, CudaBackend, KernelLaunch
from .tp import FMT_MXFP4, FMT_Q4K, FMT_Q6K, ROW, slice_shape, slice_tensor

FORMATS = {"q4k": FMT_Q4K, "q6k": FMT_Q6K, "mxfp4": FMT_MXFP4}


@dataclass
class RowParallelCase:
    fmt: str          # "q4k" | "q6k" | "mxfp4"
    m: int
    n: int
    k: int
    weight: np.ndarray       # the whole tensor, packed
    activations: np.ndarray  # (m, k) fp32


def make_case(fmt: str, m: int, n: int, k: int, seed: int, bf16_activations: bool = True) -> RowParallelCase:
    if fmt == "q4k":
        w = synth.q4k_weights(n, k, seed=seed)
    elif fmt == "q6k":
        w = synth.q6k_weights(n, k, seed=seed)
    else:
        w = synth.mxfp4_weights(n, k, seed=seed)
    return RowParallelCase(fmt, m, n, k, w, synth.activations(m, k, seed=seed + 1, bf16=bf16_activations))


def rank_inputs(case: RowParallelCase, rank: int, world: int):
    """(activation columns, weight slice, k of the slice) of one rank."""
    fid = FORMATS[case.fmt]
    _, cols, c0, _ = slice_shape(fid, ROW, case.n, case.k, rank, world)
    w = slice_tensor(fid, ROW, case.n, case.k, rank, world, case.weight)
    a = np.ascontiguousarray(case.activations[:, c0:c0 + cols])
    return a, w, cols


def launch_rank(backend: CudaBackend, case: RowParallelCase, a: Buffer, w: Buffer, out: Buffer, k_local: int) -> None:
    """Queues one rank's share on its backend: the projection of its k range and the sum over
    ranks on the communicator bound to the backend.  Q4_K and Q6_K use the ids that do both in
    one launch; MXFP4 projects with the reference's ids and sums with allreduce_sum."""
    m, n = case.m, case.n
    if case.fmt in ("q4k", "q6k"):
        kern = backend.LoadKernel(f"gemm_{case.fmt}_vec_allreduce")
        backend.LaunchKernel(kern, KernelLaunch(buffers=[a, w, out], scalars=[m, n, k_local]))
        return
    name = "gemm_mxfp4" if m == 1 else ("gemm_mxfp4_rows" if m <= 16 else "gemm_mxfp4_batched")
    backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=[a, w, out], scalars=[m, n, k_local]))
    backend.LaunchKernel(backend.LoadKernel("allreduce_sum"), KernelLaunch(buffers=[out], scalars=[m, n]))


def launch_unsharded(backend: CudaBackend, case: RowParallelCase, a: Buffer, w: Buffer, out: Buffer) -> None:
    """The same projection over the whole k on one GPU, through the reference's ids."""
    m, n, k = case.m, case.n, case.k
    if case.fmt == "mxfp4":
        name = "gemm_mxfp4" if m == 1 else ("gemm_mxfp4_rows" if m <= 16 else "gemm_mxfp4_batched")
        scalars = [m, n, k]
    elif m == 1:
        name, scalars = f"gemm_{case.fmt}_vec", [m, n, k, 1]
    else:
        name, scalars = f"gemm_{case.fmt}_batched", [m, n, k]
    backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=[a, w, out], scalars=scalars))


def launch_ffn_tail(backend: CudaBackend, case: RowParallelCase, gate: Buffer, up: Buffer, act: Buffer, w: Buffer,
                    down: Buffer, residual: Buffer, final: Buffer, k_local: int, sharded: bool) -> None:
    """The end of an FFN block as the reference's forward queues it (silu_mul, down projection,
    residual add; src/models/qwen3_5/trunk.cpp:440-470 of the reference), on one rank's k range
    with the sum over ranks (`sharded`) or on the whole k.  Through the deferred queue the three
    steps become one launch; with the sum over ranks two (the silu_mul stays a kernel of its own there)."""
    m, n = case.m, case.n
    backend.LaunchKernel(backend.LoadKernel("silu_mul"), KernelLaunch(buffers=[gate, up, act], scalars=[m * k_local]))
    if sharded:
        kern = backend.LoadKernel(f"gemm_{case.fmt}_vec_allreduce")
        backend.LaunchKernel(kern, KernelLaunch(buffers=[act, w, down], scalars=[m, n, k_local]))
    else:
        name = f"gemm_{case.fmt}_vec" if m == 1 else f"gemm_{case.fmt}_rows{m}"
        backend.LaunchKernel(backend.LoadKernel(name), KernelLaunch(buffers=[act, w, down], scalars=[m, n, k_local, 1]))
    backend.LaunchKernel(backend.LoadKernel("add"), KernelLaunch(buffers=[residual, down, final], scalars=[m * n]))


def max_rel_err(y: np.ndarray, r: np.ndarray) -> float:
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(r, dtype=np.float64)
    return float(np.abs(y - r).max() / max(np.abs(r).max(), 1e-30))
