"""Projection planning: which kernel id a (dtype, m, n, k) projection uses.

Mirrors the reference's host-side selection so that the tests drive the
backend exactly as the reference's ``ProjectBatch`` would
(src/models/qwen3_5/project.cpp:233-366, src/models/qwen3_5/internal.hpp:104-199,
src/core/decode_internal.hpp:842-942,1258-1517).
"""
from __future__ import annotations

from .backend import Buffer, CudaBackend, KernelLaunch
from .capi import StatusCode, StatusError

K_GEMM_VEC_OUTPUTS_PER_BLOCK = 8   # decode_internal.hpp:841
K_GEMM_VEC_SPLIT_TARGET = 2048     # decode_internal.hpp:853
K_GEMM_VEC_MAX_SPLIT = 8           # decode_internal.hpp:861
K_GEMM_WMMA_MIN_ROWS = 64          # decode_internal.hpp:1420
K_GEMM_WMMA_MIN_COLS = 32          # decode_internal.hpp:1434
K_TILED_MIN_ROWS = 16              # include/tessera/defaults.hpp (kDefaultTiledMinRows)
K_TILED_MIN_COLS = 65536           # include/tessera/defaults.hpp (kDefaultTiledMinCols)

Q4K, Q6K, F4E2M1 = "q4k", "q6k", "mxfp4"


def GemmVecSplit(outputs: int, k: int, target: int = K_GEMM_VEC_SPLIT_TARGET) -> int:
    """decode_internal.hpp:866-885."""
    blocks_x = (outputs + K_GEMM_VEC_OUTPUTS_PER_BLOCK - 1) // K_GEMM_VEC_OUTPUTS_PER_BLOCK
    if blocks_x == 0 or blocks_x >= target:
        return 1
    superblocks = k // 256
    split = min((target + blocks_x - 1) // blocks_x, K_GEMM_VEC_MAX_SPLIT)
    while split > 1:
        if superblocks % split == 0:
            return split
        split -= 1
    return 1


def GemmKernelName(dtype: str) -> str:
    """decode_internal.hpp:1258-1276."""
    return {Q4K: "gemm_q4k_vec", Q6K: "gemm_q6k_vec", F4E2M1: "gemm_mxfp4"}.get(dtype, "")


def GemmRowsKernelName(dtype: str, rows: int) -> str:
    """decode_internal.hpp:1369-1400."""
    if dtype in (Q4K, Q6K) and 2 <= rows <= 5:
        return f"gemm_{dtype}_rows{rows}"
    return ""


def GemmTiledKernelName(dtype: str) -> str:
    """decode_internal.hpp:1404-1418."""
    return {Q4K: "gemm_q4k_batched", Q6K: "gemm_q6k_batched", F4E2M1: "gemm_mxfp4_batched"}.get(dtype, "")


def GemmWmmaKernelName(dtype: str) -> str:
    """decode_internal.hpp:1449-1461."""
    return {Q4K: "gemm_q4k_wmma", Q6K: "gemm_q6k_wmma"}.get(dtype, "")


class Projector:
    """Per-state kernel cache and scratch, like ``Qwen35State`` holds them."""

    def __init__(self, backend: CudaBackend):
        self.backend = backend
        self._kernels = {}
        self._gemv_part = None
        self.last_kernel = ""

    def kernel(self, name: str):
        """CachedKernel (decode_internal.hpp:1297-1323): a miss is remembered."""
        if name not in self._kernels:
            try:
                self._kernels[name] = self.backend.LoadKernel(name)
            except StatusError as e:
                if e.code != StatusCode.UnsupportedFeature:
                    raise
                self._kernels[name] = None
        return self._kernels[name]

    def _part(self, nbytes: int) -> Buffer:
        if self._gemv_part is None or self._gemv_part.Size() < nbytes:
            self._gemv_part = self.backend.AllocateBuffer(nbytes)
        return self._gemv_part

    def _reduce(self, part: Buffer, out: Buffer, total: int, split: int) -> None:
        launch = KernelLaunch(grid_x=(total + 255) // 256, buffers=[part, out], scalars=[total, split])
        self.backend.LaunchKernel(self.kernel("gemm_vec_reduce"), launch)

    def ProjectGemvDevice(self, gemm, a, w, out, m, n, k) -> None:
        """internal.hpp:104-145."""
        total = m * n
        split = GemmVecSplit(total, k)
        gx = (total + 7) // 8
        if split <= 1:
            self.backend.LaunchKernel(gemm, KernelLaunch(grid_x=gx, buffers=[a, w, out],
                                                         scalars=[m, n, k, 1]))
            return
        part = self._part(split * total * 4)
        self.backend.LaunchKernel(gemm, KernelLaunch(grid_x=gx, grid_y=split, buffers=[a, w, part],
                                                     scalars=[m, n, k, split]))
        self._reduce(part, out, total, split)

    def ProjectGemvPartials(self, dtype: str, a, w, m, n, k):
        """The GEMV half of ProjectGemvDevice: launches gemm_*_vec and returns (partials, split)
        without the gemm_vec_reduce, for a caller that fuses the reduce into the tensor-parallel
        all-reduce (TpComm.reduce_allreduce).  No reference counterpart."""
        gemm = self.kernel(GemmKernelName(dtype))
        if gemm is None or not gemm.Id().endswith("_vec"):
            raise StatusError(StatusCode.UnsupportedFeature, dtype)
        self.last_kernel = gemm.Id()
        total = m * n
        split = GemmVecSplit(total, k)
        part = self._part(split * total * 4)
        self.backend.LaunchKernel(gemm, KernelLaunch(grid_x=(total + 7) // 8, grid_y=split, buffers=[a, w, part],
                                                     scalars=[m, n, k, split]))
        return part, split

    def ProjectGemvRowsDevice(self, gemm, a, w, out, m, n, k) -> None:
        """internal.hpp:154-199."""
        total = m * n
        split = GemmVecSplit(n, k)
        gx = (n + 7) // 8
        dst = self._part(split * total * 4) if split > 1 else out
        self.backend.LaunchKernel(gemm, KernelLaunch(grid_x=gx, grid_y=split, buffers=[a, w, dst],
                                                     scalars=[m, n, k, split]))
        if split > 1:
            self._reduce(dst, out, total, split)

    def ProjectBatch(self, dtype: str, a: Buffer, w: Buffer, out: Buffer, m: int, n: int, k: int) -> None:
        """project.cpp:233-366 without the opt-in W4A8 and bf16 branches."""
        b = self.backend
        if dtype == F4E2M1 and 2 <= m <= 16:
            rows = self.kernel("gemm_mxfp4_rows")
            if rows is not None:
                self.last_kernel = rows.Id()
                b.LaunchKernel(rows, KernelLaunch(grid_x=(n + 7) // 8, buffers=[a, w, out], scalars=[m, n, k]))
                return
        if 2 <= m <= 4 and GemmRowsKernelName(dtype, m):
            rows = self.kernel(GemmRowsKernelName(dtype, m))
            if rows is not None:
                self.last_kernel = rows.Id()
                self.ProjectGemvRowsDevice(rows, a, w, out, m, n, k)
                return
        if m >= K_GEMM_WMMA_MIN_ROWS and n >= K_GEMM_WMMA_MIN_COLS and k % 256 == 0 and GemmWmmaKernelName(dtype):
            wm = self.kernel(GemmWmmaKernelName(dtype))
            if wm is not None:
                self.last_kernel = wm.Id()
                b.LaunchKernel(wm, KernelLaunch(grid_x=(n + 63) // 64, grid_y=(m + 127) // 128,
                                                buffers=[a, w, out], scalars=[m, n, k]))
                return
        if (m >= K_TILED_MIN_ROWS or (m >= 2 and n >= K_TILED_MIN_COLS)) and GemmTiledKernelName(dtype):
            tiled = self.kernel(GemmTiledKernelName(dtype))
            if tiled is not None:
                self.last_kernel = tiled.Id()
                b.LaunchKernel(tiled, KernelLaunch(grid_x=((m + 31) // 32) * ((n + 31) // 32), block_x=1024,
                                                   buffers=[a, w, out], scalars=[m, n, k]))
                return
        gemm = self.kernel(GemmKernelName(dtype))
        if gemm is None:
            raise StatusError(StatusCode.UnsupportedFeature, dtype)
        self.last_kernel = gemm.Id()
        if gemm.Id().endswith("_vec"):
            self.ProjectGemvDevice(gemm, a, w, out, m, n, k)
        else:
            b.LaunchKernel(gemm, KernelLaunch(grid_x=(m * n + 7) // 8, buffers=[a, w, out], scalars=[m, n, k]))
