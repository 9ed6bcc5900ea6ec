"""Tensor-parallel helpers: the peer-memory sum all-reduce and the shard maps.

The reference runs one thread per rank inside one process and reduces the
row-parallel partials through rank 0 (src/core/tensor_parallel.cpp,
src/models/qwen3_5/trunk.cpp:226-266 of the reference).  This module drives
the C ABI's `tsr_tp_*` calls, for ranks inside one process (`attach_local`)
or one process per GPU (`connect`, which swaps the IPC handles through
torch.distributed).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi


class TpComm:
    def __init__(self, device: int, rank: int, world: int, max_floats: int):
        self.lib = capi.load_library()
        self.rank, self.world, self.device = rank, world, device
        comm = C.c_void_p()
        capi.check(self.lib.tsr_tp_create(device, rank, world, max_floats, C.byref(comm)), "tsr_tp_create")
        self.comm = comm

    def local_block(self) -> int:
        ptr, size = C.c_void_p(), C.c_uint64()
        capi.check(self.lib.tsr_tp_local_block(self.comm, C.byref(ptr), C.byref(size)))
        return ptr.value

    def ipc_handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        capi.check(self.lib.tsr_tp_ipc_handle(self.comm, buf), "tsr_tp_ipc_handle")
        return buf.raw

    def attach_ipc(self, peer_rank: int, handle: bytes) -> None:
        capi.check(self.lib.tsr_tp_attach_ipc(self.comm, peer_rank, C.c_char_p(handle)), "tsr_tp_attach_ipc")

    def attach_local(self, peer: "TpComm") -> None:
        capi.check(self.lib.tsr_tp_attach_local(self.comm, peer.rank, peer.device, peer.local_block()),
                   "tsr_tp_attach_local")

    def connect(self, dist) -> None:
        """One process per GPU: exchange the IPC handles through `dist`
        (an initialised torch.distributed module) and map every peer."""
        handles = [None] * self.world
        dist.all_gather_object(handles, self.ipc_handle())
        for r, h in enumerate(handles):
            if r != self.rank:
                self.attach_ipc(r, h)
        dist.barrier()

    def allreduce(self, data_ptr: int, count: int, stream: int) -> None:
        capi.check(self.lib.tsr_tp_allreduce(self.comm, data_ptr, count, stream), "tsr_tp_allreduce")

    def reduce_allreduce(self, partials_ptr: int, split: int, out_ptr: int, count: int, stream: int) -> None:
        """Split-K reduce of `split` regions of `count` floats fused with the all-reduce."""
        capi.check(self.lib.tsr_tp_reduce_allreduce(self.comm, partials_ptr, split, out_ptr, count, stream),
                   "tsr_tp_reduce_allreduce")

    def error_count(self) -> int:
        n = C.c_uint32()
        capi.check(self.lib.tsr_tp_error_count(self.comm, C.byref(n)))
        return n.value

    def close(self) -> None:
        if self.comm:
            self.lib.tsr_tp_destroy(self.comm)
            self.comm = None


FMT_Q4K, FMT_Q6K, FMT_MXFP4, FMT_FP8 = 0, 1, 2, 3
REPLICATED, COLUMN, ROW = 0, 1, 2  # the reference's ParallelKind (include/tessera/types.hpp:29-34)


def slice_shape(fmt: int, kind: int, rows: int, cols: int, rank: int, world: int):
    """(rows, cols, first kept column, bytes) of a rank's slice (tsr_slice_shape)."""
    lib = capi.load_library()
    r, c, c0, b = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
    capi.check(lib.tsr_slice_shape(fmt, kind, rows, cols, rank, world, C.byref(r), C.byref(c), C.byref(c0),
                                   C.byref(b)), "tsr_slice_shape")
    return r.value, c.value, c0.value, b.value


def slice_tensor(fmt: int, kind: int, rows: int, cols: int, rank: int, world: int, src: np.ndarray) -> np.ndarray:
    """A rank's slice of a packed weight tensor (uint8 array), as SliceTensor2D of the reference
    cuts it (src/core/loaders/tensor_slice.cpp:105-159), through the C ABI's tsr_slice_tensor."""
    lib = capi.load_library()
    src = np.ascontiguousarray(src.reshape(-1).view(np.uint8))
    _, _, _, nbytes = slice_shape(fmt, kind, rows, cols, rank, world)
    dst = np.empty(nbytes, dtype=np.uint8)
    capi.check(lib.tsr_slice_tensor(fmt, kind, rows, cols, rank, world, src.ctypes.data, src.nbytes,
                                    dst.ctypes.data, dst.nbytes), "tsr_slice_tensor")
    return dst


def slice_range(fmt: int, rows: int, cols: int, row_begin: int, row_end: int, col_begin: int, col_end: int,
                src: np.ndarray) -> np.ndarray:
    """Rows [row_begin, row_end) and columns [col_begin, col_end) of a packed weight tensor
    (tsr_slice_range): shard maps the kind rule cannot express."""
    lib = capi.load_library()
    src = np.ascontiguousarray(src.reshape(-1).view(np.uint8))
    unit, ubytes = {FMT_Q4K: (256, 144), FMT_Q6K: (256, 210), FMT_MXFP4: (32, 17), FMT_FP8: (1, 1)}[fmt]
    dst = np.empty((row_end - row_begin) * ((col_end - col_begin) // unit) * ubytes, dtype=np.uint8)
    capi.check(lib.tsr_slice_range(fmt, rows, cols, row_begin, row_end, col_begin, col_end, src.ctypes.data,
                                   src.nbytes, dst.ctypes.data, dst.nbytes), "tsr_slice_range")
    return dst


def rank_order_sum(partials):
    """What every rank must end with: ((p0 + p1) + p2) + ... in fp32."""
    acc = np.array(partials[0], dtype=np.float32, copy=True)
    for p in partials[1:]:
        acc = acc + np.asarray(p, dtype=np.float32)
    return acc
