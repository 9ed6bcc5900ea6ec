"""Host-side mirror of the reference's ``tessera::Backend`` interface.

Same names, argument meaning and error behaviour as
``include/tessera/backend.hpp:847-1037`` of the reference, implemented over the
C ABI; a non-Ok status is raised as :class:`StatusError` where the reference
returns ``std::unexpected``.  The C++ twin that plugs into the reference's
engine is ``tessera_b200/backend/cuda_backend.cpp``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import capi
from .capi import StatusCode, StatusError

DEVICE = 0        # MemoryKind::Device
HOST_VISIBLE = 1  # MemoryKind::HostVisible

K_MAX_BOUND_BUFFERS = 16  # kMaxBoundBuffers, backend.hpp:47
K_MAX_SCALARS = 16        # kMaxScalars, backend.hpp:48


@dataclass
class KernelLaunch:
    """backend.hpp:56-67: buffers bind first, then 64-bit scalars."""

    grid_x: int = 1
    grid_y: int = 1
    grid_z: int = 1
    block_x: int = 256
    block_y: int = 1
    block_z: int = 1
    buffers: List["Buffer"] = field(default_factory=list)
    scalars: List[int] = field(default_factory=list)


def ValidateLaunch(launch: KernelLaunch) -> StatusCode:
    """backend.hpp:138-148."""
    axes = (launch.grid_x, launch.grid_y, launch.grid_z,
            launch.block_x, launch.block_y, launch.block_z)
    if any(a == 0 for a in axes):
        return StatusCode.InvalidArgument
    if len(launch.buffers) > K_MAX_BOUND_BUFFERS or len(launch.scalars) > K_MAX_SCALARS:
        return StatusCode.InvalidArgument
    return StatusCode.Ok


class Buffer:
    """RAII device buffer (backend.hpp:72-103); freed through its owner."""

    def __init__(self, backend: "CudaBackend", handle: int, size: int, kind: int, host_map):
        self._backend, self._handle, self._size, self._kind = backend, handle, size, kind
        self._host_map = host_map

    def Size(self) -> int:
        return self._size

    def Kind(self) -> int:
        return self._kind

    def Handle(self) -> int:
        return self._handle

    def HostMap(self):
        return self._host_map

    def Owner(self) -> "CudaBackend":
        return self._backend

    def release(self) -> None:
        if self._handle and self._backend is not None:
            self._backend.FreeBuffer(self._kind, self._handle)
        self._handle = 0

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class Kernel:
    """backend.hpp:114-134."""

    def __init__(self, backend: "CudaBackend", handle: int, name: str):
        self._backend, self._handle, self._id = backend, handle, name

    def Id(self) -> str:
        return self._id

    def Handle(self) -> int:
        return self._handle

    def Owner(self) -> "CudaBackend":
        return self._backend


class CudaBackend:
    """One instance per device; all work is ordered on one stream."""

    def __init__(self, stream: Optional[int] = None):
        self._lib = capi.load_library()
        self._ctx = None
        self._device_index = 0
        self._stream_arg = stream
        self._device_name = ""

    # -- identity ---------------------------------------------------------
    def Name(self) -> str:
        return "cuda"

    def DeviceName(self) -> str:
        return self._device_name

    def SetDeviceIndex(self, index: int) -> None:
        self._device_index = index

    def DeviceIndex(self) -> int:
        return self._device_index

    def Init(self) -> None:
        """Idempotent; InvalidArgument for an out-of-range device index."""
        if self._ctx is not None:
            return
        ctx = C.c_void_p()
        if self._stream_arg is None:
            code = self._lib.tsr_create(self._device_index, C.byref(ctx))
        else:
            code = self._lib.tsr_create_on_stream(self._device_index, self._stream_arg, C.byref(ctx))
        capi.check(code, "Init")
        self._ctx = ctx
        name = C.create_string_buffer(256)
        self._lib.tsr_device_name(self._device_index, name, 256)
        self._device_name = name.value.decode()

    def close(self) -> None:
        if self._ctx is not None:
            self._lib.tsr_destroy(self._ctx)
            self._ctx = None

    def _need(self):
        if self._ctx is None:
            raise StatusError(StatusCode.DeviceError, "Init() not called")
        return self._ctx

    def stream(self) -> int:
        return self._lib.tsr_context_stream(self._need()) or 0

    def MemoryInfo(self):
        total, free = C.c_uint64(), C.c_uint64()
        self._check(self._lib.tsr_memory_info(self._need(), C.byref(total), C.byref(free)))
        return total.value, free.value

    def _check(self, code: int) -> None:
        if code != 0:
            what = self._lib.tsr_last_error(self._ctx).decode() if self._ctx else ""
            raise StatusError(code, what)

    # -- buffers ----------------------------------------------------------
    def AllocateBuffer(self, nbytes: int, kind: int = DEVICE) -> Buffer:
        if nbytes == 0:
            raise StatusError(StatusCode.InvalidArgument, "0 bytes")
        handle, host = C.c_void_p(), C.c_void_p()
        self._check(self._lib.tsr_alloc(self._need(), nbytes, kind, C.byref(handle), C.byref(host)))
        return Buffer(self, handle.value, nbytes, kind, host.value)

    def FreeBuffer(self, kind: int, handle: int) -> None:
        if self._ctx is not None and handle:
            self._lib.tsr_free(self._ctx, kind, handle)

    @staticmethod
    def _host(arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        return arr, arr.ctypes.data, arr.nbytes

    def CopyH2D(self, dst: Buffer, src: np.ndarray) -> None:
        self.CopyH2DAt(dst, 0, src)

    def CopyH2DAt(self, dst: Buffer, offset: int, src: np.ndarray) -> None:
        arr, ptr, n = self._host(src)
        if offset > dst.Size() or n > dst.Size() - offset:
            raise StatusError(StatusCode.InvalidArgument, "h2d out of range")
        self._check(self._lib.tsr_copy_h2d(self._need(), dst.Handle(), offset, ptr, n))

    def CopyD2H(self, src: Buffer, dst: np.ndarray, nbytes: Optional[int] = None) -> None:
        self.CopyD2HAt(src, 0, dst, nbytes)

    def CopyD2HAt(self, src: Buffer, offset: int, dst: np.ndarray, nbytes: Optional[int] = None) -> None:
        assert dst.flags["C_CONTIGUOUS"]
        n = dst.nbytes if nbytes is None else nbytes
        if offset > src.Size() or n > src.Size() - offset or n > dst.nbytes:
            raise StatusError(StatusCode.InvalidArgument, "d2h out of range")
        self._check(self._lib.tsr_copy_d2h(self._need(), src.Handle(), offset, dst.ctypes.data, n))

    def CopyD2D(self, src: Buffer, src_offset: int, dst: Buffer, dst_offset: int, nbytes: int) -> None:
        if (src_offset > src.Size() or nbytes > src.Size() - src_offset or
                dst_offset > dst.Size() or nbytes > dst.Size() - dst_offset):
            raise StatusError(StatusCode.InvalidArgument, "d2d out of range")
        self._check(self._lib.tsr_copy_d2d(self._need(), src.Handle(), src_offset, dst.Handle(),
                                           dst_offset, nbytes))

    def CopyPeerFrom(self, dst: Buffer, src: Buffer, nbytes: int) -> None:
        if nbytes > dst.Size() or nbytes > src.Size():
            raise StatusError(StatusCode.InvalidArgument, "peer copy out of range")
        src.Owner().Synchronize()
        self._check(self._lib.tsr_copy_peer(self._need(), dst.Handle(), src.Owner().DeviceIndex(),
                                            src.Handle(), nbytes))

    # -- kernels ----------------------------------------------------------
    def LoadKernel(self, name: str, code: bytes = b"") -> Kernel:
        """Built-ins only: non-empty code or an unknown name is UnsupportedFeature."""
        if code:
            raise StatusError(StatusCode.UnsupportedFeature, "compiled kernel modules")
        index = self._lib.tsr_kernel_lookup(name.encode())
        if index < 0:
            raise StatusError(StatusCode.UnsupportedFeature, f"kernel '{name}'")
        return Kernel(self, index + 1, name)

    def LaunchKernel(self, kernel: Kernel, launch: KernelLaunch) -> None:
        invalid = ValidateLaunch(launch)
        if invalid != StatusCode.Ok:
            raise StatusError(invalid, "ValidateLaunch")
        nb, ns = len(launch.buffers), len(launch.scalars)
        if any(b is None for b in launch.buffers):
            raise StatusError(StatusCode.InvalidArgument, "null buffer")
        bufs = (C.c_void_p * max(nb, 1))(*[b.Handle() for b in launch.buffers])
        sizes = (C.c_size_t * max(nb, 1))(*[b.Size() for b in launch.buffers])
        scal = (C.c_uint64 * max(ns, 1))(*[int(s) & 0xFFFFFFFFFFFFFFFF for s in launch.scalars])
        grid = (C.c_uint32 * 3)(launch.grid_x, launch.grid_y, launch.grid_z)
        block = (C.c_uint32 * 3)(launch.block_x, launch.block_y, launch.block_z)
        self._check(self._lib.tsr_launch(self._need(), kernel.Handle() - 1, grid, block, bufs, sizes,
                                         nb, scal, ns))

    def Synchronize(self) -> None:
        self._check(self._lib.tsr_synchronize(self._need()))

    # -- deferred submission and tensor parallelism (no reference counterpart) --
    def SetDeferred(self, mode: int) -> None:
        """0: every LaunchKernel is issued at once; 1: launches queue until the next copy or
        synchronisation, are merged where the kernels allow it, and a repeating queue is
        replayed as a CUDA graph; 2: as 1 without graphs; 3: as 1 without running silu_mul,
        rmsnorm and add inside the projection launches."""
        self._check(self._lib.tsr_set_deferred(self._need(), mode))

    def Flush(self) -> None:
        self._check(self._lib.tsr_flush(self._need()))

    def LaunchStats(self):
        """(LaunchKernel calls accepted, kernels they became on the device, CUDA graph launches)."""
        a, d, g = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._check(self._lib.tsr_launch_stats(self._need(), C.byref(a), C.byref(d), C.byref(g)))
        return a.value, d.value, g.value

    def BindTensorParallel(self, comm) -> None:
        """Makes `comm` (a tessera_b200.tp.TpComm, or None) the communicator of the
        gemm_*_vec_allreduce and allreduce_sum kernel ids."""
        self._check(self._lib.tsr_tp_bind(self._need(), comm.comm if comm is not None else None))

    def LaunchMany(self, batch: "LaunchBatch") -> None:
        """Submits a pre-marshalled list of launches (same checks as LaunchKernel)."""
        descs, count = batch.descriptors()
        if count:
            self._check(self._lib.tsr_launch_many(self._need(), descs, count, None))

    # -- conveniences for tests and the benchmark ---------------------------
    def upload(self, arr: np.ndarray) -> Buffer:
        buf = self.AllocateBuffer(max(arr.nbytes, 1))
        self.CopyH2D(buf, arr)
        return buf

    def download(self, buf: Buffer, dtype, count: int, offset: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        self.CopyD2HAt(buf, offset, out)
        return out


class LaunchBatch:
    """ctypes arguments of a fixed sequence of launches, built once: a decode loop issues the
    same launches every token, and marshalling them in Python each time would cost more than
    the launches themselves (the C++ backend has no such cost)."""

    def __init__(self):
        self.items = []
        self._keep = []
        self._descs = None

    def add(self, kernel: Kernel, launch: KernelLaunch) -> None:
        invalid = ValidateLaunch(launch)
        if invalid != StatusCode.Ok:
            raise StatusError(invalid, "ValidateLaunch")
        nb, ns = len(launch.buffers), len(launch.scalars)
        bufs = (C.c_void_p * max(nb, 1))(*[b.Handle() for b in launch.buffers])
        sizes = (C.c_size_t * max(nb, 1))(*[b.Size() for b in launch.buffers])
        scal = (C.c_uint64 * max(ns, 1))(*[int(s) & 0xFFFFFFFFFFFFFFFF for s in launch.scalars])
        grid = (C.c_uint32 * 3)(launch.grid_x, launch.grid_y, launch.grid_z)
        block = (C.c_uint32 * 3)(launch.block_x, launch.block_y, launch.block_z)
        self._keep.append(list(launch.buffers))
        self.items.append((kernel.Handle() - 1, grid, block, bufs, sizes, nb, scal, ns))
        self._descs = None

    def descriptors(self):
        """(array of tsr_launch_desc, count) for tsr_launch_many."""
        if self._descs is None:
            arr = (capi.LaunchDesc * max(len(self.items), 1))()
            for d, (kernel, grid, block, bufs, sizes, nb, scal, ns) in zip(arr, self.items):
                d.kernel = kernel
                d.grid[:] = list(grid)
                d.block[:] = list(block)
                d.n_buffers, d.n_scalars = nb, ns
                d.buffers = C.cast(bufs, C.POINTER(C.c_void_p))
                d.buffer_bytes = C.cast(sizes, C.POINTER(C.c_size_t))
                d.scalars = C.cast(scal, C.POINTER(C.c_uint64))
            self._descs = arr
        return self._descs, len(self.items)

    def __len__(self):
        return len(self.items)


def CreateBackend(stream: Optional[int] = None) -> CudaBackend:
    """backend.hpp:1062-1064."""
    return CudaBackend(stream)


def ListGpuNames() -> Sequence[str]:
    """backend.hpp:1066-1071: DeviceError when no GPU is visible."""
    lib = capi.load_library()
    count = C.c_int()
    code = lib.tsr_device_count(C.byref(count))
    if code != 0 or count.value == 0:
        raise StatusError(StatusCode.DeviceError, "no CUDA device")
    names = []
    for i in range(count.value):
        buf = C.create_string_buffer(256)
        capi.check(lib.tsr_device_name(i, buf, 256))
        names.append(buf.value.decode())
    return names
