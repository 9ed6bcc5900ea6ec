"""ctypes binding of the C ABI declared in ``include/tessera_b200.h``.

Loading fails loudly when the library has not been built
(``python -c "import __graft_entry__ as g; g.build()"`` or
``make -C tessera_b200/csrc``); nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import enum
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


class StatusCode(enum.IntEnum):
    """Values of ``tessera::StatusCode`` (include/tessera/types.hpp:38-48)."""

    Ok = 0
    InvalidArgument = 1
    FileNotFound = 2
    MalformedFile = 3
    UnsupportedFeature = 4
    OutOfMemory = 5
    DeviceError = 6
    NonFinite = 7
    NetworkError = 8


class StatusError(RuntimeError):
    """A non-Ok status from the library (the ``std::unexpected`` of the reference)."""

    def __init__(self, code: int, what: str = ""):
        self.code = StatusCode(code)
        super().__init__(f"{self.code.name}{': ' + what if what else ''}")


def library_path() -> str:
    """The built library beside this package, or the file TESSERA_B200_LIBRARY names."""
    return os.environ.get("TESSERA_B200_LIBRARY") or os.path.join(_HERE, "lib", "libtessera_b200.so")


_lib = None


class LaunchDesc(C.Structure):
    """tsr_launch_desc of include/tessera_b200.h."""

    _fields_ = [("kernel", C.c_int32), ("grid", C.c_uint32 * 3), ("block", C.c_uint32 * 3),
                ("n_buffers", C.c_int32), ("n_scalars", C.c_int32),
                ("buffers", C.POINTER(C.c_void_p)), ("buffer_bytes", C.POINTER(C.c_size_t)),
                ("scalars", C.POINTER(C.c_uint64))]


_u64 = C.c_uint64
_vp = C.c_void_p
_sz = C.c_size_t

# name -> (restype, argtypes); every symbol declared in include/tessera_b200.h
SIGNATURES = {
    "tsr_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "tsr_device_name": (C.c_int, [C.c_int, C.c_char_p, _sz]),
    "tsr_create": (C.c_int, [C.c_int, C.POINTER(_vp)]),
    "tsr_create_on_stream": (C.c_int, [C.c_int, _vp, C.POINTER(_vp)]),
    "tsr_destroy": (None, [_vp]),
    "tsr_context_device": (C.c_int, [_vp]),
    "tsr_context_stream": (_vp, [_vp]),
    "tsr_memory_info": (C.c_int, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "tsr_last_error": (C.c_char_p, [_vp]),
    "tsr_alloc": (C.c_int, [_vp, _sz, C.c_int, C.POINTER(_vp), C.POINTER(_vp)]),
    "tsr_free": (C.c_int, [_vp, C.c_int, _vp]),
    "tsr_copy_h2d": (C.c_int, [_vp, _vp, _sz, _vp, _sz]),
    "tsr_copy_d2h": (C.c_int, [_vp, _vp, _sz, _vp, _sz]),
    "tsr_copy_d2d": (C.c_int, [_vp, _vp, _sz, _vp, _sz, _sz]),
    "tsr_copy_peer": (C.c_int, [_vp, _vp, C.c_int, _vp, _sz]),
    "tsr_synchronize": (C.c_int, [_vp]),
    "tsr_kernel_count": (C.c_int, []),
    "tsr_kernel_name": (C.c_char_p, [C.c_int]),
    "tsr_kernel_lookup": (C.c_int, [C.c_char_p]),
    "tsr_launch": (C.c_int, [_vp, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                             C.POINTER(_vp), C.POINTER(_sz), C.c_int, C.POINTER(_u64), C.c_int]),
    "tsr_launch_many": (C.c_int, [_vp, C.POINTER(LaunchDesc), _sz, C.POINTER(_sz)]),
    "tsr_set_deferred": (C.c_int, [_vp, C.c_int]),
    "tsr_flush": (C.c_int, [_vp]),
    "tsr_launch_stats": (C.c_int, [_vp, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)]),
    "tsr_gemv_group": (C.c_int, [_vp, C.c_int, _vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_u64), C.c_int,
                                 _u64, _u64]),
    "tsr_tp_bind": (C.c_int, [_vp, _vp]),
    "tsr_gemm_q4k": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "tsr_gemm_q6k": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "tsr_gemm_vec_reduce": (C.c_int, [_vp, _vp, _u64, _u64, _vp]),
    "tsr_gemm_mxfp4": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "tsr_gemm_fp8": (C.c_int, [_vp, _vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "tsr_gemm_mxfp4_w4a8": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "tsr_mxfp4_row_ref": (C.c_int, [_vp, _vp, _u64, _u64, _vp]),
    "tsr_quantize_fp8": (C.c_int, [_vp, _vp, _u64, _u64, _vp]),
    "tsr_quantize_fp8_pack": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _vp]),
    "tsr_round_bf16": (C.c_int, [_vp, _u64, _vp]),
    "tsr_add": (C.c_int, [_vp, _vp, _vp, _u64, _vp]),
    "tsr_fill": (C.c_int, [_vp, C.c_int32, _u64, _vp]),
    "tsr_silu_mul": (C.c_int, [_vp, _vp, _vp, _u64, _vp]),
    "tsr_sigmoid_gate": (C.c_int, [_vp, _vp, _vp, _u64, _vp]),
    "tsr_conv1d_state": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, _u64, _u64, _vp]),
    "tsr_top_k_rows": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "tsr_gemm_dense": (C.c_int, [C.c_int, _vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "tsr_rope": (C.c_int, [_vp, _u64, _u64, _u64, _u64, _u64, C.c_float, _vp]),
    "tsr_quantize_rows": (C.c_int, [C.c_int, _vp, _vp, _vp, _u64, _u64, _vp]),
    "tsr_attention": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, _vp] + [_u64] * 9 + [_vp]),
    "tsr_attention_split": (C.c_int, [C.c_int] + [_vp] * 8 + [_u64] * 9 + [_vp]),
    "tsr_attention_combine": (C.c_int, [_vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "tsr_mrope": (C.c_int, [_vp, _vp, _u64, _u64, _u64, _u64, C.c_float, _u64, _u64, _u64, _vp]),
    "tsr_cast_f32_f16": (C.c_int, [_vp, _vp, _u64, _vp]),
    "tsr_delta_step_heads": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, _u64, _u64, _u64, _vp]),
    "tsr_embedding": (C.c_int, [C.c_int, _vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "tsr_l2norm": (C.c_int, [_vp, _vp, _u64, _u64, C.c_float, C.c_float, _vp]),
    "tsr_rmsnorm_gated": (C.c_int, [_vp, _vp, _vp, _vp, _u64, _u64, C.c_float, _u64, _u64, _vp]),
    "tsr_ssm_gate": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _vp]),
    "tsr_qgate_split": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "tsr_repeat_heads": (C.c_int, [_vp, _vp, _u64, _u64, _u64, _u64, _vp]),
    "tsr_moe_gate": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u64, _u64, _vp]),
    "tsr_moe_scale_add": (C.c_int, [_vp, _vp, _vp, _vp, _u64, _u64, _vp]),
    "tsr_moe_experts_gate_up_q4k": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, _u64, _u64, _vp]),
    "tsr_moe_experts_down": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, _u64, _u64, _vp]),
    "tsr_rmsnorm": (C.c_int, [_vp, _vp, _vp, _u64, _u64, C.c_float, _vp]),
    "tsr_dequantize": (C.c_int, [C.c_int, _vp, _vp, _vp, _u64, _u64, _vp]),
    "tsr_slice_shape": (C.c_int, [C.c_int, C.c_int, _u64, _u64, C.c_int, C.c_int, C.POINTER(_u64), C.POINTER(_u64),
                                  C.POINTER(_u64), C.POINTER(_u64)]),
    "tsr_slice_range": (C.c_int, [C.c_int, _u64, _u64, _u64, _u64, _u64, _u64, _vp, _sz, _vp, _sz]),
    "tsr_slice_tensor": (C.c_int, [C.c_int, C.c_int, _u64, _u64, C.c_int, C.c_int, _vp, _sz, _vp, _sz]),
    "tsr_gemm_q4k_noalloc_max_outputs": (_u64, []),
    "tsr_gemm_q4k_noalloc": (C.c_int, [_vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "tsr_tp_create": (C.c_int, [C.c_int, C.c_int, C.c_int, _u64, C.POINTER(_vp)]),
    "tsr_tp_destroy": (None, [_vp]),
    "tsr_tp_local_block": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_u64)]),
    "tsr_tp_ipc_handle": (C.c_int, [_vp, _vp]),
    "tsr_tp_attach_ipc": (C.c_int, [_vp, C.c_int, _vp]),
    "tsr_tp_attach_local": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "tsr_tp_allreduce": (C.c_int, [_vp, _vp, _u64, _vp]),
    "tsr_tp_reduce_allreduce": (C.c_int, [_vp, _vp, _u64, _vp, _u64, _vp]),
    "tsr_tp_error_count": (C.c_int, [_vp, C.POINTER(C.c_uint32)]),
}


def load_library():
    """Load the shared library once and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `make -C tessera_b200/csrc` "
            "(there is no CPU fallback)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str = "") -> None:
    if code != 0:
        raise StatusError(code, what)
