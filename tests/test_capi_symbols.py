"""The C-ABI library loads and exports everything include/tessera_b200.h declares."""
import ctypes as C
import os
import re

import pytest

from tessera_b200 import capi
from tessera_b200.backend import CreateBackend, KernelLaunch, ListGpuNames, ValidateLaunch
from tessera_b200.capi import StatusCode, StatusError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

REQUIRED_IDS = [
    "gemm_q4k_vec", "gemm_q6k_vec", "gemm_vec_reduce",
    "gemm_q4k_rows2", "gemm_q4k_rows3", "gemm_q4k_rows4", "gemm_q4k_rows5",
    "gemm_q6k_rows2", "gemm_q6k_rows3", "gemm_q6k_rows4", "gemm_q6k_rows5",
    "gemm_q4k_batched", "gemm_q6k_batched", "gemm_q4k_wmma", "gemm_q6k_wmma",
    "gemm_mxfp4", "gemm_mxfp4_rows", "gemm_mxfp4_batched", "gemm_mxfp4_wmma",
    "gemm_mxfp4_wmma_reduce", "mxfp4_row_ref", "gemm_fp8", "quantize_fp8",
    "quantize_fp8_pack", "quantize_fp8_pack_rows", "round_bf16", "add", "fill",
    # every other id the reference's Qwen3.5 decode loads (src/models/qwen3_5/trunk.cpp:150-215,486-530,
    # src/core/decode_device.cpp:170-210 of the reference)
    "rmsnorm", "silu_mul", "sigmoid_gate", "qgate_split", "mrope", "rope", "repeat_heads", "l2norm", "ssm_gate",
    "delta_step_heads", "rmsnorm_gated", "conv1d_state", "cast_f32_f16", "quantize_q8", "quantize_q4",
    "attention", "attention_q8", "attention_q4", "attention_fp8", "attention_split", "attention_split_gqa",
    "attention_q8_split", "attention_q4_split", "attention_fp8_split", "attention_combine", "top_k_rows",
    "embedding_f32", "embedding_bf16", "embedding_q4k", "gemm_f32", "gemm_f32_batched", "gemm_bf16",
    "gemm_bf16_batched", "gemm_bf16_wmma", "moe_gate", "moe_scale_add", "moe_experts_gate_up_q4k",
    "moe_experts_down_q4k", "moe_experts_down_q6k",
]


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tessera_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsr_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = capi.load_library()
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), f"{name} is declared but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(capi.SIGNATURES) == names


def test_kernel_table_has_the_projection_ids():
    lib = capi.load_library()
    ids = [lib.tsr_kernel_name(i).decode() for i in range(lib.tsr_kernel_count())]
    for name in REQUIRED_IDS:
        assert lib.tsr_kernel_lookup(name.encode()) == ids.index(name)
    assert lib.tsr_kernel_lookup(b"layernorm") == -1
    assert lib.tsr_kernel_name(-1) is None


def test_validate_launch_rules():
    assert ValidateLaunch(KernelLaunch()) == StatusCode.Ok
    assert ValidateLaunch(KernelLaunch(grid_y=0)) == StatusCode.InvalidArgument
    assert ValidateLaunch(KernelLaunch(block_x=0)) == StatusCode.InvalidArgument
    assert ValidateLaunch(KernelLaunch(scalars=[0] * 17)) == StatusCode.InvalidArgument


def test_argument_errors_need_no_device():
    lib = capi.load_library()
    assert lib.tsr_gemm_q4k(None, None, None, 1, 8, 256, 1, None) == StatusCode.InvalidArgument
    assert lib.tsr_create(0, None) == StatusCode.InvalidArgument
    assert lib.tsr_launch(None, 0, None, None, None, None, 0, None, 0) == StatusCode.InvalidArgument


def test_no_silent_cpu_fallback_without_a_device():
    lib = capi.load_library()
    count = C.c_int()
    lib.tsr_device_count(C.byref(count))
    if count.value > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(StatusError) as e:
        ListGpuNames()
    assert e.value.code == StatusCode.DeviceError
    b = CreateBackend()
    with pytest.raises(StatusError) as e:
        b.Init()
    assert e.value.code == StatusCode.DeviceError
    with pytest.raises(StatusError):
        b.AllocateBuffer(16)
