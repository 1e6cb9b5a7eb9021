"""ctypes view of ``include/augur_cuda_nvfp4_sm100.h``.

Loads ``libaugur_nvfp4_sm100.so`` (built in-tree by :mod:`augur_v100_b200.build`)
and declares every exported entry point with the struct layouts of the header.
There is no fallback: if the library cannot be built or loaded, importing the
symbols raises.
"""
from __future__ import annotations

import ctypes
import shutil
from ctypes import POINTER, Structure, c_float, c_int32, c_uint8, c_uint32, c_uint64, c_void_p

from . import build as _build

ABI_VERSION = 1

STATUS_OK = 0
STATUS_INVALID_ARGUMENT = -1
STATUS_UNSUPPORTED_DEVICE = -2
STATUS_OUT_OF_MEMORY = -3
STATUS_RUNTIME_FAILURE = -4
STATUS_SUBMISSION_FAILURE = -5
STATUS_COMPLETION_FAILURE = -6
STATUS_ABI_VERSION_MISMATCH = -7
STATUS_DIAGNOSTIC_FAULT_INJECTED = -8

LAYOUT_COMPACT = 0
LAYOUT_STREAM = 1
LAYOUT_STREAM_PAIR = 2
LAYOUT_TCGEN05 = 3

EPILOGUE_LINEAR_BF16 = 0
EPILOGUE_SWIGLU_BF16 = 1
EPILOGUE_LINEAR_F32 = 2

MAX_SMALL_TOKENS = 8
SCALE_COMPRESSED_TENSORS = 0
SCALE_MODELOPT = 1
STATIC_SCRATCH_BYTES = 4 << 20


class Result(Structure):
    _fields_ = [("status", c_int32), ("raw_cuda_status", c_int32)]


class PlanSnapshot(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32), ("scratch", c_uint64),
                ("scratch_len_bytes", c_uint64), ("sm_count", c_uint32), ("reserved", c_uint32)]


class RepackArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("codes", c_uint64), ("codes_len_bytes", c_uint64),
                ("scales", c_uint64), ("scales_len_bytes", c_uint64),
                ("codes_b", c_uint64), ("codes_b_len_bytes", c_uint64),
                ("scales_b", c_uint64), ("scales_b_len_bytes", c_uint64),
                ("destination", c_uint64), ("destination_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32), ("layout", c_uint32), ("reserved", c_uint32)]


class DequantArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("weight", c_uint64), ("weight_len_bytes", c_uint64),
                ("scales", c_uint64), ("scales_len_bytes", c_uint64),
                ("output_f32", c_uint64), ("output_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32), ("layout", c_uint32),
                ("global_scale", c_float), ("global_scale_b", c_float), ("reserved", c_uint32)]


class GemvArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("weight", c_uint64), ("weight_len_bytes", c_uint64),
                ("input_bf16", c_uint64), ("input_len_bytes", c_uint64),
                ("output", c_uint64), ("output_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32), ("tokens", c_uint32), ("epilogue", c_uint32),
                ("global_scale", c_float), ("global_scale_b", c_float),
                ("stored_rows", c_uint32), ("reserved1", c_uint32)]


class Bf16HeadArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("weight", c_uint64), ("weight_len_bytes", c_uint64),
                ("input", c_uint64), ("input_len_bytes", c_uint64),
                ("output", c_uint64), ("output_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32)]


class TcStep(Structure):
    _fields_ = [(name, c_uint32) for name in ("phase", "job", "tile0", "tiles", "kb0", "kb1", "parts", "slot0", "feeds", "keeps")]


class TcJob(Structure):
    _fields_ = [("phase", c_uint32), ("group0", c_uint32), ("groups", c_uint32)]


class TcProgram(Structure):
    _fields_ = [("steps", c_uint32), ("jobs", c_uint32), ("ctas", c_uint32), ("contributors", c_uint32 * 2),
                ("step", TcStep * 4), ("job", TcJob * 3)]


class MlpArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("gate_up", GemvArgs), ("down", GemvArgs)]


class NormGroupArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("add_a", c_uint64), ("add_b", c_uint64), ("add_len_bytes", c_uint64),
                ("input_f32", c_uint64), ("input_len_bytes", c_uint64),
                ("weight_f32", c_uint64), ("weight_len_bytes", c_uint64),
                ("output_f32", c_uint64), ("output_len_bytes", c_uint64),
                ("staged_bf16", c_uint64), ("staged_len_bytes", c_uint64),
                ("tokens", c_uint32), ("cols", c_uint32), ("epsilon", c_float), ("residual", c_uint32),
                ("count", c_uint32), ("reserved", c_uint32), ("projections", GemvArgs * 4)]


MAX_TP_RANKS = 8


class MlpTpArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("gate_up", GemvArgs), ("down", GemvArgs),
                ("exchange", c_uint64 * MAX_TP_RANKS), ("exchange_len_bytes", c_uint64),
                ("world", c_uint32), ("rank", c_uint32), ("sequence", c_uint32), ("reserved", c_uint32)]


class GemvTpArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("linear", GemvArgs),
                ("exchange", c_uint64 * MAX_TP_RANKS), ("exchange_len_bytes", c_uint64),
                ("world", c_uint32), ("rank", c_uint32), ("sequence", c_uint32), ("reserved", c_uint32)]


class ActQuantArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("input_bf16", c_uint64), ("input_len_bytes", c_uint64),
                ("destination", c_uint64), ("destination_len_bytes", c_uint64),
                ("tokens", c_uint32), ("cols", c_uint32), ("terms", c_uint32), ("global_scale", c_float)]


class GemmArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("weight", c_uint64), ("weight_len_bytes", c_uint64),
                ("activation", c_uint64), ("activation_len_bytes", c_uint64),
                ("output_bf16", c_uint64), ("output_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32), ("tokens", c_uint32), ("activation_terms", c_uint32),
                ("weight_global_scale", c_float), ("activation_global_scale", c_float)]


class GemmSwigluArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("weight", c_uint64), ("weight_len_bytes", c_uint64),
                ("activation", c_uint64), ("activation_len_bytes", c_uint64),
                ("output_bf16", c_uint64), ("output_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32), ("tokens", c_uint32), ("activation_terms", c_uint32),
                ("gate_global_scale", c_float), ("up_global_scale", c_float), ("activation_global_scale", c_float),
                ("reserved", c_uint32)]


class GemmSwigluQuantArgs(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_size", c_uint32),
                ("weight", c_uint64), ("weight_len_bytes", c_uint64),
                ("activation", c_uint64), ("activation_len_bytes", c_uint64),
                ("output_bf16", c_uint64), ("output_len_bytes", c_uint64),
                ("destination", c_uint64), ("destination_len_bytes", c_uint64),
                ("rows", c_uint32), ("cols", c_uint32), ("tokens", c_uint32), ("activation_terms", c_uint32),
                ("gate_global_scale", c_float), ("up_global_scale", c_float), ("activation_global_scale", c_float),
                ("destination_global_scale", c_float), ("destination_terms", c_uint32), ("reserved", c_uint32)]


# Every symbol the header declares: name -> (restype, argtypes).
_U8P = POINTER(c_uint8)
EXPORTS = {
    "augur_cuda_nvfp4_sm100_abi_version": (c_uint32, []),
    "augur_cuda_nvfp4_sm100_build_capability_v1": (c_uint32, []),
    "augur_cuda_nvfp4_sm100_stream_create_v1": (Result, [c_int32, POINTER(c_void_p)]),
    "augur_cuda_nvfp4_sm100_stream_adopt_v1": (Result, [c_int32, c_void_p, POINTER(c_void_p)]),
    "augur_cuda_nvfp4_sm100_stream_synchronize_v1": (Result, [c_void_p]),
    "augur_cuda_nvfp4_sm100_stream_destroy_v1": (Result, [c_void_p]),
    "augur_cuda_nvfp4_sm100_gemv_scratch_extent_host_v1": (Result, [c_uint32, c_uint32, c_uint32, POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_gemm_scratch_extent_host_v1": (Result, [c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_gemm_plan_scratch_extent_host_v1": (Result, [c_uint32, POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_plan_create_v1": (Result, [c_int32, c_void_p, c_uint64, POINTER(c_void_p)]),
    "augur_cuda_nvfp4_sm100_plan_describe_v1": (Result, [c_void_p, POINTER(PlanSnapshot)]),
    "augur_cuda_nvfp4_sm100_plan_destroy_v1": (Result, [c_void_p]),
    "augur_cuda_nvfp4_sm100_repack_extent_host_v1": (Result, [c_uint32, c_uint32, c_uint32, POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_repack_host_v1": (Result, [c_uint32, c_uint32, c_uint32, _U8P, _U8P, _U8P, _U8P, _U8P, c_uint64]),
    "augur_cuda_nvfp4_sm100_unpack_host_v1": (Result, [c_uint32, c_uint32, c_uint32, _U8P, c_uint64, _U8P, _U8P, _U8P, _U8P]),
    "augur_cuda_nvfp4_sm100_checkpoint_global_scale_host_v1": (Result, [c_uint32, c_float, POINTER(c_float)]),
    "augur_cuda_nvfp4_sm100_checkpoint_validate_host_v1": (Result, [c_uint64, c_uint64, _U8P, c_uint64, _U8P, c_uint64]),
    "augur_cuda_nvfp4_sm100_planes_to_ggml36_host_v1": (Result, [c_uint64, c_uint64, _U8P, _U8P, _U8P, c_uint64]),
    "augur_cuda_nvfp4_sm100_ggml36_to_planes_host_v1": (Result, [c_uint64, c_uint64, _U8P, c_uint64, _U8P, _U8P]),
    "augur_cuda_nvfp4_sm100_repack_preflight_v1": (Result, [c_int32, c_void_p, POINTER(RepackArgs)]),
    "augur_cuda_nvfp4_sm100_repack_prevalidated_submit_v1": (Result, [c_int32, c_void_p, POINTER(RepackArgs)]),
    "augur_cuda_nvfp4_sm100_dequant_f32_preflight_v1": (Result, [c_int32, c_void_p, POINTER(DequantArgs)]),
    "augur_cuda_nvfp4_sm100_dequant_f32_prevalidated_submit_v1": (Result, [c_int32, c_void_p, POINTER(DequantArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemvArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemvArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_tc_scratch_extent_host_v1": (Result, [c_uint32, c_uint32, c_uint32, POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_tc_program_describe_host_v1": (Result, [c_uint32, c_uint32, c_uint32, c_uint32, c_uint32, c_uint32,
                                                                     POINTER(TcProgram)]),
    "augur_cuda_nvfp4_sm100_gemv_tc_bf16_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemvArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_tc_bf16_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemvArgs)]),
    "augur_cuda_nvfp4_sm100_mlp_tc_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(MlpArgs)]),
    "augur_cuda_nvfp4_sm100_mlp_tc_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(MlpArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1": (Result, [c_int32, c_void_p, POINTER(GemvArgs)]),
    "augur_cuda_nvfp4_sm100_static_scratch_status_v1": (Result, [c_int32, c_void_p, POINTER(c_uint32)]),
    "augur_cuda_nvfp4_sm100_bf16_head_preflight_v1": (Result, [c_int32, c_void_p, POINTER(Bf16HeadArgs)]),
    "augur_cuda_nvfp4_sm100_bf16_head_prevalidated_submit_v1": (Result, [c_int32, c_void_p, POINTER(Bf16HeadArgs)]),
    "augur_cuda_nvfp4_sm100_mlp_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(MlpArgs)]),
    "augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(MlpArgs)]),
    "augur_cuda_nvfp4_sm100_norm_group_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(NormGroupArgs)]),
    "augur_cuda_nvfp4_sm100_norm_group_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(NormGroupArgs)]),
    "augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1": (Result, [c_uint32, c_uint32, POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_mlp_tp_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(MlpTpArgs)]),
    "augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(MlpTpArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_tp_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemvTpArgs)]),
    "augur_cuda_nvfp4_sm100_gemv_tp_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemvTpArgs)]),
    "augur_cuda_nvfp4_sm100_act_quant_preflight_v1": (Result, [c_int32, c_void_p, POINTER(ActQuantArgs)]),
    "augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1": (Result, [c_int32, c_void_p, POINTER(ActQuantArgs)]),
    "augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemmArgs)]),
    "augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemmArgs)]),
    "augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemmSwigluArgs)]),
    "augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemmSwigluArgs)]),
    "augur_cuda_nvfp4_sm100_gemm_swiglu_quant_preflight_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemmSwigluQuantArgs)]),
    "augur_cuda_nvfp4_sm100_gemm_swiglu_quant_prevalidated_submit_v1": (Result, [c_int32, c_void_p, c_void_p, POINTER(GemmSwigluQuantArgs)]),
    "augur_cuda_nvfp4_sm100_interleave_gate_up_host_v1": (Result, [c_uint32, c_uint32, _U8P, _U8P, _U8P, _U8P, _U8P, _U8P]),
    "augur_cuda_nvfp4_sm100_diagnostic_inject_submit_fault_v1": (None, [c_uint32]),
    "augur_cuda_nvfp4_sm100_allocation_snapshot_v1": (None, [POINTER(c_uint64), POINTER(c_uint64)]),
    "augur_cuda_nvfp4_sm100_launch_count_v1": (c_uint64, []),
    "augur_cuda_nvfp4_sm100_plan_device_status_v1": (Result, [c_void_p, POINTER(c_uint32)]),
}

_lib = None


def library_path():
    """Path of the shared library, (re)building it when nvcc is present and sources are newer."""
    if _build.is_stale():
        if shutil.which("nvcc") is None and not _build.LIB.exists():
            raise RuntimeError(
                "libaugur_nvfp4_sm100.so is missing and nvcc is not available to build it; "
                "this package has no other execution path")
        if shutil.which("nvcc") is not None:
            _build.build()
    return _build.LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        handle = ctypes.CDLL(str(library_path()))
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(handle, name)  # AttributeError if the header and the library disagree
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def header(struct_type):
    """A zeroed args struct with abi_version / struct_size filled in."""
    value = struct_type()
    value.abi_version = ABI_VERSION
    value.struct_size = ctypes.sizeof(struct_type)
    return value
