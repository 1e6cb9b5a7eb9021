"""Host-side owners and checked bindings over the C ABI, for Python callers.

The classes mirror the reference's safe wrappers in crates/augur-backend:
owners of device resources (``cuda_runtime.rs``: OwnedCudaStream / OwnedCudaBuffer),
an uploaded-and-repacked weight (``cuda_qwen35_qpn.rs:97-131``,
``OwnedCudaQwen35QpnWeightV1::upload_checkpoint_nvfp4``), a retained projection
that is preflighted once and then only submitted
(``cuda_qwen35_prefill_cublas/qpn.rs:60-105``) and the FFN program
(``qpn.rs:391-492``, ``CudaQwen35QpnFfnProgramV1``). torch is used for device
memory and stream plumbing only; every computation goes through the C ABI.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_uint32, c_uint64, c_void_p

import numpy as np
import torch

from . import abi


class CudaRuntimeError(RuntimeError):
    """A non-OK ``augur_cuda_result_v1`` (crates/augur-backend/src/cuda_runtime.rs CudaRuntimeError)."""

    def __init__(self, where: str, status: int, raw: int):
        super().__init__(f"{where}: status {status}, cuda {raw}")
        self.where, self.status, self.raw = where, status, raw


def _check(where: str, result: abi.Result) -> None:
    if result.status != abi.STATUS_OK:
        raise CudaRuntimeError(where, result.status, result.raw_cuda_status)


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


class Stream:
    """An ABI stream handle wrapping a torch CUDA stream (the current one by default)."""

    def __init__(self, device: int | None = None, torch_stream: torch.cuda.Stream | None = None):
        self.ordinal = torch.cuda.current_device() if device is None else int(device)
        self.torch_stream = torch_stream or torch.cuda.current_stream(self.ordinal)
        self.handle = c_void_p()
        _check("stream_adopt", abi.lib().augur_cuda_nvfp4_sm100_stream_adopt_v1(
            self.ordinal, c_void_p(self.torch_stream.cuda_stream), byref(self.handle)))

    def synchronize(self) -> None:
        _check("stream_synchronize", abi.lib().augur_cuda_nvfp4_sm100_stream_synchronize_v1(self.handle))

    def close(self) -> None:
        if self.handle:
            abi.lib().augur_cuda_nvfp4_sm100_stream_destroy_v1(self.handle)
            self.handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Plan:
    """Stream-owned scratch (split-K partials, arrival counters, activation staging)."""

    def __init__(self, stream: Stream, scratch_bytes: int):
        self.stream = stream
        self.handle = c_void_p()
        _check("plan_create", abi.lib().augur_cuda_nvfp4_sm100_plan_create_v1(
            stream.ordinal, stream.handle, c_uint64(scratch_bytes), byref(self.handle)))

    def snapshot(self) -> abi.PlanSnapshot:
        snap = abi.header(abi.PlanSnapshot)
        _check("plan_describe", abi.lib().augur_cuda_nvfp4_sm100_plan_describe_v1(self.handle, byref(snap)))
        return snap

    def device_status(self) -> int:
        word = c_uint32()
        _check("plan_device_status", abi.lib().augur_cuda_nvfp4_sm100_plan_device_status_v1(self.handle, byref(word)))
        return int(word.value)

    def close(self) -> None:
        if self.handle:
            abi.lib().augur_cuda_nvfp4_sm100_plan_destroy_v1(self.handle)
            self.handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gemv_scratch_bytes(rows: int, cols: int, tokens: int = 8) -> int:
    out = c_uint64()
    _check("gemv_scratch_extent", abi.lib().augur_cuda_nvfp4_sm100_gemv_scratch_extent_host_v1(
        rows, cols, tokens, byref(out)))
    return int(out.value)


def gemm_plan_scratch_bytes(sm_count: int = 0) -> int:
    """Plan scratch with which the prefill GEMM can cut its leftover tiles along k (0: this device's SM count)."""
    if not sm_count:
        import torch
        sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    out = c_uint64(0)
    _check("gemm_plan_scratch_extent", abi.lib().augur_cuda_nvfp4_sm100_gemm_plan_scratch_extent_host_v1(sm_count, byref(out)))
    return out.value


def gemm_scratch_bytes(rows: int, cols: int, tokens: int, terms: int) -> int:
    """Bytes of the staged (quantised) activations of a prefill linear: whole 128-row tiles per term."""
    out = c_uint64()
    _check("gemm_scratch_extent", abi.lib().augur_cuda_nvfp4_sm100_gemm_scratch_extent_host_v1(rows, cols, tokens, terms, byref(out)))
    return int(out.value)


def repack_extent(layout: int, rows: int, cols: int) -> int:
    out = c_uint64()
    _check("repack_extent", abi.lib().augur_cuda_nvfp4_sm100_repack_extent_host_v1(layout, rows, cols, byref(out)))
    return int(out.value)


def _u8p(a: np.ndarray | None):
    if a is None:
        return ctypes.cast(None, abi._U8P)
    return a.ctypes.data_as(abi._U8P)


def repack_host(layout: int, rows: int, cols: int, codes, scales, codes_b=None, scales_b=None) -> np.ndarray:
    """Host-memory repack (same permutation as the device kernel)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    if codes_b is not None:
        codes_b = np.ascontiguousarray(codes_b, dtype=np.uint8)
        scales_b = np.ascontiguousarray(scales_b, dtype=np.uint8)
    out = np.zeros(repack_extent(layout, rows, cols), dtype=np.uint8)
    _check("repack_host", abi.lib().augur_cuda_nvfp4_sm100_repack_host_v1(
        layout, rows, cols, _u8p(codes), _u8p(scales), _u8p(codes_b), _u8p(scales_b), _u8p(out), c_uint64(out.size)))
    return out


def unpack_host(layout: int, rows: int, cols: int, packed: np.ndarray):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    pair = layout == abi.LAYOUT_STREAM_PAIR
    codes = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    codes_b = np.zeros_like(codes) if pair else None
    scales_b = np.zeros_like(scales) if pair else None
    _check("unpack_host", abi.lib().augur_cuda_nvfp4_sm100_unpack_host_v1(
        layout, rows, cols, _u8p(packed), c_uint64(packed.size), _u8p(codes), _u8p(scales), _u8p(codes_b), _u8p(scales_b)))
    return (codes, scales, codes_b, scales_b) if pair else (codes, scales)


class Nvfp4Sm100Weight:
    """A weight uploaded to the device and repacked into one hot layout.

    Mirrors ``OwnedCudaQwen35QpnWeightV1::upload_checkpoint_nvfp4``
    (crates/augur-backend/src/cuda_qwen35_qpn.rs:97-131): host-side checks
    (shape, extents, block scales < 127, global scale in [2^-32, 24]), upload of
    the compact planes, repack preflight + submit on the device, synchronise.
    """

    def __init__(self, stream: Stream, layout: int, rows: int, cols: int, packed: torch.Tensor,
                 global_scale: float, global_scale_b: float = 0.0):
        self.stream, self.layout, self.rows, self.cols = stream, layout, rows, cols
        self.packed, self.global_scale, self.global_scale_b = packed, float(global_scale), float(global_scale_b)

    @staticmethod
    def checked_checkpoint(rows: int, cols: int, codes: np.ndarray, scales: np.ndarray, global_scale: float):
        if codes.size != rows * cols // 2 or scales.size != rows * cols // 16:
            raise ValueError("plane extent mismatch")
        if int(scales.max(initial=0)) >= 127:
            raise ValueError("negative or NaN block scale")
        if not (np.isfinite(global_scale) and 2.0 ** -32 <= global_scale <= 24.0):
            raise ValueError("global scale out of range")

    @classmethod
    def upload_checkpoint_nvfp4(cls, stream: Stream, layout: int, rows: int, cols: int, codes, scales,
                                global_scale: float, codes_b=None, scales_b=None, global_scale_b: float = 0.0):
        device = torch.device("cuda", stream.ordinal)
        planes = []
        for c, s, g in ((codes, scales, global_scale), (codes_b, scales_b, global_scale_b)):
            if c is None:
                planes += [None, None]
                continue
            c = np.ascontiguousarray(c, dtype=np.uint8)
            s = np.ascontiguousarray(s, dtype=np.uint8)
            cls.checked_checkpoint(rows, cols, c, s, g)
            planes += [torch.from_numpy(c).to(device), torch.from_numpy(s).to(device)]
        return cls.repack_device_planes(stream, layout, rows, cols, planes[0], planes[1], global_scale,
                                        planes[2], planes[3], global_scale_b)

    @classmethod
    def repack_device_planes(cls, stream: Stream, layout: int, rows: int, cols: int, codes: torch.Tensor,
                             scales: torch.Tensor, global_scale: float, codes_b: torch.Tensor | None = None,
                             scales_b: torch.Tensor | None = None, global_scale_b: float = 0.0):
        """Repack compact planes that already live on the device (preflight + submit + synchronise)."""
        destination = torch.empty(repack_extent(layout, rows, cols), dtype=torch.uint8, device=codes.device)
        args = abi.header(abi.RepackArgs)
        args.codes, args.codes_len_bytes = _ptr(codes), _nbytes(codes)
        args.scales, args.scales_len_bytes = _ptr(scales), _nbytes(scales)
        if codes_b is not None:
            args.codes_b, args.codes_b_len_bytes = _ptr(codes_b), _nbytes(codes_b)
            args.scales_b, args.scales_b_len_bytes = _ptr(scales_b), _nbytes(scales_b)
        args.destination, args.destination_len_bytes = _ptr(destination), _nbytes(destination)
        args.rows, args.cols, args.layout = rows, cols, layout
        lib = abi.lib()
        _check("repack_preflight", lib.augur_cuda_nvfp4_sm100_repack_preflight_v1(stream.ordinal, stream.handle, byref(args)))
        _check("repack_submit", lib.augur_cuda_nvfp4_sm100_repack_prevalidated_submit_v1(stream.ordinal, stream.handle, byref(args)))
        stream.synchronize()
        return cls(stream, layout, rows, cols, destination, global_scale, global_scale_b)

    def dequant_f32(self) -> torch.Tensor:
        """Bit-exact f32 values of the repacked tensor ([rows, cols]; pair: [2, rows, cols])."""
        pair = self.layout == abi.LAYOUT_STREAM_PAIR
        shape = (2, self.rows, self.cols) if pair else (self.rows, self.cols)
        out = torch.empty(shape, dtype=torch.float32, device=self.packed.device)
        args = abi.header(abi.DequantArgs)
        args.weight, args.weight_len_bytes = _ptr(self.packed), _nbytes(self.packed)
        args.output_f32, args.output_len_bytes = _ptr(out), _nbytes(out)
        args.rows, args.cols, args.layout = self.rows, self.cols, self.layout
        args.global_scale, args.global_scale_b = self.global_scale, self.global_scale_b
        lib = abi.lib()
        s = self.stream
        _check("dequant_preflight", lib.augur_cuda_nvfp4_sm100_dequant_f32_preflight_v1(s.ordinal, s.handle, byref(args)))
        _check("dequant_submit", lib.augur_cuda_nvfp4_sm100_dequant_f32_prevalidated_submit_v1(s.ordinal, s.handle, byref(args)))
        return out


def dequant_compact_f32(stream: Stream, codes: torch.Tensor, scales: torch.Tensor, rows: int, cols: int,
                        global_scale: float) -> torch.Tensor:
    out = torch.empty((rows, cols), dtype=torch.float32, device=codes.device)
    args = abi.header(abi.DequantArgs)
    args.weight, args.weight_len_bytes = _ptr(codes), _nbytes(codes)
    args.scales, args.scales_len_bytes = _ptr(scales), _nbytes(scales)
    args.output_f32, args.output_len_bytes = _ptr(out), _nbytes(out)
    args.rows, args.cols, args.layout, args.global_scale = rows, cols, abi.LAYOUT_COMPACT, global_scale
    lib = abi.lib()
    _check("dequant_preflight", lib.augur_cuda_nvfp4_sm100_dequant_f32_preflight_v1(stream.ordinal, stream.handle, byref(args)))
    _check("dequant_submit", lib.augur_cuda_nvfp4_sm100_dequant_f32_prevalidated_submit_v1(stream.ordinal, stream.handle, byref(args)))
    return out


def gemv_args(weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor, epilogue: int) -> abi.GemvArgs:
    args = abi.header(abi.GemvArgs)
    args.weight, args.weight_len_bytes = _ptr(weight.packed), _nbytes(weight.packed)
    args.input_bf16, args.input_len_bytes = _ptr(x), _nbytes(x)
    args.output, args.output_len_bytes = _ptr(out), _nbytes(out)
    args.rows, args.cols, args.tokens, args.epilogue = weight.rows, weight.cols, x.shape[0], epilogue
    args.global_scale, args.global_scale_b = weight.global_scale, weight.global_scale_b
    return args


class Nvfp4Sm100Projection:
    """A retained small-token projection: preflight once at bind, submit many times.

    Mirrors ``CudaQwen35QpnRetainedProjectionV1`` (qpn.rs:60-105, 202-224): the
    binding keeps the plan, stream, weight, input and output alive, is immutable
    after preflight, and ``submit_for_plan`` only enqueues.
    """

    def __init__(self, plan: Plan, weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor, epilogue: int):
        self.plan, self.weight, self.x, self.out = plan, weight, x, out
        self.args = gemv_args(weight, x, out, epilogue)

    @classmethod
    def bind(cls, plan: Plan, weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor | None = None,
             epilogue: int | None = None):
        if epilogue is None:
            epilogue = abi.EPILOGUE_SWIGLU_BF16 if weight.layout == abi.LAYOUT_STREAM_PAIR else abi.EPILOGUE_LINEAR_BF16
        if out is None:
            dtype = torch.float32 if epilogue == abi.EPILOGUE_LINEAR_F32 else torch.bfloat16
            out = torch.empty((x.shape[0], weight.rows), dtype=dtype, device=x.device)
        self = cls(plan, weight, x, out, epilogue)
        s = plan.stream
        _check("gemv_preflight", abi.lib().augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(
            s.ordinal, s.handle, plan.handle, byref(self.args)))
        return self

    def submit_for_plan(self) -> None:
        s = self.plan.stream
        _check("gemv_submit", abi.lib().augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.args)))


def gemv_tc_scratch_bytes(rows: int, cols: int, epilogue: int = abi.EPILOGUE_LINEAR_BF16) -> int:
    out = c_uint64()
    _check("gemv_tc_scratch_extent", abi.lib().augur_cuda_nvfp4_sm100_gemv_tc_scratch_extent_host_v1(rows, cols, epilogue, byref(out)))
    return int(out.value)


class Nvfp4Sm100TcProjection:
    """A retained small-token projection on the tensor-memory path: the weight is in the tcgen05 layout
    (the one the prefill GEMM uses; for the SwiGLU epilogue the interleaved gate|up tensor of
    `upload_gate_up_interleaved`), the kernel is `gemv_tc`. Same contract as `Nvfp4Sm100Projection`."""

    def __init__(self, plan: Plan, weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor, epilogue: int):
        assert weight.layout == abi.LAYOUT_TCGEN05
        self.plan, self.weight, self.x, self.out = plan, weight, x, out
        args = gemv_args(weight, x, out, epilogue)
        if epilogue == abi.EPILOGUE_SWIGLU_BF16:
            args.rows = weight.rows // 2          # the output width; the weight holds gate and up rows
        else:
            args.global_scale_b = 0.0
        self.args = args

    @classmethod
    def bind(cls, plan: Plan, weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor | None = None,
             epilogue: int = abi.EPILOGUE_LINEAR_BF16):
        width = weight.rows // 2 if epilogue == abi.EPILOGUE_SWIGLU_BF16 else weight.rows
        if out is None:
            dtype = torch.float32 if epilogue == abi.EPILOGUE_LINEAR_F32 else torch.bfloat16
            out = torch.empty((x.shape[0], width), dtype=dtype, device=x.device)
        self = cls(plan, weight, x, out, epilogue)
        s = plan.stream
        _check("gemv_tc_preflight", abi.lib().augur_cuda_nvfp4_sm100_gemv_tc_bf16_preflight_v1(
            s.ordinal, s.handle, plan.handle, byref(self.args)))
        return self

    def submit_for_plan(self) -> None:
        s = self.plan.stream
        _check("gemv_tc_submit", abi.lib().augur_cuda_nvfp4_sm100_gemv_tc_bf16_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.args)))


def mlp_tc_scratch_bytes(hidden: int, intermediate: int) -> int:
    """Plan scratch for the one-launch FFN program: counter regions plus one half of the rest per member."""
    need = max(gemv_tc_scratch_bytes(intermediate, hidden, abi.EPILOGUE_SWIGLU_BF16), gemv_tc_scratch_bytes(hidden, intermediate))
    return 2 * need + 512


class Nvfp4Sm100TcFfnProgram:
    """gate|up + SwiGLU, then down, as ONE launch on the tensor-memory path (`mlp_tc`): `gate_up` is the
    interleaved tcgen05 weight of `upload_gate_up_interleaved`, `down` a tcgen05 weight. Same contract as
    `Nvfp4Sm100FfnProgram` (qpn.rs:391-492): validated once at bind, `submit_for_plan` only enqueues."""

    def __init__(self, plan: Plan, gate_up: Nvfp4Sm100Weight, down: Nvfp4Sm100Weight, x: torch.Tensor,
                 intermediate: torch.Tensor, out: torch.Tensor, down_epilogue: int):
        assert gate_up.layout == abi.LAYOUT_TCGEN05 and down.layout == abi.LAYOUT_TCGEN05
        self.plan, self.gate_up, self.down = plan, gate_up, down
        self.x, self.intermediate, self.out = x, intermediate, out
        self.args = abi.header(abi.MlpArgs)
        first = gemv_args(gate_up, x, intermediate, abi.EPILOGUE_SWIGLU_BF16)
        first.rows = gate_up.rows // 2
        second = gemv_args(down, intermediate, out, down_epilogue)
        second.global_scale_b = 0.0
        self.args.gate_up, self.args.down = first, second

    @classmethod
    def bind(cls, plan: Plan, gate_up: Nvfp4Sm100Weight, down: Nvfp4Sm100Weight, x: torch.Tensor,
             out: torch.Tensor | None = None, down_epilogue: int = abi.EPILOGUE_LINEAR_BF16):
        tokens = x.shape[0]
        intermediate = torch.empty((tokens, gate_up.rows // 2), dtype=torch.bfloat16, device=x.device)
        if out is None:
            dtype = torch.float32 if down_epilogue == abi.EPILOGUE_LINEAR_F32 else torch.bfloat16
            out = torch.empty((tokens, down.rows), dtype=dtype, device=x.device)
        self = cls(plan, gate_up, down, x, intermediate, out, down_epilogue)
        s = plan.stream
        _check("mlp_tc_preflight", abi.lib().augur_cuda_nvfp4_sm100_mlp_tc_preflight_v1(
            s.ordinal, s.handle, plan.handle, byref(self.args)))
        return self

    def submit_for_plan(self) -> None:
        s = self.plan.stream
        _check("mlp_tc_submit", abi.lib().augur_cuda_nvfp4_sm100_mlp_tc_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.args)))


class Nvfp4Sm100FfnProgram:
    """gate|up + SwiGLU, then down, as one validated program.

    Mirrors ``CudaQwen35QpnFfnProgramV1::bind / submit_for_plan`` (qpn.rs:391-492).
    """

    def __init__(self, plan: Plan, gate_up: Nvfp4Sm100Weight, down: Nvfp4Sm100Weight, x: torch.Tensor,
                 intermediate: torch.Tensor, out: torch.Tensor, down_epilogue: int):
        self.plan, self.gate_up, self.down = plan, gate_up, down
        self.x, self.intermediate, self.out = x, intermediate, out
        self.args = abi.header(abi.MlpArgs)
        self.args.gate_up = gemv_args(gate_up, x, intermediate, abi.EPILOGUE_SWIGLU_BF16)
        self.args.down = gemv_args(down, intermediate, out, down_epilogue)

    @classmethod
    def bind(cls, plan: Plan, gate_up: Nvfp4Sm100Weight, down: Nvfp4Sm100Weight, x: torch.Tensor,
             out: torch.Tensor | None = None, down_epilogue: int = abi.EPILOGUE_LINEAR_BF16):
        tokens = x.shape[0]
        intermediate = torch.empty((tokens, gate_up.rows), dtype=torch.bfloat16, device=x.device)
        if out is None:
            dtype = torch.float32 if down_epilogue == abi.EPILOGUE_LINEAR_F32 else torch.bfloat16
            out = torch.empty((tokens, down.rows), dtype=dtype, device=x.device)
        self = cls(plan, gate_up, down, x, intermediate, out, down_epilogue)
        s = plan.stream
        _check("mlp_preflight", abi.lib().augur_cuda_nvfp4_sm100_mlp_preflight_v1(
            s.ordinal, s.handle, plan.handle, byref(self.args)))
        return self

    def submit_for_plan(self) -> None:
        s = self.plan.stream
        _check("mlp_submit", abi.lib().augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.args)))


def mlp_scratch_bytes(hidden: int, intermediate: int, tokens: int = 8) -> int:
    """Plan scratch for an FFN program: counter regions plus one half of the slot area per member."""
    need = max(gemv_scratch_bytes(intermediate, hidden, tokens), gemv_scratch_bytes(hidden, intermediate, tokens))
    return 2 * need + 512


def allocation_snapshot() -> tuple[int, int]:
    a, f = c_uint64(), c_uint64()
    abi.lib().augur_cuda_nvfp4_sm100_allocation_snapshot_v1(byref(a), byref(f))
    return int(a.value), int(f.value)


def launch_count() -> int:
    return int(abi.lib().augur_cuda_nvfp4_sm100_launch_count_v1())


def default_activation_global_scale(absmax: float = 448.0 * 6.0) -> float:
    """Per-tensor activation scale so that `absmax` maps to the top of the E4M3 x E2M1 range."""
    return float(np.float32(absmax) / np.float32(448.0 * 6.0))


class Nvfp4Sm100PrefillLinear:
    """Prefill projection: BF16 activations -> NVFP4 residual terms -> tcgen05 block-scaled GEMM.

    Mirrors the wide-token branch of the retained projection
    (crates/augur-cuda-sys/native/augur_qwen35_qpn_prefill.cuh:53-88: stage the
    activations, then one tensor-core GEMM) with both members validated at bind time.
    """

    def __init__(self, plan: Plan, weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor, terms: int,
                 activation_global_scale: float):
        assert weight.layout == abi.LAYOUT_TCGEN05
        self.plan, self.weight, self.x, self.out, self.terms = plan, weight, x, out, terms
        tokens, cols = x.shape
        self.staged = torch.empty(gemm_scratch_bytes(weight.rows, cols, tokens, terms), dtype=torch.uint8, device=x.device)
        q = abi.header(abi.ActQuantArgs)
        q.input_bf16, q.input_len_bytes = _ptr(x), _nbytes(x)
        q.destination, q.destination_len_bytes = _ptr(self.staged), _nbytes(self.staged)
        q.tokens, q.cols, q.terms, q.global_scale = tokens, cols, terms, activation_global_scale
        g = abi.header(abi.GemmArgs)
        g.weight, g.weight_len_bytes = _ptr(weight.packed), _nbytes(weight.packed)
        g.activation, g.activation_len_bytes = _ptr(self.staged), _nbytes(self.staged)
        g.output_bf16, g.output_len_bytes = _ptr(out), _nbytes(out)
        g.rows, g.cols, g.tokens, g.activation_terms = weight.rows, cols, tokens, terms
        g.weight_global_scale, g.activation_global_scale = weight.global_scale, activation_global_scale
        self.quant_args, self.gemm_args = q, g

    @classmethod
    def bind(cls, plan: Plan, weight: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor | None = None,
             terms: int = 1, activation_global_scale: float = 2.0 ** -8):
        if out is None:
            out = torch.empty((x.shape[0], weight.rows), dtype=torch.bfloat16, device=x.device)
        self = cls(plan, weight, x, out, terms, activation_global_scale)
        s, lib = plan.stream, abi.lib()
        _check("act_quant_preflight", lib.augur_cuda_nvfp4_sm100_act_quant_preflight_v1(s.ordinal, s.handle, byref(self.quant_args)))
        _check("gemm_preflight", lib.augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(s.ordinal, s.handle, plan.handle, byref(self.gemm_args)))
        return self

    def submit_quant(self) -> None:
        s = self.plan.stream
        _check("act_quant_submit", abi.lib().augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(
            s.ordinal, s.handle, byref(self.quant_args)))

    def submit_gemm(self) -> None:
        s = self.plan.stream
        _check("gemm_submit", abi.lib().augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.gemm_args)))

    def submit_for_plan(self) -> None:
        self.submit_quant()
        self.submit_gemm()

    def staged_planes(self):
        """Quantised activations back on the host: (codes [terms, tokens, cols/2], scales [terms, tokens, cols/16])."""
        tokens, cols = self.x.shape
        padded = (tokens + 127) // 128 * 128
        raw = self.staged.cpu().numpy()
        code_bytes = padded * cols // 2
        sf_bytes = repack_extent(abi.LAYOUT_TCGEN05, padded, cols) - code_bytes
        codes = raw[: self.terms * code_bytes].reshape(self.terms, padded, cols // 2)[:, :tokens].copy()
        scales = np.zeros((self.terms, tokens, cols // 16), dtype=np.uint8)
        for term in range(self.terms):
            packed = np.concatenate([raw[term * code_bytes: (term + 1) * code_bytes],
                                     raw[self.terms * code_bytes + term * sf_bytes: self.terms * code_bytes + (term + 1) * sf_bytes]])
            _, full = unpack_host(abi.LAYOUT_TCGEN05, padded, cols, packed)
            scales[term] = full[:tokens]
        return codes, scales


def upload_gate_up_interleaved(stream: Stream, inter: int, hidden: int, gate_codes, gate_scales, gate_global: float,
                               up_codes, up_scales, up_global: float) -> Nvfp4Sm100Weight:
    """The gate and up matrices as ONE tcgen05 weight of 2 * inter rows, 16 gate rows alternating with the
    matching 16 up rows, which is what the SwiGLU-fusing GEMM epilogue expects."""
    Nvfp4Sm100Weight.checked_checkpoint(inter, hidden, np.asarray(gate_codes), np.asarray(gate_scales), gate_global)
    Nvfp4Sm100Weight.checked_checkpoint(inter, hidden, np.asarray(up_codes), np.asarray(up_scales), up_global)
    gc, gs = np.ascontiguousarray(gate_codes, dtype=np.uint8), np.ascontiguousarray(gate_scales, dtype=np.uint8)
    uc, us = np.ascontiguousarray(up_codes, dtype=np.uint8), np.ascontiguousarray(up_scales, dtype=np.uint8)
    codes = np.empty((2 * inter, hidden // 2), dtype=np.uint8)
    scales = np.empty((2 * inter, hidden // 16), dtype=np.uint8)
    _check("interleave_gate_up", abi.lib().augur_cuda_nvfp4_sm100_interleave_gate_up_host_v1(
        inter, hidden, _u8p(gc), _u8p(gs), _u8p(uc), _u8p(us), _u8p(codes), _u8p(scales)))
    weight = Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_TCGEN05, 2 * inter, hidden, codes, scales, gate_global)
    weight.global_scale_b = float(up_global)
    return weight


class Nvfp4Sm100PrefillFfnProgram:
    """The MLP block for wide inputs: quantise x, gate|up GEMM with SiLU(gate)*up in its epilogue,
    quantise the intermediate, down GEMM. Four launches, all members preflighted at bind time.

    The wide-token counterpart of `Nvfp4Sm100FfnProgram` (the reference runs this shape as
    stage -> two GEMMs -> silu/pack -> stage -> GEMM, crates/augur-cuda-sys/native/augur_qwen35_qpn_prefill.cuh:97-147).
    """

    def __init__(self, plan: Plan, gate_up: Nvfp4Sm100Weight, down: Nvfp4Sm100Weight, x: torch.Tensor, out: torch.Tensor,
                 terms: int, input_global_scale: float, intermediate_global_scale: float, fuse_quantiser: bool = True,
                 keep_intermediate: bool = False):
        assert gate_up.layout == abi.LAYOUT_TCGEN05 and down.layout == abi.LAYOUT_TCGEN05
        tokens, hidden = x.shape
        inter = gate_up.rows // 2
        if gate_up.cols != hidden or down.cols != inter or down.rows != out.shape[1] or out.shape[0] != tokens:
            raise ValueError("gate|up, down, input and output shapes do not fit together")
        self.plan, self.gate_up, self.down, self.x, self.out, self.terms = plan, gate_up, down, x, out, terms
        self.intermediate = torch.empty((tokens, inter), dtype=torch.bfloat16, device=x.device)
        self.staged_x = torch.empty(gemm_scratch_bytes(gate_up.rows, hidden, tokens, terms), dtype=torch.uint8, device=x.device)
        self.staged_h = torch.empty(gemm_scratch_bytes(down.rows, inter, tokens, terms), dtype=torch.uint8, device=x.device)

        def quant(source, staged, cols, scale):
            q = abi.header(abi.ActQuantArgs)
            q.input_bf16, q.input_len_bytes = _ptr(source), _nbytes(source)
            q.destination, q.destination_len_bytes = _ptr(staged), _nbytes(staged)
            q.tokens, q.cols, q.terms, q.global_scale = tokens, cols, terms, scale
            return q

        self.quant_x = quant(x, self.staged_x, hidden, input_global_scale)
        self.quant_h = quant(self.intermediate, self.staged_h, inter, intermediate_global_scale)
        g = abi.header(abi.GemmSwigluArgs)
        g.weight, g.weight_len_bytes = _ptr(gate_up.packed), _nbytes(gate_up.packed)
        g.activation, g.activation_len_bytes = _ptr(self.staged_x), _nbytes(self.staged_x)
        g.output_bf16, g.output_len_bytes = _ptr(self.intermediate), _nbytes(self.intermediate)
        g.rows, g.cols, g.tokens, g.activation_terms = inter, hidden, tokens, terms
        g.gate_global_scale, g.up_global_scale, g.activation_global_scale = gate_up.global_scale, gate_up.global_scale_b, input_global_scale
        d = abi.header(abi.GemmArgs)
        d.weight, d.weight_len_bytes = _ptr(down.packed), _nbytes(down.packed)
        d.activation, d.activation_len_bytes = _ptr(self.staged_h), _nbytes(self.staged_h)
        d.output_bf16, d.output_len_bytes = _ptr(out), _nbytes(out)
        d.rows, d.cols, d.tokens, d.activation_terms = down.rows, inter, tokens, terms
        d.weight_global_scale, d.activation_global_scale = down.global_scale, intermediate_global_scale
        self.gate_up_args, self.down_args = g, d
        # On the two-CTA tiles the gate|up GEMM can quantise its result for the down GEMM in its own epilogue.
        self.fused = fuse_quantiser and inter % 128 == 0
        if self.fused:
            f = abi.header(abi.GemmSwigluQuantArgs)
            f.weight, f.weight_len_bytes = g.weight, g.weight_len_bytes
            f.activation, f.activation_len_bytes = g.activation, g.activation_len_bytes
            if keep_intermediate:
                f.output_bf16, f.output_len_bytes = g.output_bf16, g.output_len_bytes
            f.destination, f.destination_len_bytes = _ptr(self.staged_h), _nbytes(self.staged_h)
            f.rows, f.cols, f.tokens, f.activation_terms = inter, hidden, tokens, terms
            f.gate_global_scale, f.up_global_scale = g.gate_global_scale, g.up_global_scale
            f.activation_global_scale, f.destination_global_scale = input_global_scale, intermediate_global_scale
            f.destination_terms = terms
            self.fused_args = f

    @classmethod
    def bind(cls, plan: Plan, gate_up: Nvfp4Sm100Weight, down: Nvfp4Sm100Weight, x: torch.Tensor,
             out: torch.Tensor | None = None, terms: int = 3, input_global_scale: float = 2.0 ** -8,
             intermediate_global_scale: float = 2.0 ** -8, fuse_quantiser: bool = True, keep_intermediate: bool = False):
        """`fuse_quantiser`: quantise the intermediate inside the gate|up GEMM when the shape allows it (three
        launches instead of four); `keep_intermediate`: also write its BF16 form then (it is always written otherwise)."""
        if out is None:
            out = torch.empty((x.shape[0], down.rows), dtype=torch.bfloat16, device=x.device)
        self = cls(plan, gate_up, down, x, out, terms, input_global_scale, intermediate_global_scale, fuse_quantiser,
                   keep_intermediate)
        s, lib = plan.stream, abi.lib()
        _check("act_quant_preflight", lib.augur_cuda_nvfp4_sm100_act_quant_preflight_v1(s.ordinal, s.handle, byref(self.quant_x)))
        if self.fused:
            _check("gemm_swiglu_quant_preflight", lib.augur_cuda_nvfp4_sm100_gemm_swiglu_quant_preflight_v1(
                s.ordinal, s.handle, plan.handle, byref(self.fused_args)))
        else:
            _check("gemm_swiglu_preflight", lib.augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_preflight_v1(
                s.ordinal, s.handle, plan.handle, byref(self.gate_up_args)))
            _check("act_quant_preflight", lib.augur_cuda_nvfp4_sm100_act_quant_preflight_v1(s.ordinal, s.handle, byref(self.quant_h)))
        _check("gemm_preflight", lib.augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(s.ordinal, s.handle, plan.handle, byref(self.down_args)))
        return self

    def submit_for_plan(self) -> None:
        s, lib = self.plan.stream, abi.lib()
        _check("act_quant_submit", lib.augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(s.ordinal, s.handle, byref(self.quant_x)))
        if self.fused:
            _check("gemm_swiglu_quant_submit", lib.augur_cuda_nvfp4_sm100_gemm_swiglu_quant_prevalidated_submit_v1(
                s.ordinal, s.handle, self.plan.handle, byref(self.fused_args)))
        else:
            _check("gemm_swiglu_submit", lib.augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_prevalidated_submit_v1(
                s.ordinal, s.handle, self.plan.handle, byref(self.gate_up_args)))
            _check("act_quant_submit", lib.augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(s.ordinal, s.handle, byref(self.quant_h)))
        _check("gemm_submit", lib.augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.down_args)))


class Nvfp4Sm100NormGroupProgram:
    """[residual add] -> RMSNorm -> BF16 stage -> one to four small-token projections, as one validated program.

    Mirrors the reference's fused norm stage with grouped projections
    (crates/augur-cuda-sys/native/augur_qwen35_gdn_input_b8.cuh; the GDN input group and the post-attention group):
    `input_f32` is the residual stream [tokens, cols] (with `add_a` / `add_b` it is first overwritten by their
    sum), `norm_weight_f32` the RMSNorm weight, `weights` the projections (STREAM layout) that all read the
    normalised, BF16-rounded activations.
    """

    def __init__(self, plan: Plan, weights, input_f32: torch.Tensor, norm_weight_f32: torch.Tensor, epsilon: float,
                 add_a: torch.Tensor | None, add_b: torch.Tensor | None, stored_rows=None):
        tokens, cols = input_f32.shape
        self.plan, self.weights, self.input, self.norm_weight = plan, list(weights), input_f32, norm_weight_f32
        self.add_a, self.add_b = add_a, add_b
        self.normalised = torch.empty((tokens, cols), dtype=torch.float32, device=input_f32.device)
        self.staged = torch.empty((tokens, cols), dtype=torch.bfloat16, device=input_f32.device)
        # stored_rows[i] (0: all): member i writes only its first rows, e.g. 48 of a gate padded to 64 weight rows
        self.stored_rows = list(stored_rows) if stored_rows is not None else [0] * len(self.weights)
        self.outputs = [torch.empty((tokens, keep or w.rows), dtype=torch.bfloat16, device=input_f32.device)
                        for w, keep in zip(self.weights, self.stored_rows)]
        a = abi.header(abi.NormGroupArgs)
        if add_a is not None:
            a.add_a, a.add_b, a.add_len_bytes, a.residual = _ptr(add_a), _ptr(add_b), _nbytes(add_a), 1
        a.input_f32, a.input_len_bytes = _ptr(input_f32), _nbytes(input_f32)
        a.weight_f32, a.weight_len_bytes = _ptr(norm_weight_f32), _nbytes(norm_weight_f32)
        a.output_f32, a.output_len_bytes = _ptr(self.normalised), _nbytes(self.normalised)
        a.staged_bf16, a.staged_len_bytes = _ptr(self.staged), _nbytes(self.staged)
        a.tokens, a.cols, a.epsilon, a.count = tokens, cols, epsilon, len(self.weights)
        for index, (weight, out) in enumerate(zip(self.weights, self.outputs)):
            a.projections[index] = gemv_args(weight, self.staged, out, abi.EPILOGUE_LINEAR_BF16)
            a.projections[index].stored_rows = self.stored_rows[index]
        self.args = a

    @classmethod
    def bind(cls, plan: Plan, weights, input_f32: torch.Tensor, norm_weight_f32: torch.Tensor, epsilon: float = 1e-6,
             add_a: torch.Tensor | None = None, add_b: torch.Tensor | None = None, stored_rows=None):
        if (add_a is None) != (add_b is None):
            raise ValueError("the residual add takes both operands or none")
        self = cls(plan, weights, input_f32, norm_weight_f32, epsilon, add_a, add_b, stored_rows)
        s = plan.stream
        _check("norm_group_preflight", abi.lib().augur_cuda_nvfp4_sm100_norm_group_preflight_v1(
            s.ordinal, s.handle, plan.handle, byref(self.args)))
        return self

    def submit_for_plan(self) -> None:
        s = self.plan.stream
        _check("norm_group_submit", abi.lib().augur_cuda_nvfp4_sm100_norm_group_prevalidated_submit_v1(
            s.ordinal, s.handle, self.plan.handle, byref(self.args)))


class Bf16Head:
    """The BF16 vocabulary head bound to one (input, output) pair: weights [rows, cols] BF16 read in place,
    F32 activations [tokens <= 8, cols], F32 logits [tokens, rows]. Mirrors the reference's shared-head binding
    (crates/augur-model-qwen35-runtime/src/checkpoint_projection_cuda/dflash_head.rs): preflight at bind,
    `submit` only enqueues."""

    def __init__(self, stream: Stream, weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor):
        rows, cols = weight.shape
        self.stream, self.weight, self.x, self.out = stream, weight, x, out
        a = abi.header(abi.Bf16HeadArgs)
        a.weight, a.weight_len_bytes = _ptr(weight), _nbytes(weight)
        a.input, a.input_len_bytes = _ptr(x), _nbytes(x)
        a.output, a.output_len_bytes = _ptr(out), _nbytes(out)
        a.rows, a.cols = rows, cols
        self.args = a

    @classmethod
    def bind(cls, stream: Stream, weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None):
        if weight.dtype != torch.bfloat16 or x.dtype != torch.float32:
            raise ValueError("BF16 weights and F32 activations")
        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        self = cls(stream, weight, x, out)
        _check("bf16_head_preflight", abi.lib().augur_cuda_nvfp4_sm100_bf16_head_preflight_v1(
            stream.ordinal, stream.handle, byref(self.args)))
        return self

    def submit(self) -> None:
        _check("bf16_head_submit", abi.lib().augur_cuda_nvfp4_sm100_bf16_head_prevalidated_submit_v1(
            self.stream.ordinal, self.stream.handle, byref(self.args)))


SHAPE_SMALL_BATCH = "small-batch"
SHAPE_PREFILL = "prefill"


def classify_tokens(tokens: int) -> str:
    """The reference's batch classes (crates/augur-kernel-api/src/key.rs:354-365): up to 8 token rows are the
    small-batch class (decode and the fixed B8 verify batch), anything wider is prefill."""
    if tokens < 1:
        raise ValueError("at least one token row")
    return SHAPE_SMALL_BATCH if tokens <= abi.MAX_SMALL_TOKENS else SHAPE_PREFILL


class Nvfp4Sm100Linear:
    """One weight matrix, any number of token rows: the dispatch a model runtime does per call site.

    Keeps the weight in both hot layouts (the small-token stream layout and the tcgen05 layout) and
    binds the kernel its shape class calls for: tokens <= 8 -> `Nvfp4Sm100Projection`, otherwise
    `Nvfp4Sm100PrefillLinear` (activation quantiser with `terms` residual terms, then the block-scaled
    GEMM). Bindings are made per (input, output) pair, exactly like the two classes it chooses between.
    """

    def __init__(self, stream: Stream, rows: int, cols: int, codes, scales, global_scale: float):
        self.rows, self.cols = rows, cols
        self.small = Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_STREAM, rows, cols, codes, scales, global_scale)
        self.wide = Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_TCGEN05, rows, cols, codes, scales, global_scale)

    def bind(self, plan: Plan, x: torch.Tensor, out: torch.Tensor | None = None, terms: int = 3,
             activation_global_scale: float = 2.0 ** -8):
        if classify_tokens(x.shape[0]) == SHAPE_SMALL_BATCH:
            return Nvfp4Sm100Projection.bind(plan, self.small, x, out)
        return Nvfp4Sm100PrefillLinear.bind(plan, self.wide, x, out, terms=terms, activation_global_scale=activation_global_scale)
