"""Checkpoint-format adapters: what a loader hands over -> the planes and scalar this library takes.

Mirrors ``CheckpointNvfp4Scale`` / ``CheckpointNvfp4Matrix``
(crates/augur-model-qwen35/src/checkpoint_quant.rs:10-189):

* compressed-tensors tensors ``weight_packed`` / ``weight_scale`` / ``weight_global_scale``:
  the value is ``e2m1 * e4m3 / weight_global_scale``;
* ModelOpt tensors ``weight`` / ``weight_scale`` / ``weight_scale_2`` (W4A4 and the weight-only
  W4A16 export): the value is ``e2m1 * e4m3 * weight_scale_2``;
* GGML36 wire blocks (36 bytes per 64 elements) in both directions.

Activation scalars (``input_global_scale`` / ``input_scale``) are kept on the object and never
folded into the weight, as in the reference. All checks and byte shuffles run in the C library's
host functions; this module only carries the arrays.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import abi

COMPRESSED_TENSORS = "compressed-tensors"
MODELOPT = "modelopt"
MODELOPT_W4A16 = "modelopt-w4a16"


class CheckpointError(ValueError):
    """A checkpoint tensor the reference's loader would reject too."""


def _u8p(array: np.ndarray):
    return array.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8))


@dataclass(frozen=True)
class CheckpointNvfp4Scale:
    kind: str
    weight_scalar: float               # weight_global_scale (divides) or weight_scale_2 (multiplies)
    input_scalar: float | None = None  # input_global_scale / input_scale; None for the W4A16 export

    def __post_init__(self):
        if self.kind not in (COMPRESSED_TENSORS, MODELOPT, MODELOPT_W4A16):
            raise CheckpointError(f"unknown scale convention {self.kind!r}")
        if self.kind == MODELOPT_W4A16 and self.input_scalar is not None:
            raise CheckpointError("the weight-only export has no activation scale")
        if self.kind != MODELOPT_W4A16 and self.input_scalar is None:
            raise CheckpointError("this convention carries an activation scale")
        for value in (self.weight_scalar, self.input_scalar):
            if value is not None and not (np.isfinite(value) and value > 0):
                raise CheckpointError("expected finite positive scalars")

    def global_scale(self) -> float:
        """The multiplier the kernels take (f32): 1 / weight_global_scale or weight_scale_2."""
        out = ctypes.c_float()
        convention = abi.SCALE_COMPRESSED_TENSORS if self.kind == COMPRESSED_TENSORS else abi.SCALE_MODELOPT
        result = abi.lib().augur_cuda_nvfp4_sm100_checkpoint_global_scale_host_v1(
            convention, ctypes.c_float(self.weight_scalar), ctypes.byref(out))
        if result.status != abi.STATUS_OK:
            raise CheckpointError("the weight scalar is outside the range the kernels accept")
        return float(out.value)

    def apply_f64(self, block_value: np.ndarray) -> np.ndarray:
        """The reference's f64 statement of the value (checkpoint_quant.rs:49-58)."""
        scalar = np.float64(np.float32(self.weight_scalar))
        return block_value / scalar if self.kind == COMPRESSED_TENSORS else block_value * scalar


class CheckpointNvfp4Matrix:
    """Validated checkpoint planes: codes [rows, cols/2] (even k in the low nibble), scales [rows, cols/16]."""

    def __init__(self, rows: int, cols: int, packed, scales, scale: CheckpointNvfp4Scale):
        packed = np.ascontiguousarray(np.asarray(packed, dtype=np.uint8).reshape(-1))
        scales = np.ascontiguousarray(np.asarray(scales, dtype=np.uint8).reshape(-1))
        if rows < 0 or cols < 0 or rows >= 1 << 63 or cols >= 1 << 63:
            raise CheckpointError("shape out of range")
        result = abi.lib().augur_cuda_nvfp4_sm100_checkpoint_validate_host_v1(
            rows, cols, _u8p(packed), packed.size, _u8p(scales), scales.size)
        if result.status != abi.STATUS_OK:
            raise CheckpointError("shape/plane extent mismatch, or a negative or NaN block scale")
        self.rows, self.cols, self.scale = rows, cols, scale
        self.packed, self.scales = packed.reshape(rows, cols // 2), scales.reshape(rows, cols // 16)

    @classmethod
    def from_compressed_tensors(cls, weight_packed, weight_scale, weight_global_scale: float,
                                input_global_scale: float):
        packed = np.asarray(weight_packed, dtype=np.uint8)
        rows, cols = packed.shape[0], packed.shape[1] * 2
        return cls(rows, cols, packed, weight_scale,
                   CheckpointNvfp4Scale(COMPRESSED_TENSORS, float(weight_global_scale), float(input_global_scale)))

    @classmethod
    def from_modelopt(cls, weight, weight_scale, weight_scale_2: float, input_scale: float | None = None):
        packed = np.asarray(weight, dtype=np.uint8)
        rows, cols = packed.shape[0], packed.shape[1] * 2
        kind = MODELOPT if input_scale is not None else MODELOPT_W4A16
        return cls(rows, cols, packed, weight_scale,
                   CheckpointNvfp4Scale(kind, float(weight_scale_2), None if input_scale is None else float(input_scale)))

    @classmethod
    def from_ggml36(cls, rows: int, cols: int, wire, scale: CheckpointNvfp4Scale):
        wire = np.ascontiguousarray(np.asarray(wire, dtype=np.uint8).reshape(-1))
        codes = np.empty(rows * cols // 2, dtype=np.uint8)
        scales = np.empty(rows * cols // 16, dtype=np.uint8)
        result = abi.lib().augur_cuda_nvfp4_sm100_ggml36_to_planes_host_v1(rows, cols, _u8p(wire), wire.size, _u8p(codes), _u8p(scales))
        if result.status != abi.STATUS_OK:
            raise CheckpointError("requires K%64, the exact wire extent and block scales below 127")
        return cls(rows, cols, codes, scales, scale)

    def to_ggml36(self) -> np.ndarray:
        """Codes and scales as GGML36 wire blocks; the global scalar is not folded in."""
        if self.cols % 64 != 0:
            raise CheckpointError("requires K%64")
        wire = np.empty(self.rows * self.cols // 64 * 36, dtype=np.uint8)
        result = abi.lib().augur_cuda_nvfp4_sm100_planes_to_ggml36_host_v1(
            self.rows, self.cols, _u8p(self.packed), _u8p(self.scales), _u8p(wire), wire.size)
        if result.status != abi.STATUS_OK:
            raise CheckpointError("requires K%64 and the exact output extent")
        return wire

    def planes(self):
        """(codes, scales, global_scale) as `Nvfp4Sm100Weight.upload_checkpoint_nvfp4` takes them."""
        return self.packed, self.scales, self.scale.global_scale()
