"""Shared helpers for the parity tests."""
import numpy as np

from augur_v100_b200 import synth

TOLERANCE = 2e-2  # max relative error of a BF16 output against the fp64 oracle


def rel_error(y_bf16_bits: np.ndarray, y64: np.ndarray) -> float:
    """max |y - y64| / max(|y64|, 1e-3 * rms(y64)) over all elements."""
    y = synth.bf16_bits_to_f32(np.asarray(y_bf16_bits, dtype=np.uint16)).astype(np.float64).reshape(y64.shape)
    rms = float(np.sqrt(np.mean(y64 * y64))) or 1.0
    return float(np.max(np.abs(y - y64) / np.maximum(np.abs(y64), 1e-3 * rms)))


def rel_error_f32(y: np.ndarray, y64: np.ndarray) -> float:
    rms = float(np.sqrt(np.mean(y64 * y64))) or 1.0
    return float(np.max(np.abs(y.astype(np.float64) - y64) / np.maximum(np.abs(y64), 1e-3 * rms)))


def bf16_ulp_mismatches(a_bits: np.ndarray, b_bits: np.ndarray) -> int:
    return int(np.count_nonzero(np.asarray(a_bits, dtype=np.uint16).reshape(-1) != np.asarray(b_bits, dtype=np.uint16).reshape(-1)))


def torch_bf16_from_bits(bits: np.ndarray, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits, dtype=np.uint16).view(np.int16)).to(device).view(torch.bfloat16)


def bits_from_torch_bf16(t) -> np.ndarray:
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rms_error(y_bf16_bits: np.ndarray, y64: np.ndarray) -> float:
    """max |y - y64| / rms(y64): for end-to-end chains whose intermediate is rounded to BF16,
    where outputs near zero carry an absolute error of a few 1e-3 rms by construction."""
    y = synth.bf16_bits_to_f32(np.asarray(y_bf16_bits, dtype=np.uint16)).astype(np.float64).reshape(y64.shape)
    rms = float(np.sqrt(np.mean(y64 * y64))) or 1.0
    return float(np.max(np.abs(y - y64)) / rms)
