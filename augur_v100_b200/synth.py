"""Seeded synthetic NVFP4 tensors with the shapes and value distributions of the benchmark configs.

These stand in for real checkpoint tensors (none ship with the reference):
codes are uniform over the 16 E2M1 codes, packed two per byte along K with
the even element in the low nibble; block scales are ``|N(0,1)| * 0.5`` clamped
to the positive E4M3 range and rounded to nearest-even; the per-tensor scale is
``float32(1/448)``; activations are ``N(0,1)`` rounded to BF16. Every tensor
has its own PCG64 stream keyed by ``(seed, config, crc32(name))`` so that any
consumer regenerates identical bytes.
"""
from __future__ import annotations

import zlib

import numpy as np

GLOBAL_SCALE = float(np.float32(1.0) / np.float32(448.0))


def _rng(seed: int, config: int, name: str) -> np.random.Generator:
    return np.random.default_rng([int(seed), int(config), zlib.crc32(name.encode())])


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> BF16 bit patterns (uint16)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _e4m3_positive_table() -> np.ndarray:
    code = np.arange(127)
    exponent = code >> 3
    mantissa = (code & 7).astype(np.float64)
    return np.where(exponent == 0, 2.0 ** -6 * mantissa / 8.0, 2.0 ** (exponent - 7.0) * (1.0 + mantissa / 8.0))


def e4m3_encode_rne(values: np.ndarray) -> np.ndarray:
    """Nearest positive E4M3 code (0..126), ties to the even code; input must be >= 0."""
    table = _e4m3_positive_table()
    v = np.clip(np.asarray(values, dtype=np.float64), 0.0, 448.0)
    hi = np.clip(np.searchsorted(table, v, side="left"), 1, 126)
    lo = hi - 1
    d_lo = v - table[lo]
    d_hi = table[hi] - v
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8)


def make_weight(seed: int, config: int, name: str, rows: int, cols: int):
    """Returns (codes [rows, cols/2] u8, scales [rows, cols/16] u8, global f32)."""
    rng = _rng(seed, config, name)
    nibbles = rng.integers(0, 16, size=(rows, cols), dtype=np.uint8)
    codes = (nibbles[:, 0::2] | (nibbles[:, 1::2] << 4)).astype(np.uint8)
    raw = np.abs(rng.standard_normal(size=(rows, cols // 16), dtype=np.float32)) * np.float32(0.5)
    scales = e4m3_encode_rne(np.clip(raw, 2.0 ** -9, 448.0))
    scales = np.maximum(scales, 1).astype(np.uint8)
    return np.ascontiguousarray(codes), np.ascontiguousarray(scales), GLOBAL_SCALE


def make_activation(seed: int, config: int, name: str, tokens: int, cols: int) -> np.ndarray:
    """BF16 bit patterns [tokens, cols] of N(0,1) samples."""
    rng = _rng(seed, config, name)
    return f32_to_bf16_bits(rng.standard_normal(size=(tokens, cols), dtype=np.float32))
