"""Checkpoint-format adapters against the reference's own expectations.

Vectors and rejection cases are those of the tests in
crates/augur-model-qwen35/src/checkpoint_quant.rs:240-315; the f64 decode used to check them is the
oracle's (E2M1 x E4M3 in f64, then the typed global operation).
"""
import numpy as np
import pytest

import oracle
from augur_v100_b200 import checkpoint as ck


def _decode_f64(m: ck.CheckpointNvfp4Matrix) -> np.ndarray:
    e2m1 = np.array([oracle.decode_e2m1(c) for c in range(16)], dtype=np.float64)
    e4m3 = np.array([oracle.decode_e4m3fn(b) for b in range(127)], dtype=np.float64)
    codes = np.stack([m.packed & 15, m.packed >> 4], axis=-1).reshape(m.rows, m.cols)
    block = e2m1[codes] * np.repeat(e4m3[m.scales], 16, axis=1)
    return m.scale.apply_f64(block)


def test_global_operations_are_distinct_and_activation_scale_is_not_folded():
    packed = np.full((1, 8), 0x72, dtype=np.uint8)   # 1, 6 repeated; E4M3 0x38 is 1
    scales = np.array([[0x38]], dtype=np.uint8)
    augur = ck.CheckpointNvfp4Matrix.from_compressed_tensors(packed, scales, 2.0, 3.0)
    nvidia = ck.CheckpointNvfp4Matrix.from_modelopt(packed, scales, 2.0, 7.0)
    assert list(_decode_f64(augur)[0, :2]) == [0.5, 3.0]
    assert list(_decode_f64(nvidia)[0, :2]) == [2.0, 12.0]
    assert augur.scale.global_scale() == 0.5 and nvidia.scale.global_scale() == 2.0
    assert augur.scale.input_scalar == 3.0 and nvidia.scale.input_scalar == 7.0


def test_w4a16_has_no_activation_scale_and_multiplies():
    packed = np.full((1, 8), 0xFA, dtype=np.uint8)   # -1, -6 in low/high order
    m = ck.CheckpointNvfp4Matrix.from_modelopt(packed, np.array([[0x40]], dtype=np.uint8), 0.125)   # block scale 2
    assert m.scale.kind == ck.MODELOPT_W4A16 and m.scale.input_scalar is None
    assert list(_decode_f64(m)[0, :2]) == [-0.25, -1.5]
    for w in (0.0, -1.0, float("inf"), float("-inf"), float("nan")):
        with pytest.raises(ck.CheckpointError):
            ck.CheckpointNvfp4Matrix.from_modelopt(packed, np.array([[0x40]], dtype=np.uint8), w)


def test_small_48_row_gate_needs_no_padding():
    packed = np.full((48, 5120 // 2), 0xA2, dtype=np.uint8)
    scales = np.full((48, 5120 // 16), 0x38, dtype=np.uint8)
    m = ck.CheckpointNvfp4Matrix.from_compressed_tensors(packed, scales, 4.0, 3.0)
    values = _decode_f64(m).reshape(-1, 2)
    assert np.all(values == np.array([0.25, -0.25]))


def test_ggml36_reorder_is_lossless_and_keeps_the_scalar_apart():
    packed = np.array([(i * 37) % 256 for i in range(64)], dtype=np.uint8).reshape(2, 32)
    scales = np.array([1, 16, 56, 126, 2, 8, 64, 100], dtype=np.uint8).reshape(2, 4)
    m = ck.CheckpointNvfp4Matrix.from_modelopt(packed, scales, 0.125, 7.0)
    wire = m.to_ggml36()
    assert wire.size == 72
    flat_codes, flat_scales = packed.reshape(-1), scales.reshape(-1)
    for i in range(128):
        block = wire[(i // 64) * 36:][:36]
        lane = i % 16
        code = (block[4 + (i % 64 // 16) * 8 + lane % 8] >> (lane // 8 * 4)) & 15
        assert code == (flat_codes[i // 2] >> (i % 2 * 4)) & 15
        assert block[i % 64 // 16] == flat_scales[i // 16]
    back = ck.CheckpointNvfp4Matrix.from_ggml36(2, 64, wire, m.scale)
    assert np.array_equal(back.packed, packed) and np.array_equal(back.scales, scales)
    assert back.scale == m.scale and back.scale.global_scale() == 0.125


def test_ggml36_round_trip_on_random_planes():
    rng = np.random.default_rng(5)
    packed = rng.integers(0, 256, size=(96, 640 // 2), dtype=np.uint8)
    scales = rng.integers(0, 127, size=(96, 640 // 16), dtype=np.uint8)
    m = ck.CheckpointNvfp4Matrix.from_modelopt(packed, scales, 1.0)
    back = ck.CheckpointNvfp4Matrix.from_ggml36(96, 640, m.to_ggml36(), m.scale)
    assert np.array_equal(back.packed, packed) and np.array_equal(back.scales, scales)


def test_invalid_shape_extent_and_scale_are_rejected():
    zeros8, zero1 = np.zeros((1, 8), dtype=np.uint8), np.zeros((1, 1), dtype=np.uint8)
    for w in (0.0, -1.0, float("inf"), float("nan")):
        with pytest.raises(ck.CheckpointError):
            ck.CheckpointNvfp4Matrix.from_compressed_tensors(zeros8, zero1, w, 3.0)
    for scale in (127, 128, 255):
        with pytest.raises(ck.CheckpointError):
            ck.CheckpointNvfp4Matrix.from_modelopt(zeros8, np.array([[scale]], dtype=np.uint8), 1.0, 7.0)
    with pytest.raises(ck.CheckpointError):   # cols = 15
        ck.CheckpointNvfp4Matrix(1, 15, zeros8, zero1, ck.CheckpointNvfp4Scale(ck.MODELOPT, 1.0, 7.0))
    with pytest.raises(ck.CheckpointError):   # shape that overflows
        ck.CheckpointNvfp4Matrix((1 << 63) - 1, 16, np.zeros(0, dtype=np.uint8), np.zeros(0, dtype=np.uint8),
                                 ck.CheckpointNvfp4Scale(ck.MODELOPT, 1.0, 7.0))
    m = ck.CheckpointNvfp4Matrix.from_modelopt(zeros8, zero1, 1.0, 7.0)
    with pytest.raises(ck.CheckpointError):   # K % 64
        m.to_ggml36()
    with pytest.raises(ck.CheckpointError):   # wrong wire extent
        ck.CheckpointNvfp4Matrix.from_ggml36(1, 64, np.zeros(35, dtype=np.uint8), m.scale)
    with pytest.raises(ck.CheckpointError):   # a scalar the kernels cannot take
        ck.CheckpointNvfp4Scale(ck.COMPRESSED_TENSORS, 2.0 ** 40, 1.0).global_scale()
