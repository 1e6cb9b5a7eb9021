"""Pins the CPU oracle to the known-answer vectors of the reference's own unit tests.

Each case names the reference test it restates (paths inside the Augur project).
"""
import numpy as np
import pytest

import oracle


def test_e2m1_table_identity():
    # crates/augur-formats/src/fp4.rs:245-250
    expected = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    for code, value in enumerate(expected):
        assert oracle.decode_e2m1(code) == value
    # code 8 is +0.0 in the table, not -0.0
    assert np.float32(oracle.decode_e2m1(8)).view(np.uint32) == 0


def test_e4m3_boundaries_are_strict():
    # crates/augur-formats/src/fp4.rs:252-261
    assert oracle.decode_e4m3fn(0x38) == 1.0
    assert oracle.decode_e4m3fn(0x7E) == 448.0
    assert oracle.decode_e4m3fn(0xFE) == -448.0
    with pytest.raises(oracle.OracleError) as err:
        oracle.decode_e4m3fn(0x7F)
    assert err.value.code == oracle.NON_FINITE_VALUE
    with pytest.raises(oracle.OracleError):
        oracle.decode_e4m3fn(0xFF)
    # subnormals: m/8 * 2^-6
    assert oracle.decode_e4m3fn(0x01) == 2.0 ** -9
    assert oracle.decode_e4m3fn(0x07) == 7.0 * 2.0 ** -9
    assert oracle.decode_e4m3fn(0x08) == 2.0 ** -6


def test_nvfp4_block_scale_protocol():
    # crates/augur-formats/src/fp4.rs:263-284: qs=0x21, scale 0x38, global 2 -> [1,2,1,2]
    out = oracle.block_decode_ref([0x21] * 8, 0x38, 2.0)
    assert out[:4].tolist() == [1.0, 2.0, 1.0, 2.0]
    assert out.tolist() == [1.0, 2.0] * 8


def test_checkpoint_plane_known_answers():
    # crates/augur-model-qwen35/src/checkpoint_quant.rs:256-279, multiplicative convention
    out = oracle.block_decode_ref([0x72] * 8, 0x38, 2.0)  # codes 2 (1.0) and 7 (6.0), x2
    assert out[:2].tolist() == [2.0, 12.0]
    out = oracle.block_decode_ref([0x72] * 8, 0x38, 0.5)  # the "divide by 2" twin
    assert out[:2].tolist() == [0.5, 3.0]
    out = oracle.block_decode_ref([0xFA] * 8, 0x40, 0.125)  # codes 10 (-1.0), 15 (-6.0); scale 2
    assert out[:2].tolist() == [-0.25, -1.5]
    # :281-288 48x5120 of 0xA2 / 0x38 / divide by 4 -> alternating [0.25, -0.25]
    rows, cols = 48, 5120
    codes = np.full((rows, cols // 2), 0xA2, dtype=np.uint8)
    scales = np.full((rows, cols // 16), 0x38, dtype=np.uint8)
    w = oracle.dequant_planes_f32(codes, scales, 0.25, rows, cols)
    assert np.all(w[:, 0::2] == 0.25) and np.all(w[:, 1::2] == -0.25)


def _m46_case():
    # crates/augur-reference/tests/m46_fp4.rs:11-12,37-50
    activation = ((np.arange(64, dtype=np.float32) - np.float32(31.0)) / np.float32(17.0)).astype(np.float32)
    qs = [[(0x5C + index) & 0xFF] * 8 for index in range(8)]
    scales = [0x30 + index for index in range(8)]
    blocks = oracle.make_blocks(qs, scales, [0.125] * 8)
    return activation, blocks


def test_portable_matches_reference_bit_equal():
    activation, blocks = _m46_case()
    expected = oracle.qmatvec_nvfp4_f32_ref(blocks, 2, 64, activation)
    hot = oracle.repack_nvfp4_tensor_cpu(blocks, 2, 64)
    actual = oracle.qmatvec_nvfp4_f32_cpu_portable(hot, 2, 64, activation)
    assert actual.view(np.uint32).tolist() == expected.view(np.uint32).tolist()
    # independent fp64 evaluation of the same 2x64 case
    e2m1 = oracle.E2M1_VALUES.astype(np.float64)
    for row in range(2):
        total = 0.0
        for block in range(4):
            b = blocks[row * 4 + block]
            scale = oracle.decode_e4m3fn(b.scale_e4m3) * 0.125
            for lane in range(16):
                byte = b.qs[lane // 2]
                nib = (byte & 0xF) if lane % 2 == 0 else (byte >> 4)
                total += e2m1[nib] * scale * float(activation[block * 16 + lane])
        assert abs(float(expected[row]) - total) <= 1e-5 * max(1.0, abs(total))


def test_invalid_scale_and_shapes_fail_closed():
    # crates/augur-reference/tests/m46_fp4.rs:52-65
    bad = oracle.make_blocks([[0] * 8], [0x7F], [1.0])
    with pytest.raises(oracle.OracleError) as err:
        oracle.repack_nvfp4_tensor_cpu(bad, 1, 16)
    assert err.value.code == oracle.NON_FINITE_VALUE
    good = oracle.make_blocks([[0] * 8], [0x38], [1.0])
    with pytest.raises(oracle.OracleError) as err:
        oracle.repack_nvfp4_tensor_cpu(good, 1, 31)
    assert err.value.code == oracle.BAD_WEIGHT_SHAPE
    # validation order of qmatvec_ref (m46_fp4.rs:136-159)
    act = np.zeros(16, dtype=np.float32)
    with pytest.raises(oracle.OracleError) as err:
        oracle.qmatvec_nvfp4_f32_ref(good, 0, 16, act)
    assert err.value.code == oracle.BAD_WEIGHT_SHAPE
    with pytest.raises(oracle.OracleError) as err:
        oracle.qmatvec_nvfp4_f32_ref(good, 1, 16, np.zeros(15, dtype=np.float32))
    assert err.value.code == oracle.BAD_ACTIVATION_LENGTH
    with pytest.raises(oracle.OracleError) as err:
        oracle.qmatvec_nvfp4_f32_ref(good, 1, 16, act, out_len=0)
    assert err.value.code == oracle.BAD_OUTPUT_LENGTH
    with pytest.raises(oracle.OracleError) as err:
        oracle.qmatvec_nvfp4_f32_ref(good, 2, 16, act)
    assert err.value.code == oracle.BAD_WEIGHT_BLOCK_COUNT
    with pytest.raises(oracle.OracleError) as err:
        oracle.qmatvec_nvfp4_f32_ref(bad, 1, 16, act)
    assert err.value.code == oracle.BAD_WEIGHT
    # non-finite global scale is rejected (fp4.rs:112-114)
    inf_block = oracle.make_blocks([[0] * 8], [0x38], [float("inf")])
    with pytest.raises(oracle.OracleError):
        oracle.repack_nvfp4_tensor_cpu(inf_block, 1, 16)


def test_bf16_round_is_rne():
    # crates/augur-model-qwen35/src/reference.rs:819-826
    assert oracle.bf16_round(1.0) == 1.0
    assert oracle.bf16_round(1.0 + 2.0 ** -8) == 1.0            # tie -> even
    assert oracle.bf16_round(1.0 + 3 * 2.0 ** -8) == 1.0 + 2.0 ** -6  # tie -> even (up)
    assert oracle.bf16_round(1.0 + 2.0 ** -8 + 2.0 ** -20) == 1.0 + 2.0 ** -7
    assert np.isinf(oracle.bf16_round(float("inf")))


def test_numpy_restatement_matches_c_exhaustively():
    # every code x every finite positive scale, three global scales
    rows, cols = 127, 16
    codes = np.zeros((rows, cols // 2), dtype=np.uint8)
    for lane in range(8):
        codes[:, lane] = (2 * lane) | ((2 * lane + 1) << 4)
    scales = np.arange(127, dtype=np.uint8).reshape(rows, 1)
    for glob in (1.0 / 448.0, 0.125, 2.0, 1.0):
        a = oracle.dequant_planes_f32(codes, scales, glob, rows, cols)
        b = oracle.dequant_planes_numpy(codes, scales, glob, rows, cols)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_threaded_linear_is_bit_identical_to_serial():
    from augur_v100_b200 import synth
    rows, cols, tokens = 96, 256, 3
    codes, scales, glob = synth.make_weight(0, 99, "w", rows, cols)
    x = synth.make_activation(0, 99, "x", tokens, cols)
    y1, f1 = oracle.linear_bf16(codes, scales, glob, rows, cols, x, threads=1, want_f32=True)
    y4, f4 = oracle.linear_bf16(codes, scales, glob, rows, cols, x, threads=4, want_f32=True)
    assert np.array_equal(y1, y4) and np.array_equal(f1.view(np.uint32), f4.view(np.uint32))
    # and equal to the block-form reference, token by token
    blocks = oracle.planes_to_blocks(codes, scales, glob, rows, cols)
    for token in range(tokens):
        ref = oracle.qmatvec_nvfp4_f32_ref(blocks, rows, cols, synth.bf16_bits_to_f32(x[token]))
        assert np.array_equal(ref.view(np.uint32), f1[token].view(np.uint32))
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x, threads=2)
    assert np.allclose(y64, f1, rtol=1e-4, atol=1e-5)


def test_activation_quantiser_rule():
    # crates/augur-cuda-sys/native/augur_nvfp4_cutlass_sm120.cu:286-311,455-503
    from augur_v100_b200 import synth
    x = np.zeros((1, 16), dtype=np.float32)
    x[0, :8] = [6.0, 3.0, 0.25, 0.75, -0.25, -5.0, 1.25, 0.0]
    bits = synth.f32_to_bf16_bits(x)
    codes, scales = oracle.act_quant(bits, 1, 16, 1.0, terms=1)
    assert scales[0, 0, 0] == 0x38                # amax/6 = 1.0 exactly
    nib = [(codes[0, 0, i // 2] >> (4 * (i % 2))) & 0xF for i in range(8)]
    # ties go to the smaller magnitude, never to -0: 0.25->0, 0.75->0.5, -0.25->+0, -5->-4, 1.25->1
    assert nib == [7, 5, 0, 1, 0, 14, 2, 0]
    # scale is rounded UP: amax 6.1 -> desired 1.0167 -> next E4M3 is 1.125 (0x39)
    x[0, 0] = 6.125
    codes, scales = oracle.act_quant(synth.f32_to_bf16_bits(x), 1, 16, 1.0, terms=1)
    assert scales[0, 0, 0] == 0x39
    # all-zero group -> scale code 0 and zero codes
    codes, scales = oracle.act_quant(np.zeros((1, 16), dtype=np.uint16), 1, 16, 1.0)
    assert scales.sum() == 0 and codes.sum() == 0
    # a residual series converges
    rng = np.random.default_rng(5)
    xb = synth.f32_to_bf16_bits(rng.standard_normal((4, 64)).astype(np.float32))
    xf = synth.bf16_bits_to_f32(xb).astype(np.float64)
    errs = []
    for terms in (1, 2, 3):
        c, s = oracle.act_quant(xb, 4, 64, 2.0 ** -8, terms)
        d = oracle.act_dequant_f64(c, s, 2.0 ** -8, 4, 64, terms)
        errs.append(np.abs(d - xf).max())
    assert errs[0] > errs[1] > errs[2] and errs[2] < 2e-2


def test_rmsnorm_stage_known_answers():
    # all twos, weight one half, no epsilon: mean square 4, scale 1/2, y = 2 * 1/2 * 1/2
    x = np.full((1, 256), 2.0, dtype=np.float32)
    used, y, staged = oracle.rmsnorm_stage(x, np.full(256, 0.5, dtype=np.float32), 0.0)
    assert np.array_equal(used, x) and np.all(y == 0.5) and np.all(staged == 0x3F00)
    # the residual is one F32 add per element, stored back; the result follows the f64 definition closely
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal((3, 512)).astype(np.float32), rng.standard_normal((3, 512)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(512)).astype(np.float32)
    used, y, staged = oracle.rmsnorm_stage(None, w, 1e-6, a, b)
    assert np.array_equal(used, a + b)
    exact = used.astype(np.float64) / np.sqrt((used.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.max(np.abs(y - exact)) <= 4e-7 * np.max(np.abs(exact))
    from augur_v100_b200 import synth
    assert np.array_equal(staged, synth.f32_to_bf16_bits(y))
