"""GPU parity of the small-token linear on the tensor-memory path (`gemv_tc`), through the C ABI.

Ordered from the smallest exercise of the instruction to the benchmark's shapes, so that a failure localises:
one MMA -> four MMAs of one stage -> several stages -> ring wrap -> several row tiles -> k slabs with the
hand-over through plan scratch -> configuration 0 at full size.
Bound of every case: helpers.rel_error <= 2e-2 against the fp64 oracle fed the BF16 activations, and within
2^-6 (same denominator) of bf16_round(sequential f32): two BF16 roundings of sums whose f32 accumulation
orders differ (the tensor core's and the reference's strictly sequential one).
"""
import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, rel_error_f32, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    plan = host.Plan(stream, 64 << 20)
    yield {"torch": torch, "host": host, "stream": stream, "plan": plan, "device": torch.device("cuda", 0)}
    plan.close()
    stream.close()


def _case(ctx, rows, cols, tokens, seed, epilogue=abi.EPILOGUE_LINEAR_BF16, x_bits=None, scale=1.0):
    host = ctx["host"]
    codes, scales, glob = synth.make_weight(seed, 90, "w", rows, cols)
    if x_bits is None:
        x = synth.bf16_bits_to_f32(synth.make_activation(seed, 90, "x", tokens, cols)) * np.float32(scale)
        x_bits = synth.f32_to_bf16_bits(x)
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols, codes, scales, glob)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    proj = host.Nvfp4Sm100TcProjection.bind(ctx["plan"], w, x, epilogue=epilogue)
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0, hex(ctx["plan"].device_status())
    return codes, scales, glob, x_bits, proj


def _check(ctx, rows, cols, tokens, seed, scale=1.0):
    codes, scales, glob, x_bits, proj = _case(ctx, rows, cols, tokens, seed, scale=scale)
    got = bits_from_torch_bf16(proj.out)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    err = rel_error(got, y64)
    assert err <= TOLERANCE, err
    ref_bits = oracle.linear_bf16(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    a = synth.bf16_bits_to_f32(got).astype(np.float64)
    b = synth.bf16_bits_to_f32(ref_bits).astype(np.float64).reshape(a.shape)
    assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3 * np.sqrt(np.mean(b * b)))) <= 2.0 ** -6
    return err


def test_single_mma(ctx):
    _check(ctx, rows=128, cols=64, tokens=8, seed=1)


def test_one_stage_four_mmas(ctx):
    _check(ctx, rows=128, cols=256, tokens=8, seed=2)


def test_several_stages_and_ragged_last_stage(ctx):
    _check(ctx, rows=128, cols=1216, tokens=8, seed=3)      # 4.75 stages


def test_fewer_tokens(ctx):
    for tokens in (1, 3, 5):
        _check(ctx, rows=256, cols=512, tokens=tokens, seed=4 + tokens)


def test_ring_wrap_and_row_tiles(ctx):
    _check(ctx, rows=2560, cols=2048, tokens=8, seed=5)     # 8 stages per part, 20 tiles cut along k


def test_k_parts_hand_over_through_scratch(ctx):
    _check(ctx, rows=256, cols=5120, tokens=8, seed=6)      # 2 tiles, 20 stages: 10 parts each
    _check(ctx, rows=384, cols=17408, tokens=8, seed=7)     # 3 tiles, 68 stages: 16 parts each
    # a second launch on the same plan finds the counters clean
    _check(ctx, rows=384, cols=17408, tokens=8, seed=7)


def test_activation_magnitudes(ctx):
    # tiny, huge and mixed magnitudes: the split's per-token power-of-two scale follows the row
    for scale in (2.0 ** -60, 1e-3, 8.0, 1e4, 2.0 ** 60):
        _check(ctx, rows=128, cols=1024, tokens=8, seed=8, scale=scale)
    rows, cols, tokens = 128, 1024, 8
    x = np.random.default_rng(9).standard_normal((tokens, cols)).astype(np.float32)
    x[0] = 0.0
    x[1, ::7] *= 1e4         # outlier channels
    x[2, :16] *= 1e-6        # one group far below the rest of its row
    x[3, 5] = 3e4
    x[4, 700] = 1e5          # beyond what the first 256 elements of the row suggest: the anchors are found again
    x[5, 900] = np.inf       # a row with a non-finite element gives NaN
    codes, scales, glob, x_bits, proj = _case(ctx, rows, cols, tokens, 10, x_bits=synth.f32_to_bf16_bits(x))
    got = bits_from_torch_bf16(proj.out).reshape(tokens, rows)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=4)
    for t in range(tokens):
        if t != 5:
            assert rel_error(got[t], y64[t]) <= TOLERANCE, t
    assert np.all(got[0] & 0x7FFF == 0)
    assert np.all((got[5] & 0x7FFF) > 0x7F80)


def test_f32_epilogue(ctx):
    rows, cols, tokens = 256, 2176, 8
    codes, scales, glob, x_bits, proj = _case(ctx, rows, cols, tokens, 11, epilogue=abi.EPILOGUE_LINEAR_F32)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=4)
    # the eight-digit split of the activations and f32 accumulation: far inside the BF16 rounding step (2^-9)
    assert rel_error_f32(proj.out.cpu().numpy(), y64) <= 2e-3


def test_swiglu_epilogue(ctx):
    host = ctx["host"]
    inter, hidden, tokens = 512, 1024, 8
    gate = synth.make_weight(12, 90, "gate", inter, hidden)
    up = synth.make_weight(12, 90, "up", inter, hidden)
    up = (up[0], up[1], float(np.float32(up[2]) * np.float32(1.5)))
    weight = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(12).standard_normal((tokens, hidden)).astype(np.float32) * 8.0)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    proj = host.Nvfp4Sm100TcProjection.bind(ctx["plan"], weight, x, epilogue=abi.EPILOGUE_SWIGLU_BF16)
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0
    down = synth.make_weight(12, 90, "down", hidden, inter)
    h64, _ = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=4)
    assert rel_error(bits_from_torch_bf16(proj.out), h64) <= TOLERANCE


def test_config0_full_size(ctx):
    rows, cols, tokens = 17408, 5120, 8
    codes, scales, glob = synth.make_weight(0, 0, "weight", rows, cols)
    x_bits = synth.make_activation(0, 0, "activation", tokens, cols)
    host = ctx["host"]
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols, codes, scales, glob)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    proj = host.Nvfp4Sm100TcProjection.bind(ctx["plan"], w, x)
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0
    first = bits_from_torch_bf16(proj.out).copy()
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    assert rel_error(first, y64) <= TOLERANCE
    proj.out.zero_()
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    assert np.array_equal(bits_from_torch_bf16(proj.out), first)    # fixed-order sums: the same bits again


@pytest.mark.parametrize("hidden,inter,tokens", [(256, 512, 8), (1024, 2176, 8), (640, 1152, 1), (5120, 2176, 5)])
def test_mlp_block_as_one_launch(ctx, hidden, inter, tokens):
    host = ctx["host"]
    gate = synth.make_weight(20, 91, "gate", inter, hidden)
    up = synth.make_weight(20, 91, "up", inter, hidden)
    up = (up[0], up[1], float(np.float32(up[2]) * np.float32(1.5)))
    down = synth.make_weight(20, 91, "down", hidden, inter)
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(21).standard_normal((tokens, hidden)).astype(np.float32) * 8.0)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    plan = host.Plan(ctx["stream"], host.mlp_tc_scratch_bytes(hidden, inter))
    try:
        program = host.Nvfp4Sm100TcFfnProgram.bind(plan, gate_up_w, down_w, x)
        before = host.launch_count()
        for _ in range(3):                     # the barrier words and row maxima are left clean by every launch
            program.submit_for_plan()
        ctx["stream"].synchronize()
        assert plan.device_status() == 0, hex(plan.device_status())
        assert host.launch_count() - before == 3          # one launch per block
        h64, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=oracle.max_threads())
        h_bits = bits_from_torch_bf16(program.intermediate)
        assert rel_error(h_bits, h64) <= TOLERANCE
        y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=oracle.max_threads())
        assert rel_error(bits_from_torch_bf16(program.out), y64_from_h) <= TOLERANCE
    finally:
        plan.close()


@pytest.mark.parametrize("tokens", [1, 8])
def test_config1_full_mlp_block_as_one_launch(ctx, tokens):
    host = ctx["host"]
    hidden, inter = 5120, 17408
    gate = synth.make_weight(0, 1, "gate", inter, hidden)
    up = synth.make_weight(0, 1, "up", inter, hidden)
    down = synth.make_weight(0, 1, "down", hidden, inter)
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(tokens).standard_normal((tokens, hidden)).astype(np.float32) * 8.0)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    plan = host.Plan(ctx["stream"], host.mlp_tc_scratch_bytes(hidden, inter))
    try:
        program = host.Nvfp4Sm100TcFfnProgram.bind(plan, gate_up_w, down_w, x)
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert plan.device_status() == 0, hex(plan.device_status())
        first = bits_from_torch_bf16(program.out).copy()
        threads = oracle.max_threads()
        h64, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=threads)
        h_bits = bits_from_torch_bf16(program.intermediate)
        assert rel_error(h_bits, h64) <= TOLERANCE
        y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=threads)
        assert rel_error(first, y64_from_h) <= TOLERANCE
        program.out.zero_()
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert np.array_equal(bits_from_torch_bf16(program.out), first)
    finally:
        plan.close()


def test_more_gate_up_tiles_than_ctas_runs_in_two_waves(ctx):
    # 320 gate|up tiles on at most 2 CTAs per SM: the first wave's outputs are split while the second wave streams,
    # and the down product is cut into the k range each wave feeds (separate scales, partial sums added in f32)
    host = ctx["host"]
    hidden, inter, tokens = 256, 20480, 8
    gate = synth.make_weight(30, 92, "gate", inter, hidden)
    up = synth.make_weight(30, 92, "up", inter, hidden)
    down = synth.make_weight(30, 92, "down", hidden, inter)
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(31).standard_normal((tokens, hidden)).astype(np.float32) * 4.0)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    plan = host.Plan(ctx["stream"], host.mlp_tc_scratch_bytes(hidden, inter))
    try:
        program = host.Nvfp4Sm100TcFfnProgram.bind(plan, gate_up_w, down_w, x)
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert plan.device_status() == 0, hex(plan.device_status())
        first = bits_from_torch_bf16(program.out).copy()
        threads = oracle.max_threads()
        h64, _ = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=threads)
        h_bits = bits_from_torch_bf16(program.intermediate)
        assert rel_error(h_bits, h64) <= TOLERANCE
        y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=threads)
        assert rel_error(first, y64_from_h) <= TOLERANCE
        for _ in range(2):
            program.out.zero_()
            program.submit_for_plan()
            ctx["stream"].synchronize()
            assert np.array_equal(bits_from_torch_bf16(program.out), first)
        assert plan.device_status() == 0
    finally:
        plan.close()


def test_programs_of_different_shapes_share_a_plan(ctx):
    # the counters, maxima and per-CTA words a launch leaves in the plan are ready for whatever launch comes next:
    # a linear in k parts, the MLP block, a linear in whole tiles, in turn, each repeating its own bits
    host = ctx["host"]
    hidden, inter, tokens = 1024, 2176, 8
    gate = synth.make_weight(40, 93, "gate", inter, hidden)
    up = synth.make_weight(40, 93, "up", inter, hidden)
    down = synth.make_weight(40, 93, "down", hidden, inter)
    wide = synth.make_weight(41, 93, "wide", 128 * 300, 256)
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    wide_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, 128 * 300, 256, *wide)
    rng = np.random.default_rng(42)
    x = torch_bf16_from_bits(synth.f32_to_bf16_bits(rng.standard_normal((tokens, hidden)).astype(np.float32)), ctx["device"])
    x_inter = torch_bf16_from_bits(synth.f32_to_bf16_bits(rng.standard_normal((tokens, inter)).astype(np.float32)), ctx["device"])
    x_narrow = torch_bf16_from_bits(synth.f32_to_bf16_bits(rng.standard_normal((3, 256)).astype(np.float32)), ctx["device"])
    need = max(host.mlp_tc_scratch_bytes(hidden, inter), host.gemv_tc_scratch_bytes(128 * 300, 256))
    plan = host.Plan(ctx["stream"], need)
    try:
        programs = [host.Nvfp4Sm100TcProjection.bind(plan, down_w, x_inter),          # 8 tiles in k parts
                    host.Nvfp4Sm100TcFfnProgram.bind(plan, gate_up_w, down_w, x),     # the block
                    host.Nvfp4Sm100TcProjection.bind(plan, wide_w, x_narrow)]         # 300 whole tiles, 3 token rows
        firsts = []
        for program in programs:
            program.submit_for_plan()
            ctx["stream"].synchronize()
            firsts.append(bits_from_torch_bf16(program.out).copy())
        for order in ((1, 0, 2), (2, 1, 1, 0), (0, 2, 1)):
            for index in order:
                programs[index].out.zero_()
                programs[index].submit_for_plan()
            ctx["stream"].synchronize()
            assert plan.device_status() == 0, hex(plan.device_status())
            for index in set(order):
                assert np.array_equal(bits_from_torch_bf16(programs[index].out), firsts[index]), index
    finally:
        plan.close()


def test_one_gate_up_tile_far_larger_than_the_others(ctx):
    # the anchors of the intermediate come from every CTA's maxima: one tile whose outputs are far larger than all
    # others' (block scales times 8 on its gate and up rows) sets them for everybody, and the other tiles' groups
    # get small block scales. Same bound as every other case; the bits repeat.
    host = ctx["host"]
    hidden, inter, tokens = 256, 1536, 8
    gate = list(synth.make_weight(50, 94, "gate", inter, hidden))
    up = list(synth.make_weight(50, 94, "up", inter, hidden))
    down = synth.make_weight(50, 94, "down", hidden, inter)
    for plane in (gate, up):
        scales = plane[1].copy().reshape(inter, hidden // 16)
        tile = scales[5 * 64:6 * 64]
        scales[5 * 64:6 * 64] = np.where(tile > 0, np.minimum(tile.astype(np.int32) + 24, 0x7E), tile).astype(scales.dtype)   # E4M3 exponent + 3
        plane[1] = scales.reshape(plane[1].shape)
    gate, up = tuple(gate), tuple(up)
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(51).standard_normal((tokens, hidden)).astype(np.float32))
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    plan = host.Plan(ctx["stream"], host.mlp_tc_scratch_bytes(hidden, inter))
    try:
        program = host.Nvfp4Sm100TcFfnProgram.bind(plan, gate_up_w, down_w, x)
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert plan.device_status() == 0, hex(plan.device_status())
        first = bits_from_torch_bf16(program.out).copy()
        threads = oracle.max_threads()
        h64, _ = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=threads)
        ratio = np.abs(h64[:, 5 * 64:6 * 64]).max() / np.abs(np.delete(h64, np.s_[5 * 64:6 * 64], axis=1)).max()
        assert ratio > 32.0, ratio            # the case is what it claims to be
        h_bits = bits_from_torch_bf16(program.intermediate)
        assert rel_error(h_bits, h64) <= TOLERANCE
        y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=threads)
        assert rel_error(first, y64_from_h) <= TOLERANCE
        program.out.zero_()
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert np.array_equal(bits_from_torch_bf16(program.out), first)
        assert plan.device_status() == 0
    finally:
        plan.close()
