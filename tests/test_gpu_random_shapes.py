"""GPU parity on seeded random shapes, through the C ABI: the small-token linear and MLP block on both small-token
kernels (tensor-memory and mma.sync), and the prefill linear (quantiser + GEMM). The hand-picked cases of the other files walk the
kernels' branches one by one; these draw shapes, token counts, magnitudes and global scales at random, so that a
partition or edge that nobody thought of still meets the oracle. A shape the preflight refuses is skipped, not failed.
Bounds as elsewhere: helpers.rel_error <= 2e-2 against the fp64 oracle; the quantiser's planes bit-exact.
"""
import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    plan = host.Plan(stream, max(96 << 20, host.gemm_plan_scratch_bytes()))
    yield {"torch": torch, "host": host, "stream": stream, "plan": plan, "device": torch.device("cuda", 0)}
    plan.close()
    stream.close()


@pytest.mark.parametrize("seed", [11, 12])
def test_small_token_linear_on_random_shapes(ctx, seed):
    host, rng = ctx["host"], np.random.default_rng(seed)
    ran = 0
    for case in range(12):
        rows, cols = int(rng.integers(1, 65)) * 128, int(rng.integers(1, 130)) * 64
        tokens, scale = int(rng.integers(1, 9)), float(2.0 ** rng.integers(-12, 13))
        codes, scales, glob = synth.make_weight(seed * 100 + case, 77, "w", rows, cols)
        x = (rng.standard_normal((tokens, cols)) * scale).astype(np.float32)
        if case % 4 == 0:
            x[:, rng.integers(0, cols)] *= 300.0     # an outlier channel: far above the sample the anchors come from
        x_bits = synth.f32_to_bf16_bits(x)
        weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols, codes, scales, glob)
        try:
            projection = host.Nvfp4Sm100TcProjection.bind(ctx["plan"], weight, torch_bf16_from_bits(x_bits, ctx["device"]))
        except host.CudaRuntimeError:
            continue
        for _ in range(2):      # the second launch finds the plan's counters as the first left them
            projection.submit_for_plan()
        ctx["stream"].synchronize()
        assert ctx["plan"].device_status() == 0, (rows, cols, tokens, hex(ctx["plan"].device_status()))
        y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
        error = rel_error(bits_from_torch_bf16(projection.out), y64)
        assert error <= TOLERANCE, (rows, cols, tokens, scale, error)
        ran += 1
    assert ran >= 8


@pytest.mark.parametrize("seed", [21, 22])
def test_one_launch_mlp_block_on_random_shapes(ctx, seed):
    host, rng = ctx["host"], np.random.default_rng(seed)
    ran = 0
    for case in range(5):
        # up to 330 x 128 intermediate columns: more gate|up tiles than twice the CTAs takes the two-wave program
        hidden, inter = int(rng.integers(1, 25)) * 128, int(rng.integers(1, 70 if case else 330)) * 128
        tokens = int(rng.integers(1, 9))
        gate = synth.make_weight(seed * 100 + case, 78, "gate", inter, hidden)
        up = synth.make_weight(seed * 100 + case, 78, "up", inter, hidden)
        down = synth.make_weight(seed * 100 + case, 78, "down", hidden, inter)
        x_bits = synth.f32_to_bf16_bits((rng.standard_normal((tokens, hidden)) * 4.0).astype(np.float32))
        gate_up_weight = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
        down_weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
        plan = host.Plan(ctx["stream"], host.mlp_tc_scratch_bytes(hidden, inter))
        try:
            try:
                program = host.Nvfp4Sm100TcFfnProgram.bind(plan, gate_up_weight, down_weight, torch_bf16_from_bits(x_bits, ctx["device"]))
            except host.CudaRuntimeError:
                continue
            for _ in range(3):
                program.submit_for_plan()
            ctx["stream"].synchronize()
            assert plan.device_status() == 0, (hidden, inter, tokens, hex(plan.device_status()))
            h64, _ = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=oracle.max_threads())
            h_bits = bits_from_torch_bf16(program.intermediate)
            assert rel_error(h_bits, h64) <= TOLERANCE, (hidden, inter, tokens)
            y64 = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=oracle.max_threads())
            assert rel_error(bits_from_torch_bf16(program.out), y64) <= TOLERANCE, (hidden, inter, tokens)
            ran += 1
        finally:
            plan.close()
    assert ran >= 3


@pytest.mark.parametrize("seed", [41, 42])
def test_mma_sync_linear_and_mlp_block_on_random_shapes(ctx, seed):
    host, rng = ctx["host"], np.random.default_rng(seed)
    ran = 0
    for case in range(10):
        rows, cols = int(rng.integers(1, 260)) * 32, int(rng.integers(1, 65)) * 128
        tokens, scale = int(rng.integers(1, 9)), float(2.0 ** rng.integers(-12, 13))
        codes, scales, glob = synth.make_weight(seed * 100 + case, 80, "w", rows, cols)
        x_bits = synth.f32_to_bf16_bits((rng.standard_normal((tokens, cols)) * scale).astype(np.float32))
        weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
        try:
            projection = host.Nvfp4Sm100Projection.bind(ctx["plan"], weight, torch_bf16_from_bits(x_bits, ctx["device"]))
        except host.CudaRuntimeError:
            continue
        for _ in range(2):
            projection.submit_for_plan()
        ctx["stream"].synchronize()
        assert ctx["plan"].device_status() == 0, (rows, cols, tokens, hex(ctx["plan"].device_status()))
        y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
        error = rel_error(bits_from_torch_bf16(projection.out), y64)
        assert error <= TOLERANCE, (rows, cols, tokens, scale, error)
        ran += 1
    for case in range(4):
        hidden, inter, tokens = int(rng.integers(1, 25)) * 128, int(rng.integers(1, 70)) * 128, int(rng.integers(1, 9))
        gate = synth.make_weight(seed * 100 + case, 81, "gate", inter, hidden)
        up = synth.make_weight(seed * 100 + case, 81, "up", inter, hidden)
        down = synth.make_weight(seed * 100 + case, 81, "down", hidden, inter)
        x_bits = synth.f32_to_bf16_bits((rng.standard_normal((tokens, hidden)) * 4.0).astype(np.float32))
        gate_up_weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM_PAIR, inter, hidden,
                                                                       gate[0], gate[1], gate[2], up[0], up[1], up[2])
        down_weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, hidden, inter, *down)
        plan = host.Plan(ctx["stream"], host.mlp_scratch_bytes(hidden, inter))
        try:
            try:
                program = host.Nvfp4Sm100FfnProgram.bind(plan, gate_up_weight, down_weight, torch_bf16_from_bits(x_bits, ctx["device"]))
            except host.CudaRuntimeError:
                continue
            for _ in range(2):
                program.submit_for_plan()
            ctx["stream"].synchronize()
            assert plan.device_status() == 0, (hidden, inter, tokens, hex(plan.device_status()))
            h64, _ = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=oracle.max_threads())
            h_bits = bits_from_torch_bf16(program.intermediate)
            assert rel_error(h_bits, h64) <= TOLERANCE, (hidden, inter, tokens)
            y64 = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=oracle.max_threads())
            assert rel_error(bits_from_torch_bf16(program.out), y64) <= TOLERANCE, (hidden, inter, tokens)
            ran += 1
        finally:
            plan.close()
    assert ran >= 10


@pytest.mark.parametrize("seed", [31, 32])
def test_prefill_linear_on_random_shapes(ctx, seed):
    host, rng = ctx["host"], np.random.default_rng(seed)
    ran = 0
    for case in range(8):
        rows, cols = int(rng.integers(1, 41)) * 128, int(rng.integers(1, 60)) * 64
        tokens, terms = int(rng.integers(1, 700)), int(rng.integers(1, 4))
        glob = float(rng.choice([2.0 ** -8, 0.01, 0.3, 1.0]))
        w_codes, w_scales, g_w = synth.make_weight(seed * 100 + case, 79, "w", rows, cols)
        x_bits = synth.f32_to_bf16_bits((rng.standard_normal((tokens, cols)) * rng.choice([0.05, 1.0, 20.0])).astype(np.float32))
        weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols, w_codes, w_scales, g_w)
        try:
            linear = host.Nvfp4Sm100PrefillLinear.bind(ctx["plan"], weight, torch_bf16_from_bits(x_bits, ctx["device"]), terms=terms,
                                                       activation_global_scale=glob)
        except host.CudaRuntimeError:
            continue
        for _ in range(2):
            linear.submit_for_plan()
        ctx["stream"].synchronize()
        assert ctx["plan"].device_status() == 0, (rows, cols, tokens, terms, hex(ctx["plan"].device_status()))
        codes, scales = linear.staged_planes()
        want_codes, want_scales = oracle.act_quant(x_bits, tokens, cols, glob, terms)
        assert np.array_equal(scales, want_scales) and np.array_equal(codes, want_codes), (rows, cols, tokens, terms, glob)
        a64 = oracle.act_dequant_f64(codes, scales, glob, tokens, cols, terms)
        y64 = oracle.linear_f64_xf64(w_codes, w_scales, g_w, rows, cols, a64, threads=oracle.max_threads())
        error = rel_error(bits_from_torch_bf16(linear.out), y64)
        assert error <= TOLERANCE, (rows, cols, tokens, terms, glob, error)
        ran += 1
    assert ran >= 6
