"""GPU parity at the exact shapes the benchmark times.

Configuration 1: the whole MLP block 5120 -> 2 x 17408 -> 5120 at 1 and 8 token rows (the 7-or-8 row-group
split of the gate|up launch and the 4 k-slabs x 37 CTAs of the down launch only exist at this size).
Configuration 2: the 4096-token GEMMs on 17408 x 5120 and 5120 x 17408 weights, one and three activation
terms, on a plan that has room for the leftover-tile hand-over (the down shape cuts its last 24 tiles along
k). Every output column of 64 sampled token rows is compared with the CPU oracle, as the reference's own
full-shape component tests do (crates/augur-backend/src/cuda_nvfp4_sm70.rs:745-867).

Tolerances, all stated here:
* a GEMM output against the fp64 oracle fed the same inputs: helpers.rel_error <= 2e-2
  (max |y - y64| / max(|y64|, 1e-3 rms));
* the three-term GEMM against the oracle fed the BF16 activations (the reference semantics): the
  quantisation error of the activations is spread over all outputs, so it is measured against the rms,
  max |y - y64| / rms <= 2e-2, and the rel_error figure is printed beside it;
* a two-GEMM chain against the independently rounded oracle chain: max |y - y64| / rms <= 2e-2.
"""
import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, rms_error, torch_bf16_from_bits

pytestmark = pytest.mark.gpu

HIDDEN, INTER = 5120, 17408


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    yield {"torch": torch, "host": host, "stream": stream, "device": torch.device("cuda", 0)}
    stream.close()


@pytest.fixture(scope="module")
def mlp_weights(ctx):
    host = ctx["host"]
    gate = synth.make_weight(0, 1, "gate", INTER, HIDDEN)
    up = synth.make_weight(0, 1, "up", INTER, HIDDEN)
    down = synth.make_weight(0, 1, "down", HIDDEN, INTER)
    gate_up = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM_PAIR, INTER, HIDDEN, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, HIDDEN, INTER, *down)
    return gate, up, down, gate_up, down_w


@pytest.mark.parametrize("tokens", [1, 8])
def test_config1_full_mlp_block(ctx, mlp_weights, tokens):
    host = ctx["host"]
    gate, up, down, gate_up, down_w = mlp_weights
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(tokens).standard_normal((tokens, HIDDEN)).astype(np.float32) * 8.0)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    plan = host.Plan(ctx["stream"], host.mlp_scratch_bytes(HIDDEN, INTER))
    try:
        program = host.Nvfp4Sm100FfnProgram.bind(plan, gate_up, down_w, x)
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert plan.device_status() == 0
        first = bits_from_torch_bf16(program.out).copy()
        h_bits = bits_from_torch_bf16(program.intermediate)
        threads = oracle.max_threads()
        h64, y64 = oracle.mlp_f64(gate, up, down, HIDDEN, INTER, x_bits, threads=threads)
        # each GEMM of the block against the fp64 oracle on the inputs it actually read
        assert rel_error(h_bits, h64) <= TOLERANCE
        y64_from_h = oracle.linear_f64(down[0], down[1], down[2], HIDDEN, INTER, h_bits, threads=threads)
        assert rel_error(first, y64_from_h) <= TOLERANCE
        # and the chain as a whole
        assert rms_error(first, y64) <= TOLERANCE
        # a second submit gives the same bits (fixed-order combination, counters left clean)
        program.out.zero_()
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert np.array_equal(bits_from_torch_bf16(program.out), first)
    finally:
        plan.close()


@pytest.mark.parametrize("rows,cols", [(INTER, HIDDEN), (HIDDEN, INTER)], ids=["17408x5120", "5120x17408"])
def test_config2_prefill_gemm_full_size(ctx, rows, cols):
    host, torch = ctx["host"], ctx["torch"]
    tokens, sampled = 4096, 64
    codes, scales, glob = synth.make_weight(0, 2, "w", rows, cols)
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols, codes, scales, glob)
    x_bits = synth.make_activation(0, 2, "x", tokens, cols)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    pick = np.sort(np.random.default_rng(5).choice(tokens, size=sampled, replace=False))
    pick[0], pick[-1] = 0, tokens - 1
    threads = oracle.max_threads()
    y64_bf16_activations = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits[pick], threads=threads)
    plan = host.Plan(ctx["stream"], host.gemm_plan_scratch_bytes())   # room for the leftover-tile hand-over
    try:
        for terms in (1, 3):
            g_a = 2.0 ** -8
            lin = host.Nvfp4Sm100PrefillLinear.bind(plan, weight, x, terms=terms, activation_global_scale=g_a)
            lin.submit_for_plan()
            ctx["stream"].synchronize()
            assert plan.device_status() == 0
            got = bits_from_torch_bf16(lin.out[torch.from_numpy(pick).to(ctx["device"])])
            a_codes, a_scales = lin.staged_planes()
            a64 = oracle.act_dequant_f64(np.ascontiguousarray(a_codes[:, pick]), np.ascontiguousarray(a_scales[:, pick]),
                                         g_a, sampled, cols, terms)
            y64 = oracle.linear_f64_xf64(codes, scales, glob, rows, cols, a64, threads=threads)
            # the kernel itself: fp64 oracle fed the very activations the quantiser staged
            assert rel_error(got, y64) <= TOLERANCE, terms
            if terms == 3:
                # the path as a whole against the reference semantics (BF16 activations)
                spread = rms_error(got, y64_bf16_activations)
                print(f"{rows}x{cols} three terms vs BF16-activation oracle: max|err|/rms {spread:.3e}, "
                      f"rel_error {rel_error(got, y64_bf16_activations):.3e}")
                assert spread <= TOLERANCE
            del lin
    finally:
        plan.close()
