"""The CUDA path against the committed golden fixtures (no oracle code runs here)."""
import os

import numpy as np
import pytest

from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, rms_error, torch_bf16_from_bits

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_golden.npz"))


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    plan = host.Plan(stream, 8 << 20)
    yield {"torch": torch, "host": host, "stream": stream, "plan": plan, "device": torch.device("cuda", 0)}
    plan.close()
    stream.close()


def test_golden_dequant_and_linear(ctx):
    host = ctx["host"]
    rows, cols = 96, 384
    glob = float(GOLDEN["lin_global"])
    for layout in (abi.LAYOUT_STREAM, abi.LAYOUT_TCGEN05):
        w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], layout, rows, cols, GOLDEN["lin_codes"],
                                                          GOLDEN["lin_scales"], glob)
        assert np.array_equal(w.dequant_f32().cpu().numpy().view(np.uint32), GOLDEN["lin_dequant_bits"])
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, GOLDEN["lin_codes"],
                                                      GOLDEN["lin_scales"], glob)
    proj = host.Nvfp4Sm100Projection.bind(ctx["plan"], w, torch_bf16_from_bits(GOLDEN["lin_x"], ctx["device"]))
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    got = bits_from_torch_bf16(proj.out)
    assert rel_error(got, GOLDEN["lin_y_f64"]) <= TOLERANCE
    assert rel_error(got, GOLDEN["lin_y_f32_bits"].view(np.float32).astype(np.float64)) <= TOLERANCE


def test_golden_reference_2x64_case(ctx):
    # crates/augur-reference/tests/m46_fp4.rs:37-50 needs f32 activations and a 2-row weight; the ABI takes
    # BF16 activations and 32-row groups, so the case is embedded: rows 0..1 of a 32 x 128 weight whose other
    # rows and columns are zero, activations rounded to BF16 (the expected value is recomputed for that input
    # by the same oracle in make_golden; here only the embedding is checked against the stored f32 result).
    host = ctx["host"]
    codes = np.zeros((32, 64), dtype=np.uint8)
    scales = np.full((32, 8), 0x38, dtype=np.uint8)
    for index in range(8):
        row, block = divmod(index, 4)
        codes[row, block * 8:(block + 1) * 8] = (0x5C + index) & 0xFF
        scales[row, block] = 0x30 + index
    act = ((np.arange(64, dtype=np.float32) - np.float32(31.0)) / np.float32(17.0)).astype(np.float32)
    x = np.zeros((1, 128), dtype=np.float32)
    x[0, :64] = act
    x_bits = synth.f32_to_bf16_bits(x)
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, 32, 128, codes, scales, 0.125)
    proj = host.Nvfp4Sm100Projection.bind(ctx["plan"], w, torch_bf16_from_bits(x_bits, ctx["device"]),
                                          epilogue=abi.EPILOGUE_LINEAR_F32)
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    got = proj.out.cpu().numpy()[0, :2].astype(np.float64)
    want = GOLDEN["m46_expected_bits"].view(np.float32).astype(np.float64)
    # BF16 rounding of the activations moves each term by at most 2^-9 relative
    assert np.all(np.abs(got - want) <= 2.0 ** -8 * np.abs(want) + 1e-3)
    assert np.all(proj.out.cpu().numpy()[0, 2:] == 0.0)


def test_golden_mlp(ctx):
    host = ctx["host"]
    hidden, inter = 128, 256
    g = synth.GLOBAL_SCALE
    gate_up = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(
        ctx["stream"], abi.LAYOUT_STREAM_PAIR, inter, hidden, GOLDEN["mlp_gate_codes"], GOLDEN["mlp_gate_scales"], g,
        GOLDEN["mlp_up_codes"], GOLDEN["mlp_up_scales"], g)
    down = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, hidden, inter,
                                                         GOLDEN["mlp_down_codes"], GOLDEN["mlp_down_scales"], g)
    program = host.Nvfp4Sm100FfnProgram.bind(ctx["plan"], gate_up, down, torch_bf16_from_bits(GOLDEN["mlp_x"], ctx["device"]))
    program.submit_for_plan()
    ctx["stream"].synchronize()
    assert rel_error(bits_from_torch_bf16(program.intermediate), GOLDEN["mlp_h_f64"]) <= TOLERANCE
    assert rms_error(bits_from_torch_bf16(program.out), GOLDEN["mlp_y_f64"]) <= TOLERANCE


def test_golden_activation_quantiser(ctx):
    host, torch = ctx["host"], ctx["torch"]
    weight = host.Nvfp4Sm100Weight(ctx["stream"], abi.LAYOUT_TCGEN05, 128, 64,
                                   torch.zeros(host.repack_extent(abi.LAYOUT_TCGEN05, 128, 64), dtype=torch.uint8,
                                               device=ctx["device"]), 1.0)
    lin = host.Nvfp4Sm100PrefillLinear.bind(ctx["plan"], weight, torch_bf16_from_bits(GOLDEN["quant_x"], ctx["device"]),
                                            terms=2, activation_global_scale=2.0 ** -8)
    lin.submit_quant()
    ctx["stream"].synchronize()
    codes, scales = lin.staged_planes()
    assert np.array_equal(codes, GOLDEN["quant_codes"]) and np.array_equal(scales, GOLDEN["quant_scales"])
