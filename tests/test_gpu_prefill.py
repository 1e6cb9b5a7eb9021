"""GPU parity of the prefill path: activation quantiser and tcgen05 block-scaled GEMM."""
from ctypes import byref

import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, rms_error, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    plan = host.Plan(stream, 1 << 20)
    yield {"torch": torch, "host": host, "stream": stream, "plan": plan, "device": torch.device("cuda", 0)}
    plan.close()
    stream.close()


@pytest.mark.parametrize("tokens,cols,terms,glob", [(128, 64, 1, 1.0), (128, 256, 2, 2.0 ** -8), (256, 2176, 3, 0.01),
                                                    (384, 5120, 1, 2.0 ** -8), (5, 128, 2, 0.5), (200, 320, 3, 2.0 ** -8)])
def test_activation_quantiser_is_bit_exact(ctx, tokens, cols, terms, glob):
    host, torch = ctx["host"], ctx["torch"]
    rng = np.random.default_rng(tokens + cols)
    x = rng.standard_normal((tokens, cols)).astype(np.float32)
    x[0, :16] = 0.0                       # an all-zero group
    x[1, 16:32] *= 1e-6                   # below the smallest scale
    x[2, 32:48] *= 1e4                    # saturates the largest scale when glob is small
    x[3, :8] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25]   # ties (after scaling by an exact scale)
    x[3, 8:16] = [-0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 6.0, -6.0]
    x[4, 3] = -1e-4                       # a negative quotient that rounds to zero: code 0, not "minus zero"
    x[4, 16:24] = [np.nan, 1.0, -2.0, 0.3, np.nan, 6.0, -0.1, 0.0]   # a NaN quotient clamps to -6; the maximum leaves NaNs out
    x[4, 40] = np.inf                     # largest scale, code +6, every later residual infinite
    x[4, 50] = -np.inf
    x_bits = synth.f32_to_bf16_bits(x)
    weight = host.Nvfp4Sm100Weight(ctx["stream"], abi.LAYOUT_TCGEN05, 128, cols,
                                   torch.zeros(host.repack_extent(abi.LAYOUT_TCGEN05, 128, cols), dtype=torch.uint8,
                                               device=ctx["device"]), 1.0)
    lin = host.Nvfp4Sm100PrefillLinear.bind(ctx["plan"], weight, torch_bf16_from_bits(x_bits, ctx["device"]),
                                            terms=terms, activation_global_scale=glob)
    lin.submit_quant()
    ctx["stream"].synchronize()
    codes, scales = lin.staged_planes()
    want_codes, want_scales = oracle.act_quant(x_bits, tokens, cols, glob, terms)
    assert np.array_equal(scales, want_scales)
    assert np.array_equal(codes, want_codes)


@pytest.mark.parametrize("glob", [0.01, 0.37, 3.0e-3, 1.0 / 3.0, 7.5])
def test_activation_quantiser_is_bit_exact_for_any_global_scale(ctx, glob):
    """A global scale that is not a power of two makes every divisor a full-width significand: level * divisor is
    then inexact, and the residual must be x - RN(level * divisor) with both roundings (a fused multiply-subtract
    shifts the third term's block scales); the quotients hardly ever sit on a tie, but the residuals' largest
    magnitudes sit right on an E4M3 boundary far more often than chance."""
    host, torch = ctx["host"], ctx["torch"]
    tokens, cols, terms = 192, 1024, 3
    rng = np.random.default_rng(int(glob * 1e6))
    x = (rng.standard_normal((tokens, cols)) * rng.choice([0.01, 1.0, 30.0], size=(tokens, 1))).astype(np.float32)
    x_bits = synth.f32_to_bf16_bits(x)
    weight = host.Nvfp4Sm100Weight(ctx["stream"], abi.LAYOUT_TCGEN05, 128, cols,
                                   torch.zeros(host.repack_extent(abi.LAYOUT_TCGEN05, 128, cols), dtype=torch.uint8,
                                               device=ctx["device"]), 1.0)
    lin = host.Nvfp4Sm100PrefillLinear.bind(ctx["plan"], weight, torch_bf16_from_bits(x_bits, ctx["device"]),
                                            terms=terms, activation_global_scale=glob)
    lin.submit_quant()
    ctx["stream"].synchronize()
    codes, scales = lin.staged_planes()
    want_codes, want_scales = oracle.act_quant(x_bits, tokens, cols, glob, terms)
    assert np.array_equal(scales, want_scales)
    assert np.array_equal(codes, want_codes)


def _run_gemm(ctx, w_planes, a_codes, a_scales, rows, cols, tokens, terms, g_w, g_a, plan=None):
    """Uploads explicit weight and (already quantised) activation planes and runs the GEMM entry."""
    host, torch = ctx["host"], ctx["torch"]
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols,
                                                           w_planes[0], w_planes[1], g_w)
    # staged activations hold whole 128-row tiles per term; rows past `tokens` are filled with NaN scales and
    # arbitrary codes here, to show that nothing of them reaches the stored rows
    padded = (tokens + 127) // 128 * 128
    code_planes, scale_regions = [], []
    for t in range(terms):
        codes = np.full((padded, cols // 2), 0xF7, dtype=np.uint8)
        scales = np.full((padded, cols // 16), 0x7E, dtype=np.uint8)
        codes[:tokens], scales[:tokens] = a_codes[t], a_scales[t]
        packed = host.repack_host(abi.LAYOUT_TCGEN05, padded, cols, codes, scales)
        packed = packed.copy()
        region = packed[padded * cols // 2:]
        if padded != tokens:   # poison the scale bytes of the padding rows with the E4M3 NaN pattern
            probe_scales = np.zeros((padded, cols // 16), dtype=np.uint8)
            probe_scales[tokens:] = 1
            marks = host.repack_host(abi.LAYOUT_TCGEN05, padded, cols, np.zeros_like(codes), probe_scales)[padded * cols // 2:]
            region[marks == 1] = 0x7F
        code_planes.append(packed[: padded * cols // 2])
        scale_regions.append(region)
    staged = torch.from_numpy(np.concatenate(code_planes + scale_regions)).to(ctx["device"])
    guard = torch.full(((tokens + 2) * rows,), float("nan"), dtype=torch.bfloat16, device=ctx["device"])
    out = guard[rows:(tokens + 1) * rows].view(tokens, rows)
    args = abi.header(abi.GemmArgs)
    args.weight, args.weight_len_bytes = weight.packed.data_ptr(), weight.packed.numel()
    args.activation, args.activation_len_bytes = staged.data_ptr(), staged.numel()
    args.output_bf16, args.output_len_bytes = out.data_ptr(), out.numel() * 2
    args.rows, args.cols, args.tokens, args.activation_terms = rows, cols, tokens, terms
    args.weight_global_scale, args.activation_global_scale = g_w, g_a
    s, plan, lib = ctx["stream"], plan or ctx["plan"], abi.lib()
    res = lib.augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(s.ordinal, s.handle, plan.handle, byref(args))
    assert res.status == 0, (res.status, res.raw_cuda_status)
    res = lib.augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args))
    assert res.status == 0, (res.status, res.raw_cuda_status)
    s.synchronize()
    status = plan.device_status()
    assert status == 0, hex(status)
    # nothing is written before the first or after the last token row
    assert bool(torch.isnan(guard[:rows]).all()) and bool(torch.isnan(guard[(tokens + 1) * rows:]).all())
    return bits_from_torch_bf16(out)


def _check_gemm(ctx, rows, cols, tokens, terms=1, seed=0, unit_scales=False, plan=None):
    w_codes, w_scales, g_w = synth.make_weight(seed, 70, "w", rows, cols)
    g_a = 2.0 ** -8
    x_bits = synth.make_activation(seed, 70, "x", tokens, cols)
    a_codes, a_scales = oracle.act_quant(x_bits, tokens, cols, g_a, terms)
    if unit_scales:
        w_scales = np.full_like(w_scales, 0x38)
        a_scales = np.full_like(a_scales, 0x38)
    got = _run_gemm(ctx, (w_codes, w_scales), a_codes, a_scales, rows, cols, tokens, terms, g_w, g_a, plan=plan)
    a64 = oracle.act_dequant_f64(a_codes, a_scales, g_a, tokens, cols, terms)
    y64 = oracle.linear_f64_xf64(w_codes, w_scales, g_w, rows, cols, a64, threads=oracle.max_threads())
    err = rel_error(got, y64)
    assert err <= TOLERANCE, err
    return err


# Ordered from the smallest exercise of the instruction to the full pipeline, so that a failure
# localises: one MMA -> distinct scales -> four MMAs per stage -> N = 256 -> several stages -> many tiles.
def test_gemm_single_mma_unit_scales(ctx):
    _check_gemm(ctx, rows=128, cols=64, tokens=128, unit_scales=True)


def test_gemm_single_mma_distinct_scales(ctx):
    _check_gemm(ctx, rows=128, cols=64, tokens=128)


def test_gemm_one_stage_four_mmas(ctx):
    _check_gemm(ctx, rows=128, cols=256, tokens=128, seed=1)


def test_gemm_n256_tile(ctx):
    _check_gemm(ctx, rows=256, cols=256, tokens=128, seed=2)


def test_gemm_ragged_k_and_n(ctx):
    _check_gemm(ctx, rows=384, cols=320, tokens=128, seed=3)       # k tail of 64, n tail of 128


def test_gemm_many_stages(ctx):
    _check_gemm(ctx, rows=256, cols=2176, tokens=128, seed=4)      # 8.5 stages: ring wrap + tail


def test_gemm_many_tiles_persistent(ctx):
    _check_gemm(ctx, rows=5120, cols=512, tokens=1024, seed=5)     # 160 tiles > SM count


def test_gemm_pair_tile_single(ctx):
    _check_gemm(ctx, rows=256, cols=256, tokens=256, seed=7)       # one 256 x 256 tile on one CTA pair, one stage


def test_gemm_pair_tile_ring_wrap(ctx):
    _check_gemm(ctx, rows=512, cols=2304, tokens=512, seed=8)      # 9 k blocks through the 5-stage ring, 4 tiles


def test_gemm_pair_tile_residual_terms(ctx):
    _check_gemm(ctx, rows=256, cols=1024, tokens=256, terms=3, seed=9)


def test_gemm_pair_tiles_more_than_pairs(ctx):
    _check_gemm(ctx, rows=2560, cols=256, tokens=2048, seed=10)    # 80 tiles over at most 74 pairs


@pytest.mark.parametrize("tokens", [1, 9, 100, 129, 300, 511])
def test_gemm_any_token_count(ctx, tokens):
    # the last 128-row tile is partly padding: computed, never stored
    _check_gemm(ctx, rows=512, cols=512, tokens=tokens, seed=11, terms=2 if tokens == 300 else 1)


def test_gemm_pair_tile_ragged_k_and_tokens(ctx):
    # 256 x 256 pair tile whose last k block is a quarter full and whose token rows end at 200 of 256
    _check_gemm(ctx, rows=256, cols=320, tokens=200, seed=12)
    _check_gemm(ctx, rows=512, cols=2176, tokens=256, seed=13, terms=2)    # the tp-8 k slice of the down projection


def test_gemm_pair_tiles_terms_share_weight_scales_across_tiles(ctx):
    # an odd number of k blocks (3), two activation terms and more tiles than CTA pairs: the weight-row scale
    # buffers alternate per k block across the tile boundary while two terms share each copy
    _check_gemm(ctx, rows=2560, cols=768, tokens=2048, terms=2, seed=14)


@pytest.mark.parametrize("cols,terms", [(4864, 1), (2560, 2), (320, 1)])
def test_gemm_pair_tiles_leftover_round_cut_along_k(ctx, cols, terms):
    # 80 pair tiles for at most 74 pairs: with a plan that has room for the handed-over accumulators the 6 tiles
    # of the last round are cut along k between the pairs (19 k blocks, 8 parts per tile; 10 k blocks with two
    # terms); with 2 k blocks the idle time saved is not worth a hand-over and the tiles stay whole
    host = ctx["host"]
    big = host.Plan(ctx["stream"], host.gemm_plan_scratch_bytes())
    try:
        _check_gemm(ctx, rows=2560, cols=cols, tokens=2048, terms=terms, seed=21, plan=big)
        # the flags are back at zero: a second launch on the same plan gives the same result
        _check_gemm(ctx, rows=2560, cols=cols, tokens=2048, terms=terms, seed=21, plan=big)
    finally:
        big.close()


def test_gemm_fewer_pair_tiles_than_pairs_all_cut_along_k(ctx):
    # 2 pair tiles of 20 k blocks: with room in the plan every tile is cut between the pairs of the whole device
    host = ctx["host"]
    big = host.Plan(ctx["stream"], host.gemm_plan_scratch_bytes())
    try:
        _check_gemm(ctx, rows=512, cols=5120, tokens=256, seed=22, plan=big)
        _check_gemm(ctx, rows=256, cols=17408, tokens=200, terms=2, seed=23, plan=big)   # one tile, 68 k blocks, ragged tokens
    finally:
        big.close()


def test_gemm_residual_terms(ctx):
    e1 = _check_gemm(ctx, rows=256, cols=1024, tokens=128, terms=1, seed=6)
    e3 = _check_gemm(ctx, rows=256, cols=1024, tokens=128, terms=3, seed=6)
    assert e1 <= TOLERANCE and e3 <= TOLERANCE


def test_prefill_linear_end_to_end_and_quantisation_error(ctx):
    # BF16 activations in, BF16 out; reports how far W4A4 with 1..3 residual terms is from the
    # BF16-activation oracle (the number the block-scaled MMA path trades for tensor throughput).
    host = ctx["host"]
    rows, cols, tokens = 512, 5120, 256
    w_codes, w_scales, g_w = synth.make_weight(0, 2, "gate", rows, cols)
    x_bits = synth.make_activation(0, 2, "x", tokens, cols)
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, rows, cols, w_codes, w_scales, g_w)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    y64 = oracle.linear_f64(w_codes, w_scales, g_w, rows, cols, x_bits, threads=oracle.max_threads())
    rms = np.sqrt(np.mean(y64 * y64))
    errors = {}
    for terms in (1, 2, 3):
        lin = host.Nvfp4Sm100PrefillLinear.bind(ctx["plan"], weight, x, terms=terms, activation_global_scale=2.0 ** -8)
        lin.submit_for_plan()
        ctx["stream"].synchronize()
        assert ctx["plan"].device_status() == 0
        got = synth.bf16_bits_to_f32(bits_from_torch_bf16(lin.out)).astype(np.float64).reshape(y64.shape)
        errors[terms] = float(np.sqrt(np.mean((got - y64) ** 2)) / rms)
        # kernel error in isolation: fp64 oracle fed the very activations the quantiser produced
        codes, scales = lin.staged_planes()
        a64 = oracle.act_dequant_f64(codes, scales, 2.0 ** -8, tokens, cols, terms)
        yq = oracle.linear_f64_xf64(w_codes, w_scales, g_w, rows, cols, a64, threads=oracle.max_threads())
        assert rel_error(bits_from_torch_bf16(lin.out), yq) <= TOLERANCE
    print("relative rms error vs BF16-activation oracle by residual terms:", errors)
    assert errors[1] < 0.2 and errors[2] < errors[1] / 3 and errors[3] < errors[2] / 3
    assert errors[3] <= TOLERANCE


@pytest.mark.parametrize("tokens", [1, 8, 9, 200])
def test_linear_dispatch_by_token_count(ctx, tokens):
    # tokens <= 8 take the small-token kernel, wider inputs the quantiser + GEMM; both within the bound
    host = ctx["host"]
    rows, cols = 256, 1024
    codes, scales, glob = synth.make_weight(3, 71, "w", rows, cols)
    linear = host.Nvfp4Sm100Linear(ctx["stream"], rows, cols, codes, scales, glob)
    x_bits = synth.make_activation(3, 71, "x", tokens, cols)
    binding = linear.bind(ctx["plan"], torch_bf16_from_bits(x_bits, ctx["device"]))
    assert isinstance(binding, host.Nvfp4Sm100Projection if tokens <= 8 else host.Nvfp4Sm100PrefillLinear)
    assert host.classify_tokens(tokens) == (host.SHAPE_SMALL_BATCH if tokens <= 8 else host.SHAPE_PREFILL)
    binding.submit_for_plan()
    ctx["stream"].synchronize()
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    assert rms_error(bits_from_torch_bf16(binding.out), y64) <= TOLERANCE


@pytest.mark.parametrize("hidden,inter,tokens", [(512, 1024, 256), (512, 1024, 100), (1024, 2176, 384)])
def test_prefill_mlp_program_with_fused_swiglu(ctx, hidden, inter, tokens):
    # quantise x -> gate|up GEMM with SiLU(gate)*up in the epilogue -> quantise h -> down GEMM, three residual terms
    host = ctx["host"]
    gate = synth.make_weight(4, 72, "gate", inter, hidden)
    up = synth.make_weight(4, 72, "up", inter, hidden)
    down = synth.make_weight(4, 72, "down", hidden, inter)
    up = (up[0], up[1], float(np.float32(up[2]) * np.float32(1.5)))     # distinct global scales for gate and up
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(23).standard_normal((tokens, hidden)).astype(np.float32) * 8.0)
    h64, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=oracle.max_threads())
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    program = host.Nvfp4Sm100PrefillFfnProgram.bind(
        ctx["plan"], gate_up_w, down_w, x, terms=3, keep_intermediate=True,
        input_global_scale=host.default_activation_global_scale(float(np.abs(synth.bf16_bits_to_f32(x_bits)).max())),
        intermediate_global_scale=host.default_activation_global_scale(float(np.abs(h64).max()) * 1.05))
    assert program.fused   # any token count: an odd last 128-row tile leaves one CTA of a pair without rows
    before = host.allocation_snapshot()
    for _ in range(2):
        program.submit_for_plan()
    ctx["stream"].synchronize()
    assert host.allocation_snapshot() == before and ctx["plan"].device_status() == 0
    # SiLU(gate)*up is heavy-tailed (largest values 20-30 x the rms), so each element is held to 2e-2 of
    # its own magnitude or of the rms, whichever is larger
    def worst(bits, want):
        got = synth.bf16_bits_to_f32(bits).astype(np.float64).reshape(want.shape)
        rms = np.sqrt(np.mean(want * want))
        return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), rms)))

    # the intermediate is the product of two GEMM outputs, each within the bound: (1 + e)^2
    assert worst(bits_from_torch_bf16(program.intermediate), h64) <= 2 * TOLERANCE
    assert worst(bits_from_torch_bf16(program.out), y64) <= TOLERANCE
    # the intermediate the down projection consumed is the one in memory: redo the down step from it in the oracle
    y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, bits_from_torch_bf16(program.intermediate),
                                   threads=oracle.max_threads())
    assert worst(bits_from_torch_bf16(program.out), y64_from_h) <= TOLERANCE


def test_fused_intermediate_quantiser_equals_the_quantiser_kernel(ctx):
    # gate|up GEMM that quantises its SiLU(gate)*up result in the epilogue against the same GEMM followed by act_quant:
    # identical staged bytes for every token row, identical final output; with and without the BF16 intermediate
    host, torch = ctx["host"], ctx["torch"]
    hidden, inter, tokens = 512, 1024, 500          # padded to 512: two pair tiles of token rows, the second ragged
    gate = synth.make_weight(5, 73, "gate", inter, hidden)
    up = synth.make_weight(5, 73, "up", inter, hidden)
    down = synth.make_weight(5, 73, "down", hidden, inter)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(29).standard_normal((tokens, hidden)).astype(np.float32) * 8.0)
    gate_up_w = host.upload_gate_up_interleaved(ctx["stream"], inter, hidden, *gate, *up)
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_TCGEN05, hidden, inter, *down)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    options = dict(terms=3, input_global_scale=0.02, intermediate_global_scale=0.004)
    plain = host.Nvfp4Sm100PrefillFfnProgram.bind(ctx["plan"], gate_up_w, down_w, x, fuse_quantiser=False, **options)
    fused = host.Nvfp4Sm100PrefillFfnProgram.bind(ctx["plan"], gate_up_w, down_w, x, keep_intermediate=True, **options)
    lean = host.Nvfp4Sm100PrefillFfnProgram.bind(ctx["plan"], gate_up_w, down_w, x, **options)
    assert not plain.fused and fused.fused and lean.fused
    lean.intermediate.fill_(float("nan"))
    for program in (plain, fused, lean):
        program.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0
    padded, terms = 512, 3
    code_bytes = padded * inter // 2

    def staged_rows(program):
        raw = program.staged_h.cpu().numpy()
        codes = raw[: terms * code_bytes].reshape(terms, padded, inter // 2)[:, :tokens]
        scales = []
        sf_bytes = host.repack_extent(abi.LAYOUT_TCGEN05, padded, inter) - code_bytes
        for term in range(terms):
            packed = np.concatenate([raw[term * code_bytes:(term + 1) * code_bytes],
                                     raw[terms * code_bytes + term * sf_bytes: terms * code_bytes + (term + 1) * sf_bytes]])
            scales.append(host.unpack_host(abi.LAYOUT_TCGEN05, padded, inter, packed)[1][:tokens])
        return codes, np.stack(scales)

    want_codes, want_scales = staged_rows(plain)
    for program in (fused, lean):
        got_codes, got_scales = staged_rows(program)
        assert np.array_equal(got_scales, want_scales) and np.array_equal(got_codes, want_codes)
        assert torch.equal(program.out.view(torch.int16), plain.out.view(torch.int16))
    assert torch.equal(fused.intermediate.view(torch.int16), plain.intermediate.view(torch.int16))
    assert bool(torch.isnan(lean.intermediate).all())     # never written when not asked for
