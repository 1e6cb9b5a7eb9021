"""GPU parity of the repack, dequantise and small-token (1..8) linear paths, through the C ABI."""
import ctypes
from ctypes import byref

import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, rel_error_f32, rms_error, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    plan = host.Plan(stream, 64 << 20)
    yield {"torch": torch, "host": host, "stream": stream, "plan": plan, "device": torch.device("cuda", 0)}
    plan.close()
    stream.close()


def _exhaustive_planes():
    """Every E2M1 code against every finite non-negative E4M3 scale: 127 rows x 128 columns."""
    rows, cols = 127, 128
    codes = np.zeros((rows, cols // 2), dtype=np.uint8)
    for b in range(cols // 2):
        codes[:, b] = ((2 * b) % 16) | (((2 * b + 1) % 16) << 4)
    scales = np.repeat(np.arange(127, dtype=np.uint8).reshape(rows, 1), cols // 16, axis=1)
    return rows, cols, codes, scales


def test_dequant_compact_bit_exact_exhaustive(ctx):
    torch, host = ctx["torch"], ctx["host"]
    rows, cols, codes, scales = _exhaustive_planes()
    for glob in (synth.GLOBAL_SCALE, 0.125, 2.0, 1.0):
        got = host.dequant_compact_f32(ctx["stream"], torch.from_numpy(codes).to(ctx["device"]),
                                       torch.from_numpy(scales).to(ctx["device"]), rows, cols, glob).cpu().numpy()
        want = oracle.dequant_planes_f32(codes, scales, glob, rows, cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # code 8 must decode to +0.0 (not -0.0) for every scale
    assert not np.any(got.view(np.uint32)[:, 8::16] & 0x80000000)


@pytest.mark.parametrize("layout,rows,cols", [
    (abi.LAYOUT_STREAM, 96, 384), (abi.LAYOUT_STREAM_PAIR, 48, 256), (abi.LAYOUT_TCGEN05, 384, 320)])
def test_device_repack_matches_host_and_decodes_bit_exact(ctx, layout, rows, cols):
    host = ctx["host"]
    pair = layout == abi.LAYOUT_STREAM_PAIR
    ca, sa, ga = synth.make_weight(1, 50, "a", rows, cols)
    cb, sb, gb = synth.make_weight(1, 50, "b", rows, cols) if pair else (None, None, 0.0)
    gb = 0.37 if pair else 0.0
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], layout, rows, cols, ca, sa, ga, cb, sb, gb)
    assert np.array_equal(w.packed.cpu().numpy(), host.repack_host(layout, rows, cols, ca, sa, cb, sb))
    got = w.dequant_f32().cpu().numpy()
    want_a = oracle.dequant_planes_f32(ca, sa, ga, rows, cols)
    if pair:
        want_b = oracle.dequant_planes_f32(cb, sb, gb, rows, cols)
        assert np.array_equal(got[0].view(np.uint32), want_a.view(np.uint32))
        assert np.array_equal(got[1].view(np.uint32), want_b.view(np.uint32))
    else:
        assert np.array_equal(got.view(np.uint32), want_a.view(np.uint32))


def test_dequant_full_config0_tensor_bit_exact(ctx):
    # the whole 17408 x 5120 seeded tensor, compared as u32 words
    torch, host = ctx["torch"], ctx["host"]
    rows, cols = 17408, 5120
    codes, scales, glob = synth.make_weight(0, 0, "weight", rows, cols)
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
    got = w.dequant_f32()
    want = torch.from_numpy(oracle.dequant_planes_numpy(codes, scales, glob, rows, cols)).to(ctx["device"])
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def _linear_case(ctx, rows, cols, tokens, seed, epilogue=abi.EPILOGUE_LINEAR_BF16, x_bits=None):
    host = ctx["host"]
    codes, scales, glob = synth.make_weight(seed, 60, "w", rows, cols)
    if x_bits is None:
        x_bits = synth.make_activation(seed, 60, "x", tokens, cols)
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    proj = host.Nvfp4Sm100Projection.bind(ctx["plan"], w, x, epilogue=epilogue)
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0
    return codes, scales, glob, x_bits, proj


@pytest.mark.parametrize("rows,cols,tokens", [
    (32, 128, 1), (32, 128, 8), (64, 256, 3), (96, 640, 8), (128, 2176, 8), (160, 5248, 5), (2048, 1024, 8),
    (320, 17408, 8), (544, 5120, 1)])
def test_linear_matches_fp64_oracle(ctx, rows, cols, tokens):
    codes, scales, glob, x_bits, proj = _linear_case(ctx, rows, cols, tokens, seed=rows + cols + tokens)
    got = bits_from_torch_bf16(proj.out)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=4)
    assert rel_error(got, y64) <= TOLERANCE
    ref_bits = oracle.linear_bf16(codes, scales, glob, rows, cols, x_bits, threads=4)
    # against bf16_round(sequential f32): at most one BF16 ulp apart anywhere
    a = synth.bf16_bits_to_f32(got).astype(np.float64)
    b = synth.bf16_bits_to_f32(ref_bits).astype(np.float64)
    assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3 * np.sqrt(np.mean(b * b)))) <= 2.0 ** -7


@pytest.mark.parametrize("rows,cols", [(10240, 5120), (5120, 5120), (5120, 10240)])
def test_whole_model_sweep_projection_shapes(ctx, rows, cols):
    # the stand-ins for the attention / GDN in- and out-projections of the M = 8 whole-model sweep, full size
    codes, scales, glob, x_bits, proj = _linear_case(ctx, rows, cols, 8, seed=rows // 512 + cols // 1024)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    assert rel_error(bits_from_torch_bf16(proj.out), y64) <= TOLERANCE


@pytest.mark.parametrize("rows,cols,tokens", [(12288, 5120, 8), (1024, 5120, 8), (6144, 5120, 1), (5120, 6144, 8), (48 + 16, 5120, 8)])
def test_attention_and_gdn_projection_shapes(ctx, rows, cols, tokens):
    # the real model's attention / GDN projections (crates/augur-model-qwen35/src/checkpoint_profile.rs:29-104):
    # 12288 / 1024 / 6144 x 5120 inputs, 5120 x 6144 output; the 48-row gates are padded to the 32-row group (64)
    codes, scales, glob, x_bits, proj = _linear_case(ctx, rows, cols, tokens, seed=rows // 64 + cols // 128 + tokens)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    assert rel_error(bits_from_torch_bf16(proj.out), y64) <= TOLERANCE


def test_one_hot_activations_read_back_the_weights_exactly(ctx):
    # x = e_k makes y[n] = bf16(w[n][k]): checks every fragment position of the layout
    rows, cols, tokens = 64, 256, 8
    x = np.zeros((tokens, cols), dtype=np.float32)
    ks = [0, 1, 9, 17, 100, 127, 128, 255]
    for t, k in enumerate(ks):
        x[t, k] = 1.0
    codes, scales, glob, x_bits, proj = _linear_case(ctx, rows, cols, tokens, seed=7, x_bits=synth.f32_to_bf16_bits(x))
    w = oracle.dequant_planes_f32(codes, scales, 1.0, rows, cols)      # e2m1 * e4m3, exact in f32
    got = synth.bf16_bits_to_f32(bits_from_torch_bf16(proj.out)).reshape(tokens, rows)
    for t, k in enumerate(ks):
        want = synth.bf16_bits_to_f32(synth.f32_to_bf16_bits((w[:, k] * np.float32(glob)).astype(np.float32)))
        assert np.array_equal(got[t], want), (t, k)


def test_extreme_activation_ranges_stay_within_tolerance(ctx):
    # per-token power-of-two normalisation: tiny, huge and mixed-magnitude rows
    rows, cols, tokens = 96, 640, 8
    rng = np.random.default_rng(3)
    x = rng.standard_normal((tokens, cols)).astype(np.float32)
    x[0] *= 1e-20
    x[1] *= 1e20
    x[2, 5] = 3e4
    x[3] *= 2.0 ** -60
    x[4] = 0.0
    x[5, ::7] *= 1e6
    codes, scales, glob, x_bits, proj = _linear_case(ctx, rows, cols, tokens, seed=11, x_bits=synth.f32_to_bf16_bits(x))
    got = bits_from_torch_bf16(proj.out).reshape(tokens, rows)
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=2)
    for t in range(tokens):
        assert rel_error(got[t], y64[t]) <= TOLERANCE, t
    assert np.all(got[4] & 0x7FFF == 0)


def test_f32_epilogue_returns_unrounded_sums(ctx):
    rows, cols, tokens = 128, 2176, 8
    codes, scales, glob, x_bits, proj = _linear_case(ctx, rows, cols, tokens, seed=5, epilogue=abi.EPILOGUE_LINEAR_F32)
    got = proj.out.cpu().numpy()
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=2)
    assert rel_error_f32(got, y64) <= 1e-3


def test_config0_full_size_linear(ctx):
    # configuration 0 of the benchmark definition: M=8, K=5120, N=17408, seed 0
    rows, cols, tokens = 17408, 5120, 8
    host = ctx["host"]
    codes, scales, glob = synth.make_weight(0, 0, "weight", rows, cols)
    x_bits = synth.make_activation(0, 0, "activation", tokens, cols)
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    proj = host.Nvfp4Sm100Projection.bind(ctx["plan"], w, x)
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    first = bits_from_torch_bf16(proj.out).copy()
    y64 = oracle.linear_f64(codes, scales, glob, rows, cols, x_bits, threads=oracle.max_threads())
    assert rel_error(first, y64) <= TOLERANCE
    # deterministic: a second submit gives the same bits (fixed-order combination, clean counters)
    proj.out.zero_()
    proj.submit_for_plan()
    ctx["stream"].synchronize()
    assert np.array_equal(bits_from_torch_bf16(proj.out), first)
    # M=1 on the same weight equals row 0 of the M=8 result up to accumulation order
    proj1 = host.Nvfp4Sm100Projection.bind(ctx["plan"], w, x[:1].contiguous())
    proj1.submit_for_plan()
    ctx["stream"].synchronize()
    assert rel_error(bits_from_torch_bf16(proj1.out), y64[:1]) <= TOLERANCE


def _mlp_weights(ctx, hidden, inter, seed):
    host = ctx["host"]
    gate = synth.make_weight(seed, 61, "gate", inter, hidden)
    up = synth.make_weight(seed, 61, "up", inter, hidden)
    down = synth.make_weight(seed, 61, "down", hidden, inter)
    gate_up = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(
        ctx["stream"], abi.LAYOUT_STREAM_PAIR, inter, hidden, gate[0], gate[1], gate[2], up[0], up[1], up[2])
    down_w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(
        ctx["stream"], abi.LAYOUT_STREAM, hidden, inter, down[0], down[1], down[2])
    return gate, up, down, gate_up, down_w


@pytest.mark.parametrize("hidden,inter,tokens", [(128, 256, 8), (256, 2176, 8), (640, 1152, 1), (5120, 2176, 8)])
def test_mlp_program_matches_oracle(ctx, hidden, inter, tokens):
    host = ctx["host"]
    gate, up, down, gate_up, down_w = _mlp_weights(ctx, hidden, inter, seed=hidden + inter)
    # scale activations up so that SiLU is exercised away from zero (weights carry a 1/448 factor)
    x_f = np.random.default_rng(17).standard_normal((tokens, hidden)).astype(np.float32) * 8.0
    x_bits = synth.f32_to_bf16_bits(x_f)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    program = host.Nvfp4Sm100FfnProgram.bind(ctx["plan"], gate_up, down_w, x)
    program.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0
    h64, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=4)
    assert rel_error(bits_from_torch_bf16(program.intermediate), h64) <= TOLERANCE
    # the down projection consumes the BF16-rounded intermediate the kernel actually wrote
    y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter,
                                   bits_from_torch_bf16(program.intermediate), threads=4)
    assert rel_error(bits_from_torch_bf16(program.out), y64_from_h) <= TOLERANCE
    # end to end against the oracle chain, whose intermediate is rounded independently: the largest
    # of 40960 rounding-noise samples sits near 2e-2 of the rms for the short K = 2176 case
    assert rms_error(bits_from_torch_bf16(program.out), y64) <= 2 * TOLERANCE
    h_ref, y_ref = oracle.mlp_bf16(gate, up, down, hidden, inter, x_bits, threads=4)
    assert rms_error(bits_from_torch_bf16(program.out), synth.bf16_bits_to_f32(y_ref).astype(np.float64)) <= 2 * TOLERANCE


def test_hot_path_allocates_nothing_and_counts_launches(ctx):
    # crates/augur-backend/src/cuda_qwen35_qpn.rs:690-707: allocation snapshots around the hot loop
    host, torch = ctx["host"], ctx["torch"]
    gate, up, down, gate_up, down_w = _mlp_weights(ctx, 256, 512, seed=3)
    x = torch_bf16_from_bits(synth.make_activation(3, 61, "x", 8, 256), ctx["device"])
    program = host.Nvfp4Sm100FfnProgram.bind(ctx["plan"], gate_up, down_w, x)
    program.submit_for_plan()
    ctx["stream"].synchronize()
    before_alloc, before_launch = host.allocation_snapshot(), host.launch_count()
    torch_before = torch.cuda.memory_stats()["allocation.all.allocated"]
    for _ in range(16):
        program.submit_for_plan()
    ctx["stream"].synchronize()
    assert host.allocation_snapshot() == before_alloc
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == torch_before
    assert host.launch_count() - before_launch == 32     # per program: gate|up + down


def test_cuda_graph_capture_and_replay_with_refreshed_inputs(ctx):
    # crates/augur-backend/src/cuda_qwen35_qpn.rs:621-652
    host, torch = ctx["host"], ctx["torch"]
    hidden, inter, tokens = 256, 512, 8
    gate, up, down, gate_up, down_w = _mlp_weights(ctx, hidden, inter, seed=9)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        stream = host.Stream(0, side)
        plan = host.Plan(stream, host.mlp_scratch_bytes(hidden, inter))
        x = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=ctx["device"])
        program = host.Nvfp4Sm100FfnProgram.bind(plan, gate_up, down_w, x)
        program.submit_for_plan()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            program.submit_for_plan()
        for seed in (1, 2):
            x_bits = synth.f32_to_bf16_bits(np.random.default_rng(seed).standard_normal((tokens, hidden)).astype(np.float32) * 8)
            x.copy_(torch_bf16_from_bits(x_bits, ctx["device"]))
            graph.replay()
            side.synchronize()
            _, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=2)
            assert rms_error(bits_from_torch_bf16(program.out), y64) <= TOLERANCE
        plan.close()


def _gemv_valid(ctx, rows=64, cols=256, tokens=8):
    host, torch = ctx["host"], ctx["torch"]
    codes, scales, glob = synth.make_weight(2, 62, "w", rows, cols)
    w = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
    x = torch_bf16_from_bits(synth.make_activation(2, 62, "x", tokens, cols), ctx["device"])
    # guard bands around the output prove rejected calls never write (cuda_qwen35_qpn.rs:435-482)
    guarded = torch.full((tokens * rows + 256,), 0x5A5A, dtype=torch.int16, device=ctx["device"])
    out = guarded[128:128 + tokens * rows].view(torch.bfloat16).view(tokens, rows)
    return w, x, guarded, out


GEMV_MUTATIONS = [
    ("abi", lambda a: setattr(a, "abi_version", 0), abi.STATUS_ABI_VERSION_MISMATCH),
    ("struct_size", lambda a: setattr(a, "struct_size", a.struct_size + 8), abi.STATUS_INVALID_ARGUMENT),
    ("stored rows without the matching output extent", lambda a: setattr(a, "stored_rows", 1), abi.STATUS_INVALID_ARGUMENT),
    ("stored rows beyond the weight", lambda a: setattr(a, "stored_rows", a.rows + 32), abi.STATUS_INVALID_ARGUMENT),
    ("reserved1", lambda a: setattr(a, "reserved1", 7), abi.STATUS_INVALID_ARGUMENT),
    ("weight len-1", lambda a: setattr(a, "weight_len_bytes", a.weight_len_bytes - 1), abi.STATUS_INVALID_ARGUMENT),
    ("weight len+2304", lambda a: setattr(a, "weight_len_bytes", a.weight_len_bytes + 2304), abi.STATUS_INVALID_ARGUMENT),
    ("input len", lambda a: setattr(a, "input_len_bytes", a.input_len_bytes - 2), abi.STATUS_INVALID_ARGUMENT),
    ("output len", lambda a: setattr(a, "output_len_bytes", a.output_len_bytes + 2), abi.STATUS_INVALID_ARGUMENT),
    ("weight misaligned", lambda a: setattr(a, "weight", a.weight + 16), abi.STATUS_INVALID_ARGUMENT),
    ("input misaligned", lambda a: setattr(a, "input_bf16", a.input_bf16 + 2), abi.STATUS_INVALID_ARGUMENT),
    ("output misaligned", lambda a: setattr(a, "output", a.output + 2), abi.STATUS_INVALID_ARGUMENT),
    ("alias out=in", lambda a: setattr(a, "output", a.input_bf16), abi.STATUS_INVALID_ARGUMENT),
    ("alias in inside weight", lambda a: setattr(a, "input_bf16", a.weight + 256), abi.STATUS_INVALID_ARGUMENT),
    ("tokens 0", lambda a: setattr(a, "tokens", 0), abi.STATUS_INVALID_ARGUMENT),
    ("tokens 9", lambda a: setattr(a, "tokens", 9), abi.STATUS_INVALID_ARGUMENT),
    ("rows 48", lambda a: setattr(a, "rows", 48), abi.STATUS_INVALID_ARGUMENT),
    ("cols 192", lambda a: setattr(a, "cols", 192), abi.STATUS_INVALID_ARGUMENT),
    ("epilogue 3", lambda a: setattr(a, "epilogue", 3), abi.STATUS_INVALID_ARGUMENT),
    ("epilogue swiglu on single", lambda a: setattr(a, "epilogue", abi.EPILOGUE_SWIGLU_BF16), abi.STATUS_INVALID_ARGUMENT),
    ("scale NaN", lambda a: setattr(a, "global_scale", float("nan")), abi.STATUS_INVALID_ARGUMENT),
    ("scale 0", lambda a: setattr(a, "global_scale", 0.0), abi.STATUS_INVALID_ARGUMENT),
    ("scale 25", lambda a: setattr(a, "global_scale", 25.0), abi.STATUS_INVALID_ARGUMENT),
    ("stray scale_b", lambda a: setattr(a, "global_scale_b", 1.0), abi.STATUS_INVALID_ARGUMENT),
    ("null weight", lambda a: setattr(a, "weight", 0), abi.STATUS_INVALID_ARGUMENT),
]


def test_descriptor_mutation_fuzz_rejects_and_never_writes(ctx):
    # crates/augur-backend/src/cuda_nvfp4_sm70.rs:579-610
    host, torch = ctx["host"], ctx["torch"]
    lib, s, plan = abi.lib(), ctx["stream"], ctx["plan"]
    w, x, guarded, out = _gemv_valid(ctx)
    good = host.gemv_args(w, x, out, abi.EPILOGUE_LINEAR_BF16)
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(s.ordinal, s.handle, plan.handle, byref(good)).status == 0
    launches = host.launch_count()
    for name, mutate, expected in GEMV_MUTATIONS:
        args = host.gemv_args(w, x, out, abi.EPILOGUE_LINEAR_BF16)
        mutate(args)
        for fn in (lib.augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1, lib.augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1):
            assert fn(s.ordinal, s.handle, plan.handle, byref(args)).status == expected, name
    # a stream that does not own the plan, and an output that aliases the plan scratch
    other = host.Stream(0, torch.cuda.Stream())
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(other.ordinal, other.handle, plan.handle, byref(good)).status == abi.STATUS_INVALID_ARGUMENT
    snap = plan.snapshot()
    args = host.gemv_args(w, x, out, abi.EPILOGUE_LINEAR_BF16)
    args.output = snap.scratch
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(s.ordinal, s.handle, plan.handle, byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    # preflight asks the driver who owns each range: pinned host memory is not device memory
    pinned = torch.empty(x.numel() * 2, dtype=torch.uint8).pin_memory()
    args = host.gemv_args(w, x, out, abi.EPILOGUE_LINEAR_BF16)
    args.input_bf16 = pinned.data_ptr()
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(s.ordinal, s.handle, plan.handle, byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    s.synchronize()
    assert host.launch_count() == launches
    assert bool((guarded == 0x5A5A).all())
    # the valid descriptor writes the output and only the output
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(good)).status == 0
    s.synchronize()
    assert bool((guarded[:128] == 0x5A5A).all()) and bool((guarded[-128:] == 0x5A5A).all())
    assert not bool((guarded[128:-128] == 0x5A5A).all())


def test_host_side_fault_injection(ctx):
    host = ctx["host"]
    lib, s, plan = abi.lib(), ctx["stream"], ctx["plan"]
    w, x, guarded, out = _gemv_valid(ctx)
    args = host.gemv_args(w, x, out, abi.EPILOGUE_LINEAR_BF16)
    launches = host.launch_count()
    lib.augur_cuda_nvfp4_sm100_diagnostic_inject_submit_fault_v1(2)
    for _ in range(2):
        res = lib.augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args))
        assert res.status == abi.STATUS_DIAGNOSTIC_FAULT_INJECTED
    s.synchronize()
    assert host.launch_count() == launches and bool((guarded == 0x5A5A).all())
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args)).status == 0
    s.synchronize()


def test_mlp_program_cross_validation(ctx):
    # all members and cross aliases are checked before the first enqueue (augur_qwen35_qpn_prefill.cuh:97-115)
    host, torch = ctx["host"], ctx["torch"]
    lib, s, plan = abi.lib(), ctx["stream"], ctx["plan"]
    gate, up, down, gate_up, down_w = _mlp_weights(ctx, 256, 512, seed=4)
    x = torch_bf16_from_bits(synth.make_activation(4, 61, "x", 8, 256), ctx["device"])
    program = host.Nvfp4Sm100FfnProgram.bind(plan, gate_up, down_w, x)
    launches = host.launch_count()

    def rejected(mutate):
        args = abi.MlpArgs.from_buffer_copy(program.args)
        mutate(args)
        a = lib.augur_cuda_nvfp4_sm100_mlp_preflight_v1(s.ordinal, s.handle, plan.handle, byref(args)).status
        b = lib.augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args)).status
        return a != 0 and b != 0

    other = torch.empty_like(program.intermediate)
    assert rejected(lambda a: setattr(a.down, "input_bf16", other.data_ptr()))          # down does not read what gate_up wrote
    assert rejected(lambda a: setattr(a.down, "output", a.gate_up.input_bf16))           # output aliases the program input
    assert rejected(lambda a: setattr(a.down, "tokens", 4))
    assert rejected(lambda a: setattr(a.gate_up, "epilogue", abi.EPILOGUE_LINEAR_BF16))
    assert rejected(lambda a: setattr(a.down, "epilogue", abi.EPILOGUE_SWIGLU_BF16))
    assert rejected(lambda a: setattr(a.down, "weight", a.gate_up.weight))
    s.synchronize()
    assert host.launch_count() == launches


@pytest.mark.parametrize("counted_on", ["host", "device"])
def test_exchange_reduce_with_eight_sources_on_one_gpu(ctx, counted_on):
    # The tensor-parallel down launch for rank 0 of 8, on one GPU: the tiles of ranks 1..7 are written into rank 0's
    # exchange buffer from the host beforehand (so nothing waits), the launch pushes its own tiles into eight
    # buffers, and its reduce step must deliver bf16(own + the seven others, in rank order) for every row group.
    host, torch = ctx["host"], ctx["torch"]
    # sequence 3 passed by the host, or the first launch of a fresh buffer counting for itself (sequence 1)
    hidden, inter, tokens, world, seq = 256, 512, 8, 8, (3 if counted_on == "host" else 1)
    gate, up, down, gate_up, down_w = _mlp_weights(ctx, hidden, inter, seed=21)
    x_bits = synth.f32_to_bf16_bits(np.random.default_rng(21).standard_normal((tokens, hidden)).astype(np.float32) * 8.0)
    x = torch_bf16_from_bits(x_bits, ctx["device"])
    program = host.Nvfp4Sm100FfnProgram.bind(ctx["plan"], gate_up, down_w, x)
    groups = hidden // 32
    extent = ctypes.c_uint64()
    assert abi.lib().augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(hidden, world, byref(extent)).status == 0
    others = np.random.default_rng(22).standard_normal((world, tokens, hidden)).astype(np.float32)
    # [parity][source][group][lane][4 lines of {value, seq, value, seq}]
    image = np.zeros((2, world, groups, 32, 4, 4), dtype=np.uint32)
    lane = np.arange(32)
    g, t4 = lane >> 2, lane & 3
    for source in range(1, world):
        for group in range(groups):
            for i in range(8):
                token = 2 * t4 + (i & 1)
                row = group * 32 + (i >> 2) * 16 + g + ((i >> 1) & 1) * 8
                image[seq & 1, source, group, lane, i // 2, (i & 1) * 2] = others[source, token, row].view(np.uint32)
                image[seq & 1, source, group, lane, i // 2, (i & 1) * 2 + 1] = seq
    assert image.nbytes + 256 == extent.value     # the tiles, then the sequence counter
    buffers = [torch.zeros(extent.value, dtype=torch.uint8, device=ctx["device"]) for _ in range(world)]
    buffers[0][:image.nbytes].copy_(torch.from_numpy(image.view(np.uint8).reshape(-1)))
    args = abi.header(abi.MlpTpArgs)
    args.gate_up, args.down = program.args.gate_up, program.args.down
    for r in range(world):
        args.exchange[r] = buffers[r].data_ptr()
    args.exchange_len_bytes, args.world, args.rank = extent.value, world, 0
    args.sequence = seq if counted_on == "host" else 0
    s, plan, lib = ctx["stream"], ctx["plan"], abi.lib()
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_preflight_v1(s.ordinal, s.handle, plan.handle, byref(args)).status == 0
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args)).status == 0
    s.synchronize()
    assert plan.device_status() == 0
    h_bits = bits_from_torch_bf16(program.intermediate)
    own = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=4)
    want = own + others[1:].astype(np.float64).sum(axis=0)
    # the others' tiles are f32 values, so the fp64 sum of all eight is what one BF16 rounding of the f32 sum must match
    assert rel_error(bits_from_torch_bf16(program.out), want) <= TOLERANCE
    # the counter in the tail of rank 0's buffer: one launch counted and no arrivals left, or untouched
    tail = buffers[0][image.nbytes:].cpu().numpy().view(np.uint32)
    assert list(tail[:2]) == ([1, 0] if counted_on == "device" else [0, 0])
    # its own tiles arrived in every buffer, flagged with the sequence number
    for r in range(1, world):
        pushed = buffers[r][:image.nbytes].cpu().numpy().view(np.uint32).reshape(2, world, groups, 32, 4, 4)
        assert np.all(pushed[seq & 1, 0, :, :, :, 1] == seq) and np.all(pushed[seq & 1, 0, :, :, :, 3] == seq)
        assert not pushed[1 - (seq & 1)].any() and not pushed[seq & 1, 1:].any()


def test_exchange_wait_that_runs_out_is_reported_and_leaves_the_context_usable(ctx):
    # Failure detection without a fault: rank 0 of 2 runs alone, the tiles of rank 1 never arrive, every wait of
    # the reduce step runs out (bounded polls), the launch ends by itself, the plan's status word says which wait
    # gave up, and the same stream goes on working.
    host, torch = ctx["host"], ctx["torch"]
    hidden, inter, tokens, world = 128, 256, 8, 2
    gate, up, down, gate_up, down_w = _mlp_weights(ctx, hidden, inter, seed=23)
    x = torch_bf16_from_bits(synth.make_activation(23, 63, "x", tokens, hidden), ctx["device"])
    plan = host.Plan(ctx["stream"], host.mlp_scratch_bytes(hidden, inter))
    program = host.Nvfp4Sm100FfnProgram.bind(plan, gate_up, down_w, x)
    extent = ctypes.c_uint64()
    assert abi.lib().augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(hidden, world, byref(extent)).status == 0
    buffers = [torch.zeros(extent.value, dtype=torch.uint8, device=ctx["device"]) for _ in range(world)]
    args = abi.header(abi.MlpTpArgs)
    args.gate_up, args.down = program.args.gate_up, program.args.down
    for r in range(world):
        args.exchange[r] = buffers[r].data_ptr()
    args.exchange_len_bytes, args.world, args.rank, args.sequence = extent.value, world, 0, 1
    s, lib = ctx["stream"], abi.lib()
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args)).status == 0
    s.synchronize()                              # returns: the waits are bounded
    assert plan.device_status() == 0x203
    plan.close()
    # the context is intact: an ordinary program on the same stream still matches the oracle
    codes, scales, glob, x_bits, proj = _linear_case(ctx, 64, 256, 4, seed=24)
    y64 = oracle.linear_f64(codes, scales, glob, 64, 256, x_bits, threads=2)
    assert rel_error(bits_from_torch_bf16(proj.out), y64) <= TOLERANCE


@pytest.mark.parametrize("residual", [False, True], ids=["gdn-input", "post-attention"])
def test_norm_group_program(ctx, residual):
    # [residual add] -> RMSNorm -> BF16 stage -> projections, one program (the reference's GDN-input and post-attention groups)
    host, torch = ctx["host"], ctx["torch"]
    tokens, cols, eps = 8, 5120, 1e-6
    # GDN input group: qkv, z and the two 48-row gates (padded to 64 weight rows, stored trimmed); post-attention: two projections
    shapes = [(10240, cols), (6144, cols), (64, cols), (64, cols)] if not residual else [(1024, cols), (2048, cols)]
    stored = [0, 0, 48, 48] if not residual else [0, 0]
    rng = np.random.default_rng(31)
    a = rng.standard_normal((tokens, cols)).astype(np.float32) * 3
    b = rng.standard_normal((tokens, cols)).astype(np.float32)
    norm_weight = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    planes = [synth.make_weight(7, 64, f"w{i}", rows, cols) for i, (rows, _) in enumerate(shapes)]
    weights = [host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, *planes[i])
               for i, (rows, _) in enumerate(shapes)]
    device = ctx["device"]
    if residual:
        x_dev = torch.zeros((tokens, cols), dtype=torch.float32, device=device)
        program = host.Nvfp4Sm100NormGroupProgram.bind(ctx["plan"], weights, x_dev, torch.from_numpy(norm_weight).to(device), eps,
                                                       torch.from_numpy(a).to(device), torch.from_numpy(b).to(device), stored_rows=stored)
        want_x, want_y, want_staged = oracle.rmsnorm_stage(None, norm_weight, eps, a, b)
    else:
        x_dev = torch.from_numpy(a).to(device)
        program = host.Nvfp4Sm100NormGroupProgram.bind(ctx["plan"], weights, x_dev, torch.from_numpy(norm_weight).to(device), eps,
                                                       stored_rows=stored)
        want_x, want_y, want_staged = oracle.rmsnorm_stage(a, norm_weight, eps)
    before = host.allocation_snapshot(), host.launch_count()
    program.submit_for_plan()
    ctx["stream"].synchronize()
    assert host.allocation_snapshot() == before[0] and host.launch_count() - before[1] == 2    # norm stage + one grid for all members
    assert ctx["plan"].device_status() == 0
    # the norm stage is bit-exact with the CPU statement of the reference kernel's order
    assert np.array_equal(x_dev.cpu().numpy().view(np.uint32), want_x.view(np.uint32))
    assert np.array_equal(program.normalised.cpu().numpy().view(np.uint32), want_y.view(np.uint32))
    assert np.array_equal(bits_from_torch_bf16(program.staged).reshape(want_staged.shape), want_staged)
    for (rows, _), keep, (codes, scales, glob), out in zip(shapes, stored, planes, program.outputs):
        y64 = oracle.linear_f64(codes, scales, glob, rows, cols, want_staged, threads=oracle.max_threads())
        if keep:    # the trimmed store: [tokens][48], the padding rows are computed and never written
            assert tuple(out.shape) == (tokens, keep)
            y64 = np.ascontiguousarray(y64[:, :keep])
        assert rel_error(bits_from_torch_bf16(out), y64) <= TOLERANCE
    # a second submit finds counters and staged fragments in order
    program.submit_for_plan()
    ctx["stream"].synchronize()
    assert ctx["plan"].device_status() == 0
    for (rows, _), keep, (codes, scales, glob), out in zip(shapes, stored, planes, program.outputs):
        y64 = oracle.linear_f64(codes, scales, glob, rows, cols, want_staged, threads=oracle.max_threads())
        assert rel_error(bits_from_torch_bf16(out), np.ascontiguousarray(y64[:, :keep]) if keep else y64) <= TOLERANCE


@pytest.mark.parametrize("cols", [256, 6144, 6400])
def test_norm_stage_row_widths(ctx, cols):
    # rows up to 6144 columns are held in registers by the norm stage, wider ones take the looping path: the same bits
    host, torch = ctx["host"], ctx["torch"]
    tokens, eps, rows = 5, 1e-5, 64
    rng = np.random.default_rng(cols)
    a = rng.standard_normal((tokens, cols)).astype(np.float32) * 2
    b = rng.standard_normal((tokens, cols)).astype(np.float32)
    norm_weight = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    codes, scales, glob = synth.make_weight(9, 65, "w", rows, cols)
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
    device = ctx["device"]
    for residual in (False, True):
        x_dev = torch.zeros((tokens, cols), dtype=torch.float32, device=device) if residual else torch.from_numpy(a).to(device)
        extra = (torch.from_numpy(a).to(device), torch.from_numpy(b).to(device)) if residual else ()
        program = host.Nvfp4Sm100NormGroupProgram.bind(ctx["plan"], [weight], x_dev, torch.from_numpy(norm_weight).to(device), eps, *extra)
        program.submit_for_plan()
        ctx["stream"].synchronize()
        assert ctx["plan"].device_status() == 0
        want_x, want_y, want_staged = oracle.rmsnorm_stage(None, norm_weight, eps, a, b) if residual else oracle.rmsnorm_stage(a, norm_weight, eps)
        assert np.array_equal(x_dev.cpu().numpy().view(np.uint32), want_x.view(np.uint32))
        assert np.array_equal(program.normalised.cpu().numpy().view(np.uint32), want_y.view(np.uint32))
        assert np.array_equal(bits_from_torch_bf16(program.staged).reshape(want_staged.shape), want_staged)
        y64 = oracle.linear_f64(codes, scales, glob, rows, cols, want_staged, threads=oracle.max_threads())
        assert rel_error(bits_from_torch_bf16(program.outputs[0]), y64) <= TOLERANCE


def test_norm_group_rejects_inconsistent_members(ctx):
    host, torch = ctx["host"], ctx["torch"]
    tokens, cols = 4, 512
    codes, scales, glob = synth.make_weight(8, 65, "w", 64, cols)
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, 64, cols, codes, scales, glob)
    x = torch.zeros((tokens, cols), dtype=torch.float32, device=ctx["device"])
    w = torch.ones(cols, dtype=torch.float32, device=ctx["device"])
    program = host.Nvfp4Sm100NormGroupProgram.bind(ctx["plan"], [weight], x, w)
    s, plan, lib = ctx["stream"], ctx["plan"], abi.lib()

    def status(mutate):
        args = abi.NormGroupArgs.from_buffer_copy(program.args)
        mutate(args)
        launches = host.launch_count()
        result = lib.augur_cuda_nvfp4_sm100_norm_group_prevalidated_submit_v1(s.ordinal, s.handle, plan.handle, byref(args))
        assert host.launch_count() == launches      # nothing was enqueued
        return result.status

    program.submit_for_plan()                       # the unmodified descriptor is accepted
    s.synchronize()
    for mutate in (lambda a: setattr(a, "count", 0), lambda a: setattr(a, "count", 5), lambda a: setattr(a, "residual", 2),
                   lambda a: setattr(a, "cols", cols + 128), lambda a: setattr(a, "tokens", 9), lambda a: setattr(a, "epsilon", -1.0),
                   lambda a: setattr(a, "add_a", a.input_f32), lambda a: setattr(a, "staged_bf16", a.output_f32),
                   lambda a: setattr(a.projections[0], "input_bf16", a.output_f32),
                   lambda a: setattr(a.projections[0], "tokens", 3),
                   lambda a: setattr(a.projections[1], "rows", 32),
                   lambda a: setattr(a.projections[0], "output", a.staged_bf16),
                   lambda a: setattr(a, "abi_version", 2)):
        assert status(mutate) in (abi.STATUS_INVALID_ARGUMENT, abi.STATUS_ABI_VERSION_MISMATCH)
