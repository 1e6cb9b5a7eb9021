"""The small-token linear for hosts that may not allocate device memory.

Some hosts give all device memory to their own arena when they start, or run their serving loop
under a checked no-allocation rule; such a host cannot create a plan (plan creation calls
cudaMalloc). `augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1` serves them from a fixed
scratch array inside the library. This test calls it through the C ABI, twice in a row, and checks
each result against the plan-based entry point on the same inputs and against the CPU oracle; it
also checks that the call allocates nothing, that the entry's status word reads clean, that the
other two epilogues work from the fixed array, and that a shape too large for it is refused.

Collected last on purpose (file name), so that a run that stops at the first failure has already
executed every other test.
"""
from ctypes import byref

import numpy as np
import pytest

from ctypes import c_uint32

import oracle
from augur_v100_b200 import abi, synth
from helpers import TOLERANCE, bits_from_torch_bf16, rel_error, rel_error_f32, torch_bf16_from_bits

pytestmark = pytest.mark.gpu


def _max_rel_diff(a_bits, b_bits):
    a = synth.bf16_bits_to_f32(a_bits).astype(np.float64)
    b = synth.bf16_bits_to_f32(b_bits).astype(np.float64)
    rms = float(np.sqrt(np.mean(b * b))) or 1.0
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3 * rms)))


def test_static_scratch_entry_matches_plan_entry_twice_and_allocates_nothing():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    lib = abi.lib()
    stream = host.Stream(0)
    rows, cols, tokens = 2048, 5120, 8            # cut between CTAs: exercises the scratch slots and counters
    codes, scales, glob = synth.make_weight(3, 95, "w", rows, cols)
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_STREAM, rows, cols, codes, scales, glob)
    plan = host.Plan(stream, host.gemv_scratch_bytes(rows, cols, tokens))
    try:
        for call in range(2):
            x = torch_bf16_from_bits(synth.make_activation(call, 95, "x", tokens, cols), device)
            reference = host.Nvfp4Sm100Projection.bind(plan, weight, x)
            reference.submit_for_plan()
            stream.synchronize()
            out = torch.full((tokens, rows), float("nan"), dtype=torch.bfloat16, device=device)
            args = host.gemv_args(weight, x, out, abi.EPILOGUE_LINEAR_BF16)
            allocations = host.allocation_snapshot()
            torch_allocations = torch.cuda.memory_stats()["allocation.all.allocated"]
            result = lib.augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1(stream.ordinal, stream.handle, byref(args))
            assert result.status == abi.STATUS_OK, (result.status, result.raw_cuda_status)
            stream.synchronize()
            assert host.allocation_snapshot() == allocations
            assert torch.cuda.memory_stats()["allocation.all.allocated"] == torch_allocations
            got, want = bits_from_torch_bf16(out), bits_from_torch_bf16(reference.out)
            assert _max_rel_diff(got, want) <= TOLERANCE, call
            # and against the reference arithmetic itself, not only against this library's other entry
            y64 = oracle.linear_f64(codes, scales, glob, rows, cols, synth.make_activation(call, 95, "x", tokens, cols),
                                    threads=oracle.max_threads())
            assert rel_error(got, y64) <= TOLERANCE, call
            word = c_uint32(0xFFFFFFFF)
            result = lib.augur_cuda_nvfp4_sm100_static_scratch_status_v1(stream.ordinal, stream.handle, byref(word))
            assert result.status == abi.STATUS_OK and word.value == 0
        # the f32 epilogue from the fixed array
        out32 = torch.full((tokens, rows), float("nan"), dtype=torch.float32, device=device)
        args = host.gemv_args(weight, x, out32, abi.EPILOGUE_LINEAR_F32)
        result = lib.augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1(stream.ordinal, stream.handle, byref(args))
        assert result.status == abi.STATUS_OK, (result.status, result.raw_cuda_status)
        stream.synchronize()
        assert rel_error_f32(out32.cpu().numpy(), y64) <= TOLERANCE
        # the fused SiLU(gate) * up epilogue (paired layout), against the plan entry bit for bit
        pair_rows = 1024
        gate = synth.make_weight(4, 95, "gate", pair_rows, cols)
        up = synth.make_weight(4, 95, "up", pair_rows, cols)
        pair = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_STREAM_PAIR, pair_rows, cols, *gate, *up)
        pair_plan = host.Plan(stream, host.gemv_scratch_bytes(pair_rows, cols, tokens))
        try:
            reference = host.Nvfp4Sm100Projection.bind(pair_plan, pair, x)
            reference.submit_for_plan()
            stream.synchronize()
            out = torch.full((tokens, pair_rows), float("nan"), dtype=torch.bfloat16, device=device)
            args = host.gemv_args(pair, x, out, abi.EPILOGUE_SWIGLU_BF16)
            result = lib.augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1(stream.ordinal, stream.handle, byref(args))
            assert result.status == abi.STATUS_OK, (result.status, result.raw_cuda_status)
            stream.synchronize()
            assert torch.equal(out.view(torch.int16), reference.out.view(torch.int16))
        finally:
            pair_plan.close()
        out = torch.empty((tokens, rows), dtype=torch.bfloat16, device=device)
        # too large for the fixed array: refused before anything is enqueued
        big_rows, big_cols = 32768, 17408
        launches = host.launch_count()
        args = abi.header(abi.GemvArgs)
        args.weight, args.weight_len_bytes = weight.packed.data_ptr(), big_rows * big_cols * 9 // 16
        args.input_bf16, args.input_len_bytes = x.data_ptr() + (1 << 40), tokens * big_cols * 2
        args.output, args.output_len_bytes = out.data_ptr() + (2 << 40), tokens * big_rows * 2
        args.rows, args.cols, args.tokens, args.global_scale = big_rows, big_cols, tokens, glob
        result = lib.augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1(stream.ordinal, stream.handle, byref(args))
        assert result.status == abi.STATUS_INVALID_ARGUMENT
        assert host.launch_count() == launches
    finally:
        plan.close()
        stream.close()
