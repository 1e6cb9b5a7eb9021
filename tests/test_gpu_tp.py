"""Tensor-parallel MLP on real GPUs (needs at least two): the all-reduce fused into the down launch
(peer stores and flags over NVLink), and the NCCL all-reduce of BF16 partial outputs."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOKENS = 8
SIZES = {"small": (1024, 4096), "full": (5120, 17408)}   # "full" is the benchmark's MLP block


def _inputs(size):
    from augur_v100_b200 import synth
    hidden, inter = SIZES[size]
    gate = synth.make_weight(0, 81, "gate", inter, hidden)
    up = synth.make_weight(0, 81, "up", inter, hidden)
    down = synth.make_weight(0, 81, "down", hidden, inter)
    x = synth.f32_to_bf16_bits(np.random.default_rng(81).standard_normal((TOKENS, hidden)).astype(np.float32) * 8)
    return gate, up, down, x


def _worker(rank, world, port, queue, fused, size):
    import torch
    import torch.distributed as dist
    from augur_v100_b200 import host, tp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    hidden, inter = SIZES[size]
    gate, up, down, x_bits = _inputs(size)
    stream = host.Stream(rank)
    plan = host.Plan(stream, host.mlp_scratch_bytes(hidden, inter // world))
    x = torch.from_numpy(x_bits.view(np.int16)).to(torch.device("cuda", rank)).view(torch.bfloat16)
    exchange = tp.ExchangeBuffers(hidden, rank, world) if fused else None
    block = tp.TensorParallelMlp(plan, gate, up, down, x, rank, world, exchange=exchange)
    # Different inputs on consecutive submits: a tile or a flag left over from an earlier
    # sequence (same parity two submits back) would show in the last result.
    final = x.clone()
    for scale in (0.5, 2.0, -1.0, 1.0):
        x.copy_(final * scale)
        block.submit()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    queue.put((rank, block.out.view(torch.int16).cpu().numpy().view(np.uint16),
               block.program.intermediate.view(torch.int16).cpu().numpy().view(np.uint16)))
    dist.barrier()
    dist.destroy_process_group()
    plan.close()


@pytest.mark.parametrize("world,fused,size", [(2, True, "small"), (2, False, "small"), (4, True, "small"), (8, True, "small"),
                                              (2, True, "full"), (4, True, "full"), (8, True, "full")],
                         ids=["2-fused-exchange", "2-nccl", "4-fused-exchange", "8-fused-exchange",
                              "2-fused-exchange-full-size", "4-fused-exchange-full-size", "8-fused-exchange-full-size"])
def test_tensor_parallel_mlp_matches_oracle(world, fused, size):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    import oracle
    from augur_v100_b200 import synth
    from helpers import TOLERANCE, rel_error, rms_error
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, queue, fused, size)) for r in range(world)]
    for p in procs:
        p.start()
    results = {rank: (out, h) for rank, out, h in (queue.get(timeout=600) for _ in range(world))}
    got = results[0][0]
    if fused:   # every rank adds the same tiles in the same order
        for rank in range(1, world):
            assert np.array_equal(got, results[rank][0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    hidden, inter = SIZES[size]
    gate, up, down, x_bits = _inputs(size)
    threads = oracle.max_threads()
    h64, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, x_bits, threads=threads)
    # rank r holds columns [r * inter / world, (r + 1) * inter / world) of the intermediate
    h_bits = np.concatenate([results[rank][1].reshape(TOKENS, inter // world) for rank in range(world)], axis=1)
    assert rel_error(h_bits, h64) <= TOLERANCE
    y64_from_h = oracle.linear_f64(down[0], down[1], down[2], hidden, inter, h_bits, threads=threads)
    if fused:
        # f32 partial sums of all ranks added in rank order, one rounding: the standard bound of a single GEMM
        assert rel_error(got, y64_from_h) <= TOLERANCE
    else:
        # NCCL adds per-rank BF16 partials: `world` roundings of partial sums that may cancel, so the bound
        # is taken against the rms of the output
        assert rms_error(got, y64_from_h) <= TOLERANCE
    assert rms_error(got, y64) <= TOLERANCE


P_HIDDEN, P_INTER, P_TOKENS, P_CHUNK = 512, 1024, 640, 256


def _prefill_inputs():
    from augur_v100_b200 import synth
    gate = synth.make_weight(1, 82, "gate", P_INTER, P_HIDDEN)
    up = synth.make_weight(1, 82, "up", P_INTER, P_HIDDEN)
    down = synth.make_weight(1, 82, "down", P_HIDDEN, P_INTER)
    x = synth.f32_to_bf16_bits(np.random.default_rng(82).standard_normal((P_TOKENS, P_HIDDEN)).astype(np.float32) * 8)
    return gate, up, down, x


def _prefill_worker(rank, world, port, queue, h_absmax):
    import torch
    import torch.distributed as dist
    from augur_v100_b200 import host, synth, tp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    gate, up, down, x_bits = _prefill_inputs()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        stream = host.Stream(rank, side)
        plan = host.Plan(stream, 1 << 20)
        x = torch.from_numpy(x_bits.view(np.int16)).to(torch.device("cuda", rank)).view(torch.bfloat16)
        block = tp.TensorParallelPrefillMlp.from_checkpoint(
            plan, gate, up, down, x, rank, world, chunk_tokens=P_CHUNK, terms=3,
            input_global_scale=host.default_activation_global_scale(float(np.abs(synth.bf16_bits_to_f32(x_bits)).max())),
            intermediate_global_scale=host.default_activation_global_scale(h_absmax * 1.05))
        for _ in range(2):
            block.submit()
        side.synchronize()
        assert plan.device_status() == 0
        queue.put((rank, block.out.view(torch.int16).cpu().numpy().view(np.uint16)))
        dist.barrier()
    dist.destroy_process_group()
    plan.close()


def test_two_rank_chunked_prefill_mlp_matches_oracle():
    # 640 token rows in chunks of 256 (the last one ragged), each chunk's all-reduce on its own stream
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    import oracle
    from augur_v100_b200 import synth
    gate, up, down, x_bits = _prefill_inputs()
    h64, y64 = oracle.mlp_f64(gate, up, down, P_HIDDEN, P_INTER, x_bits, threads=8)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_prefill_worker, args=(r, 2, port, queue, float(np.abs(h64).max()))) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert np.array_equal(results[0], results[1])
    y = synth.bf16_bits_to_f32(results[0]).astype(np.float64).reshape(y64.shape)
    rms = np.sqrt(np.mean(y64 * y64))
    assert np.max(np.abs(y - y64) / np.maximum(np.abs(y64), rms)) <= 2e-2
