"""Tensor-parallel MLP on real GPUs (needs at least two): NCCL all-reduce of the BF16 partial outputs."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HIDDEN, INTER, TOKENS = 1024, 4096, 8


def _inputs():
    from augur_v100_b200 import synth
    gate = synth.make_weight(0, 81, "gate", INTER, HIDDEN)
    up = synth.make_weight(0, 81, "up", INTER, HIDDEN)
    down = synth.make_weight(0, 81, "down", HIDDEN, INTER)
    x = synth.f32_to_bf16_bits(np.random.default_rng(81).standard_normal((TOKENS, HIDDEN)).astype(np.float32) * 8)
    return gate, up, down, x


def _worker(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    from augur_v100_b200 import host, tp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    gate, up, down, x_bits = _inputs()
    stream = host.Stream(rank)
    plan = host.Plan(stream, host.mlp_scratch_bytes(HIDDEN, INTER // world))
    x = torch.from_numpy(x_bits.view(np.int16)).to(torch.device("cuda", rank)).view(torch.bfloat16)
    block = tp.TensorParallelMlp(plan, gate, up, down, x, rank, world)
    for _ in range(2):
        block.submit()
    torch.cuda.synchronize()
    if rank == 0:
        queue.put(block.out.view(torch.int16).cpu().numpy().view(np.uint16))
    dist.barrier()
    dist.destroy_process_group()
    plan.close()


def test_two_rank_tensor_parallel_mlp_matches_oracle():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import oracle
    from augur_v100_b200 import synth
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    got = queue.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    gate, up, down, x_bits = _inputs()
    _, y64 = oracle.mlp_f64(gate, up, down, HIDDEN, INTER, x_bits, threads=4)
    y = synth.bf16_bits_to_f32(got).astype(np.float64).reshape(y64.shape)
    assert np.max(np.abs(y - y64)) / np.sqrt(np.mean(y64 * y64)) <= 4e-2
