"""Tensor-parallel sharding logic on the CPU: two gloo ranks, oracle arithmetic per shard."""
import os
import socket

import numpy as np
import pytest

import oracle
from augur_v100_b200 import synth, tp

HIDDEN, INTER, TOKENS = 256, 512, 8


def _weights():
    return (synth.make_weight(0, 80, "gate", INTER, HIDDEN), synth.make_weight(0, 80, "up", INTER, HIDDEN),
            synth.make_weight(0, 80, "down", HIDDEN, INTER))


def _x():
    return synth.f32_to_bf16_bits(np.random.default_rng(80).standard_normal((TOKENS, HIDDEN)).astype(np.float32) * 8)


def _rank_partial(rank, world):
    gate, up, down = _weights()
    g, u, d = tp.shard_mlp(gate, up, down, rank, world)
    shard = INTER // world
    h64, partial = oracle.mlp_f64(g, u, d, HIDDEN, shard, _x())
    return h64, partial


def test_shards_partition_the_planes():
    gate, up, down = _weights()
    for world in (1, 2, 4):
        tp.check_shardable(HIDDEN, INTER, world)
        rows = [tp.shard_rows(gate[0], gate[1], r, world) for r in range(world)]
        assert np.array_equal(np.concatenate([r[0] for r in rows]), gate[0])
        assert np.array_equal(np.concatenate([r[1] for r in rows]), gate[1])
        cols = [tp.shard_cols(down[0], down[1], r, world) for r in range(world)]
        assert np.array_equal(np.concatenate([c[0] for c in cols], axis=1), down[0])
        assert np.array_equal(np.concatenate([c[1] for c in cols], axis=1), down[1])
    with pytest.raises(ValueError):
        tp.check_shardable(HIDDEN, INTER, 8)      # 64-column slices are not a multiple of 128
    with pytest.raises(ValueError):
        tp.check_shardable(HIDDEN, INTER, 3)


def test_sum_of_rank_partials_equals_the_unsharded_block():
    gate, up, down = _weights()
    _, full = oracle.mlp_f64(gate, up, down, HIDDEN, INTER, _x())
    for world in (2, 4):
        total = sum(_rank_partial(r, world)[1] for r in range(world))
        assert np.allclose(total, full, rtol=1e-9, atol=1e-12)


def _worker(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _, partial = _rank_partial(rank, world)
    # the exchange step: partials are rounded to BF16 and summed, as the GPU path does
    t = torch.from_numpy(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(partial.astype(np.float32))).copy())
    dist.all_reduce(t)
    dist.barrier()
    if rank == 0:
        queue.put(t.numpy())
    dist.destroy_process_group()


def test_two_gloo_ranks_all_reduce_to_the_full_result():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    reduced = queue.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    gate, up, down = _weights()
    _, full = oracle.mlp_f64(gate, up, down, HIDDEN, INTER, _x())
    rms = np.sqrt(np.mean(full * full))
    assert np.max(np.abs(reduced - full)) / rms <= 2e-2


def test_exchange_sequence_never_yields_zero_and_alternates_parity_across_the_wrap():
    from augur_v100_b200 import tp
    exchange = tp.ExchangeBuffers.__new__(tp.ExchangeBuffers)   # the counter alone; no device is touched
    exchange.sequence, exchange.host_counted = 0, True
    assert [exchange.next_sequence() for _ in range(3)] == [1, 2, 3]
    exchange.sequence = 0xFFFFFFFC
    wrapped = [exchange.next_sequence() for _ in range(4)]
    assert wrapped == [0xFFFFFFFD, 0xFFFFFFFE, 1, 2]
    assert all((a ^ b) & 1 for a, b in zip(wrapped, wrapped[1:]))
    # launches that count on the device are passed 0 every time
    exchange.host_counted = False
    assert [exchange.next_sequence() for _ in range(2)] == [0, 0]
    # the device-side rule (launch count -> sequence) is the same series: never 0, parity alternating across the wrap
    assert [launches % 0xFFFFFFFE + 1 for launches in (0, 1, 2)] == [1, 2, 3]
    device = [launches % 0xFFFFFFFE + 1 for launches in (0xFFFFFFFC, 0xFFFFFFFD, 0xFFFFFFFE, 0xFFFFFFFF, 0, 1)]   # the u32 counter wraps too
    assert 0 not in device and all((a ^ b) & 1 for a, b in zip(device, device[1:]))


def test_exchange_extent_matches_the_layout():
    from augur_v100_b200 import tp
    # [2 parities][world][hidden / 32 row groups] tiles of 256 {value, flag} pairs (8 bytes each)
    # and 256 bytes at the end for the sequence counter of launches that count on the device
    assert tp.exchange_extent(5120, 8) == 2 * 8 * 160 * 256 * 8 + 256
    assert tp.exchange_extent(1024, 2) == 2 * 2 * 32 * 2048 + 256
    import pytest
    with pytest.raises(ValueError):
        tp.exchange_extent(5120, 9)
