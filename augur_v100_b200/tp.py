"""Tensor-parallel sharding of the NVFP4 MLP block over the GPUs of one box.

Column-parallel gate|up: rank r owns output rows [r*I/p, (r+1)*I/p) of the gate and up
matrices (contiguous row slices of the code and scale planes) and computes its slice of
SiLU(gate)*up locally. Row-parallel down: rank r owns k-columns [r*I/p, (r+1)*I/p) of the
down matrix (a strided slice: I/(2p) code bytes and I/(16p) scale bytes of every row) and
produces a full-width [tokens, hidden] partial sum. One all-reduce (sum) of that partial
completes the block; the reference has no multi-GPU code, this is the only exchange step.
"""
from __future__ import annotations

import numpy as np


def check_shardable(hidden: int, intermediate: int, world: int) -> None:
    if world < 1 or intermediate % world != 0:
        raise ValueError("intermediate size must divide by the number of ranks")
    shard = intermediate // world
    if shard % 128 != 0:
        raise ValueError("each rank's slice of the intermediate dimension must be a multiple of 128")
    if hidden % 128 != 0:
        raise ValueError("hidden size must be a multiple of 128")


def shard_rows(codes: np.ndarray, scales: np.ndarray, rank: int, world: int):
    """Column-parallel slice (output rows) of a [rows, cols] weight in compact planes."""
    rows = codes.shape[0]
    lo, hi = rank * rows // world, (rank + 1) * rows // world
    return np.ascontiguousarray(codes[lo:hi]), np.ascontiguousarray(scales[lo:hi])


def shard_cols(codes: np.ndarray, scales: np.ndarray, rank: int, world: int):
    """Row-parallel slice (k columns) of a [rows, cols] weight in compact planes."""
    cols = codes.shape[1] * 2
    lo, hi = rank * cols // world, (rank + 1) * cols // world
    if lo % 16 or hi % 16:
        raise ValueError("k slices must fall on 16-element block boundaries")
    return np.ascontiguousarray(codes[:, lo // 2:hi // 2]), np.ascontiguousarray(scales[:, lo // 16:hi // 16])


def shard_mlp(gate, up, down, rank: int, world: int):
    """(codes, scales, global) triples of one rank's gate, up and down shards."""
    gc, gs = shard_rows(gate[0], gate[1], rank, world)
    uc, us = shard_rows(up[0], up[1], rank, world)
    dc, ds = shard_cols(down[0], down[1], rank, world)
    return (gc, gs, gate[2]), (uc, us, up[2]), (dc, ds, down[2])


class TensorParallelMlp:
    """One rank's share of the MLP block: local FFN program + all-reduce of the BF16 output."""

    def __init__(self, plan, gate, up, down, x, rank: int, world: int, process_group=None):
        from . import abi, host
        hidden, intermediate = gate[0].shape[1] * 2, gate[0].shape[0]
        check_shardable(hidden, intermediate, world)
        g, u, d = shard_mlp(gate, up, down, rank, world)
        shard = intermediate // world
        stream = plan.stream
        self.gate_up = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(
            stream, abi.LAYOUT_STREAM_PAIR, shard, hidden, g[0], g[1], g[2], u[0], u[1], u[2])
        self.down = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_STREAM, hidden, shard, *d)
        self.program = host.Nvfp4Sm100FfnProgram.bind(plan, self.gate_up, self.down, x)
        self.world, self.group = world, process_group

    @property
    def out(self):
        return self.program.out

    def submit(self) -> None:
        """Enqueue the local block and, with more than one rank, the all-reduce of its output."""
        self.program.submit_for_plan()
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(self.program.out, group=self.group)
