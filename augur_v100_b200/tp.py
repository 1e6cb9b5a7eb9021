"""Tensor-parallel sharding of the NVFP4 MLP block over the GPUs of one box.

Column-parallel gate|up: rank r owns output rows [r*I/p, (r+1)*I/p) of the gate and up
matrices (contiguous row slices of the code and scale planes) and computes its slice of
SiLU(gate)*up locally. Row-parallel down: rank r owns k-columns [r*I/p, (r+1)*I/p) of the
down matrix (a strided slice: I/(2p) code bytes and I/(16p) scale bytes of every row) and
produces a full-width [tokens, hidden] partial sum. One all-reduce (sum) of that partial
completes the block; the reference has no multi-GPU code, this is the only exchange step.

Two ways to do that exchange:

* fused (default when the ranks can map each other's memory): the down launch itself delivers
  every finished 32-row tile to all ranks over NVLink and adds the ranks' tiles in rank order
  (``augur_cuda_nvfp4_sm100_mlp_tp_*``); f32 partial sums, one rounding, no collective launch;
* NCCL: the local program writes a BF16 partial and ``torch.distributed.all_reduce`` sums it.
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


def exchange_extent(hidden: int, world: int) -> int:
    """Bytes of one rank's exchange buffer for a down projection with `hidden` output rows."""
    from ctypes import byref, c_uint64

    from . import abi
    out = c_uint64()
    result = abi.lib().augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(hidden, world, byref(out))
    if result.status != abi.STATUS_OK:
        raise ValueError(f"no exchange layout for hidden={hidden}, world={world}")
    return int(out.value)


class ExchangeBuffers:
    """Peer-mapped exchange buffers of all ranks.

    One object serves every program with the same output width: programs run one after another on the
    rank's stream, and every launch that uses the buffers advances a sequence number, on every rank alike.
    By default the launches count that sequence themselves (a counter in the tail of each rank's own
    buffer), so that bound programs can be captured into a CUDA graph and replayed; with
    `host_counted=True` the number is counted here and passed with every submit instead.
    Device memory comes from torch's symmetric-memory allocator (plumbing: it creates the
    allocation, exchanges the handles between the processes and maps every peer's buffer here).
    """

    def __init__(self, hidden: int, rank: int, world: int, process_group=None, host_counted: bool = False):
        import os

        import torch
        import torch.distributed as dist
        # Only plain peer stores are used: the buffers need no NVLink multicast object bound to them.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        group = process_group if process_group is not None else dist.group.WORLD
        self.rank, self.world, self.hidden = rank, world, hidden
        self.bytes = exchange_extent(hidden, world)
        self.tensor = symm.empty(self.bytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.tensor, group)
        self.pointers = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.pointers) != world or self.pointers[rank] != self.tensor.data_ptr():
            raise RuntimeError("symmetric-memory rendezvous returned an unexpected pointer table")
        self.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group)   # nobody publishes a flag before every buffer is zero
        self.host_counted = host_counted
        self.sequence = 0

    def next_sequence(self) -> int:
        """The `sequence` member of the next submit: 0 when the launches count on the device."""
        if not self.host_counted:
            return 0
        # 1, 2, ..., 0xFFFFFFFE, 1, ...: never 0 (the value of a fresh buffer), and the parity alternates across the wrap
        self.sequence = 1 if self.sequence >= 0xFFFFFFFE else self.sequence + 1
        return self.sequence

    def fill(self, args) -> None:
        """Writes the pointer table and this rank's place in it into an `MlpTpArgs` / `GemvTpArgs`."""
        for r, pointer in enumerate(self.pointers):
            args.exchange[r] = pointer
        args.exchange_len_bytes, args.world, args.rank = self.bytes, self.world, self.rank
        args.sequence = 0 if not self.host_counted else 1


class FusedExchangeProgram:
    """A bound FFN program of this rank's shards whose down launch also does the all-reduce."""

    def __init__(self, program, exchange: ExchangeBuffers):
        from ctypes import byref

        from . import abi, host
        down_rows = program.args.down.rows
        if exchange.hidden != down_rows:
            raise ValueError("exchange buffers were made for another hidden size")
        args = abi.header(abi.MlpTpArgs)
        args.gate_up, args.down = program.args.gate_up, program.args.down
        exchange.fill(args)
        plan = program.plan
        host._check("mlp_tp_preflight", abi.lib().augur_cuda_nvfp4_sm100_mlp_tp_preflight_v1(
            plan.stream.ordinal, plan.stream.handle, plan.handle, byref(args)))
        self.program, self.exchange, self.args = program, exchange, args

    @property
    def out(self):
        return self.program.out

    def submit_for_plan(self) -> None:
        from ctypes import byref

        from . import abi, host
        self.args.sequence = self.exchange.next_sequence()
        plan = self.program.plan
        host._check("mlp_tp_submit", abi.lib().augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1(
            plan.stream.ordinal, plan.stream.handle, plan.handle, byref(self.args)))


class RowParallelLinear:
    """A bound small-token projection over this rank's k-slice whose launch also does the all-reduce
    (the output projections outside the MLP block: every rank ends up with the full sum)."""

    def __init__(self, projection, exchange: ExchangeBuffers):
        from ctypes import byref

        from . import abi, host
        if exchange.hidden != projection.args.rows:
            raise ValueError("exchange buffers were made for another output width")
        args = abi.header(abi.GemvTpArgs)
        args.linear = projection.args
        exchange.fill(args)
        plan = projection.plan
        host._check("gemv_tp_preflight", abi.lib().augur_cuda_nvfp4_sm100_gemv_tp_preflight_v1(
            plan.stream.ordinal, plan.stream.handle, plan.handle, byref(args)))
        self.projection, self.exchange, self.args = projection, exchange, args

    @property
    def out(self):
        return self.projection.out

    def submit_for_plan(self) -> None:
        from ctypes import byref

        from . import abi, host
        self.args.sequence = self.exchange.next_sequence()
        plan = self.projection.plan
        host._check("gemv_tp_submit", abi.lib().augur_cuda_nvfp4_sm100_gemv_tp_prevalidated_submit_v1(
            plan.stream.ordinal, plan.stream.handle, plan.handle, byref(self.args)))


class TensorParallelMlp:
    """One rank's share of the MLP block, with the all-reduce fused into the down launch
    (`exchange` given) or done by NCCL on the BF16 partial (`exchange` None)."""

    def __init__(self, plan, gate, up, down, x, rank: int, world: int, process_group=None, exchange=None,
                 out=None):
        from . import abi, host
        hidden, intermediate = gate[0].shape[1] * 2, gate[0].shape[0]
        check_shardable(hidden, intermediate, world)
        g, u, d = shard_mlp(gate, up, down, rank, world)
        shard = intermediate // world
        stream = plan.stream
        self.gate_up = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(
            stream, abi.LAYOUT_STREAM_PAIR, shard, hidden, g[0], g[1], g[2], u[0], u[1], u[2])
        self.down = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(stream, abi.LAYOUT_STREAM, hidden, shard, *d)
        self.program = host.Nvfp4Sm100FfnProgram.bind(plan, self.gate_up, self.down, x, out=out)
        self.world, self.group = world, process_group
        self.fused = FusedExchangeProgram(self.program, exchange) if exchange is not None else None

    @property
    def out(self):
        return self.program.out

    def submit(self) -> None:
        """Enqueue the block; the result is the full sum on every rank when the call's work is done."""
        if self.fused is not None:
            self.fused.submit_for_plan()
            return
        self.program.submit_for_plan()
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(self.program.out, group=self.group)


class TensorParallelPrefillMlp:
    """One rank's share of the MLP block for wide inputs, processed in chunks of token rows.

    Per chunk: quantise x, gate|up GEMM with fused SwiGLU on this rank's intermediate slice, quantise the
    slice, down GEMM over this rank's k-slice -> a full-width BF16 partial; then one all-reduce (NCCL,
    BF16, sum) of the chunk's [rows, hidden] output. The all-reduce of chunk c runs on its own stream
    while the compute stream is already working on chunk c + 1, so that only the last chunk's
    collective is exposed.
    """

    def __init__(self, plan, gate_up_weight, down_weight, x, world: int, chunk_tokens: int = 4096, terms: int = 3,
                 input_global_scale: float = 2.0 ** -8, intermediate_global_scale: float = 2.0 ** -8,
                 process_group=None):
        """`gate_up_weight` / `down_weight`: this rank's shards, already on the device (interleaved gate|up rows
        of its intermediate slice; the matching k-slice of down), both in the tcgen05 layout."""
        import torch

        from . import host
        self.gate_up, self.down = gate_up_weight, down_weight
        tokens, hidden = x.shape
        self.out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=x.device)
        self.chunks = []
        for first in range(0, tokens, chunk_tokens):
            last = min(first + chunk_tokens, tokens)
            self.chunks.append(host.Nvfp4Sm100PrefillFfnProgram.bind(
                plan, self.gate_up, self.down, x[first:last], out=self.out[first:last], terms=terms,
                input_global_scale=input_global_scale, intermediate_global_scale=intermediate_global_scale))
        self.world, self.group, self.plan = world, process_group, plan
        self.compute = plan.stream.torch_stream
        self.comm = torch.cuda.Stream(device=x.device) if world > 1 else None
        self.events = [torch.cuda.Event() for _ in self.chunks] if world > 1 else []

    @classmethod
    def from_checkpoint(cls, plan, gate, up, down, x, rank: int, world: int, **options):
        """Shards full (codes, scales, global) matrices for `rank` and uploads the shards."""
        from . import abi, host
        hidden, intermediate = gate[0].shape[1] * 2, gate[0].shape[0]
        check_shardable(hidden, intermediate, world)
        if (intermediate // world) % 64 != 0:
            raise ValueError("each rank's slice of the intermediate dimension must be a multiple of 64")
        g, u, d = shard_mlp(gate, up, down, rank, world)
        shard = intermediate // world
        gate_up_weight = host.upload_gate_up_interleaved(plan.stream, shard, hidden, g[0], g[1], g[2], u[0], u[1], u[2])
        down_weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(plan.stream, abi.LAYOUT_TCGEN05, hidden, shard, *d)
        return cls(plan, gate_up_weight, down_weight, x, world, **options)

    def submit(self) -> None:
        """Enqueue all chunks; when it returns, the compute stream is ordered after the last all-reduce."""
        import torch
        import torch.distributed as dist
        for index, chunk in enumerate(self.chunks):
            chunk.submit_for_plan()
            if self.world > 1:
                self.events[index].record(self.compute)
                with torch.cuda.stream(self.comm):
                    self.comm.wait_event(self.events[index])
                    dist.all_reduce(chunk.out, group=self.group)
        if self.world > 1:
            self.compute.wait_stream(self.comm)
