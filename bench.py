#!/usr/bin/env python
"""Benchmark of the NVFP4 quantized-linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (sm_100a kernels)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path, timed on host cores

Headline workload (configuration 1 of the benchmark definition): the 27B-class NVFP4 MLP block at the
fixed 8-row verify batch - gate|up 5120 -> 2x17408 fused with SiLU(gate)*up, then down 17408 -> 5120 -
with synthetic weights of the benchmark's value distributions. One pass streams LAYERS distinct layers
(2.4 GB of weights at N=1, far more than L2), so every weight byte comes from HBM; one step is PASSES
such passes, so that the timed region of a default run lasts about a second. With N > 1 the block is
tensor-parallel: column-parallel gate|up, row-parallel down, the all-reduce of the 8 x 5120 output
inside the down launch (peer stores over NVLink) or by NCCL.

Two small-token kernels exist. On one GPU the headline runs the block as ONE launch of the tensor-memory kernel
(`tc_program_kernel`: tcgen05 block-scaled MMA straight on the weight tiles TMA delivers); with N > 1 it runs the
`mma.sync` kernel (`gemv_kernel`, two launches per block), which carries the fused exchange. `--small-token-kernel`
overrides the choice on one GPU.

Prints one JSON line (rank 0). `value` is whole-job GB/s of algorithmic bytes with inputs resident in
HBM; `e2e` is the same through the public host API with the activations copied from pinned host memory
and the result read back for every pass. The other configurations of the benchmark definition are
reported under their own keys of the same line, each outside the headline's timed region:
`config0` (single 17408 x 5120 linear, M=8), `config1_m1` (the MLP block at M=1), `config1_other_kernel`
(the block on the small-token kernel that the headline does not use), `config2_prefill` (M=4096 GEMMs), `config3_sweep` (64-layer whole-model linear
sweep at M=8), `config4_prefill_mlp` (chunked tensor-parallel prefill MLP), `head_bf16` (the BF16 vocabulary head),
`norm_group` (RMSNorm + stage + four projections of one input, grouped against one launch per projection); with more than
one GPU also `config1_shard_without_exchange` (every rank's shard of the block alone: what the exchange and rank skew cost).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

HIDDEN, INTER, TOKENS, LAYERS = 5120, 17408, 8, 16
PASSES = 64
ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def layer_bytes(tokens: int = TOKENS) -> int:
    """Algorithmic bytes of one MLP layer: every weight byte once + the input + the output (whole job)."""
    weights = 3 * HIDDEN * INTER * 9 // 16          # 0.5 B code + 1/16 B scale per element
    return weights + 2 * tokens * HIDDEN * 2


def linear_bytes(rows: int, cols: int, tokens: int) -> int:
    return rows * cols * 9 // 16 + tokens * cols * 2 + tokens * rows * 2


def measured_peaks():
    """(HBM GB/s, dense BF16 TFLOP/s burst, source) from the driver-written file, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return float(data["hbm_gbs"]), float(data["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (earlier measurement on this pool)"


DATASHEET_FP4_TFLOPS = 9000.0    # dense NVFP4 per B200; no measured FP4 figure exists on this pool


KERNELS = {
    # name of the choice -> (kernel, launches per block, tracked ncu summary, dtype line)
    "tensor_memory": ("tc_program_kernel", 1, "tc_program_kernel_mlp_m8.md",
                      "e2m1 x e2m1 -> f32 on tcgen05 (kind::mxf4nvf4, E4M3 block scales in the MMA); BF16 activations as eight exact radix-8 NVFP4 terms"),
    "mma_sync": ("gemv_kernel", 2, "gemv_kernel_mlp_m8.md",
                 "bf16 x bf16 -> f32 (E2M1 codes as BF16 fragments on mma.sync, E4M3 block scales applied in f32)"),
}


def recorded_traffic(summary):
    """DRAM bytes of the launches of one MLP block from the tracked ncu summary of the kernel, or None."""
    path = os.path.join(ROOT, "profiles", summary)
    try:
        with open(path) as handle:
            match = re.search(r"dram_bytes_per_(?:launch_pair|block):\s*([0-9.eE+]+)", handle.read())
        return float(match.group(1)) if match else None
    except OSError:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.window = [None, None]     # wall-clock bounds of the timed region

    def mark_begin(self):
        self.window[0] = time.time()

    def mark_end(self):
        self.window[1] = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [field.strip() for field in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        begin, end = self.window
        for stamp, row in self.rows:
            if len(row) < 9 or (begin is not None and stamp < begin) or (end is not None and stamp > end + 0.05):
                continue
            try:
                sm.append(float(row[1]))
                sm_max.append(float(row[2]))
            except ValueError:
                continue
            for name, field in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[5:9]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# the CPU path (C restatement of the reference's Rust, all host threads): the reference arm, and
# the cpu_baseline of the library arm. One procedure for both.
# ---------------------------------------------------------------------------------------------
def cpu_mlp_planes(inter: int):
    """Synthetic gate / up / down planes of an MLP block with intermediate size `inter` (a multiple of 128)."""
    from augur_v100_b200 import synth
    gate = synth.make_weight(0, 1, "gate", inter, HIDDEN)
    up = synth.make_weight(0, 1, "up", inter, HIDDEN)
    down = synth.make_weight(0, 1, "down", HIDDEN, inter)
    x = synth.f32_to_bf16_bits(np.random.default_rng(0).standard_normal((TOKENS, HIDDEN)).astype(np.float32) * 8.0)
    return gate, up, down, x


def cpu_layer_seconds(threads: int, repeats: int, inter: int = INTER):
    """Times `repeats` passes of one MLP layer (M=8) with intermediate size `inter` through the CPU oracle."""
    import oracle
    gate, up, down, x = cpu_mlp_planes(inter)
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        oracle.mlp_bf16(gate, up, down, HIDDEN, inter, x, threads=threads)
        times.append(time.perf_counter() - start)
    return times


def mlp_bytes(inter: int) -> int:
    return 3 * HIDDEN * inter * 9 // 16 + 2 * TOKENS * HIDDEN * 2


REFERENCE_BUDGET_SECONDS = 150.0


def cpu_reference_run(warmup: int, steps: int, budget_seconds: float):
    """`warmup` untimed and `steps` timed CPU steps within the budget; returns (GB/s, seconds per step, sample, threads).

    A step is one pass over one MLP layer, or over a slice of it (the first `inter` intermediate columns of
    gate, up and down: the same arithmetic per byte) when whole layers would not fit the budget."""
    import oracle
    threads = oracle.max_threads()
    probe_inter = 1024
    probe = min(cpu_layer_seconds(threads, 2, probe_inter))
    per_step = budget_seconds / max(warmup + steps, 1)
    inter = int(min(INTER, max(128, per_step / probe * probe_inter))) // 128 * 128
    times = cpu_layer_seconds(threads, warmup + steps, inter)[warmup:]
    seconds = sum(times) / len(times)
    sample = (f"one MLP layer (M=8, 5120 -> 2x{inter} -> 5120) per step, mean of {steps} steps after {warmup} warm-up"
              + ("" if inter == INTER else f": the first {inter} of {INTER} intermediate columns, to fit the steps in {budget_seconds:.0f} s"))
    return mlp_bytes(inter) / seconds / 1e9, seconds, sample, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, seconds, sample, threads = cpu_reference_run(args.warmup, args.steps, REFERENCE_BUDGET_SECONDS)
    print(json.dumps({
        "impl": "reference", "metric": "nvfp4_linear_m8_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config1: NVFP4 MLP block, M=8, hidden 5120, intermediate 17408; " + sample,
                   "host_threads": threads},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------
def device_planes(torch, generator, rows, cols, device):
    """Random compact planes made on the device: uniform codes, |N(0,1)|*0.5 scales (E4M3, RNE), in 0x01..0x7e."""
    codes = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device=device, generator=generator)
    raw = (torch.randn((rows, cols // 16), device=device, generator=generator).abs() * 0.5).clamp(2.0 ** -9, 448.0)
    scales = raw.to(torch.float8_e4m3fn).view(torch.uint8).clamp(1, 0x7E)
    return codes, scales


class Context:
    """What every part of the run shares: device, stream, ranks, timing helpers."""

    def __init__(self, torch, dist, host, abi, device, stream, side, world, rank):
        self.torch, self.dist, self.host, self.abi = torch, dist, host, abi
        self.device, self.stream, self.side, self.world, self.rank = device, stream, side, world, rank
        self.hbm_peak, self.bf16_peak, self.peak_source = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, body, steps):
        """Milliseconds for `steps` calls of `body`: CUDA events on the launching stream, barrier and device
        synchronisation on both sides, the maximum over ranks."""
        torch = self.torch
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            body()
        end.record()
        self.barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=self.device)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def hbm_entry(self, per_gpu_bytes, total_bytes, ms):
        achieved = per_gpu_bytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "gbs": total_bytes / (ms * 1e-3) / 1e9,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": self.hbm_peak, "unit": "GB/s",
                             "frac": achieved / self.hbm_peak, "peak_source": self.peak_source, "traffic": None}}


def build_mlp_layers(ctx, layers, keep_first_planes=False, kernel="mma_sync", seed=1234):
    """`layers` distinct MLP layers of this rank's shard in the hot layouts of `kernel`; optionally the compact planes
    of the first, on the host."""
    from augur_v100_b200 import synth
    torch, host, abi = ctx.torch, ctx.host, ctx.abi
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(seed + ctx.rank)
    shard = INTER // ctx.world

    def interleave(gate_plane, up_plane):   # 16 gate rows, then the matching 16 up rows
        width = gate_plane.shape[1]
        return torch.stack([gate_plane.view(shard // 16, 16, width), up_plane.view(shard // 16, 16, width)], dim=1).reshape(2 * shard, width).contiguous()

    built, first = [], None
    for index in range(layers):
        gc, gs = device_planes(torch, generator, shard, HIDDEN, ctx.device)
        uc, us = device_planes(torch, generator, shard, HIDDEN, ctx.device)
        dc, ds = device_planes(torch, generator, HIDDEN, shard, ctx.device)
        if kernel == "tensor_memory":
            gate_up = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_TCGEN05, 2 * shard, HIDDEN, interleave(gc, uc),
                                                                 interleave(gs, us), synth.GLOBAL_SCALE)
            gate_up.global_scale_b = synth.GLOBAL_SCALE
            down = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_TCGEN05, HIDDEN, shard, dc, ds, synth.GLOBAL_SCALE)
        else:
            gate_up = host.Nvfp4Sm100Weight.repack_device_planes(
                ctx.stream, abi.LAYOUT_STREAM_PAIR, shard, HIDDEN, gc, gs, synth.GLOBAL_SCALE, uc, us, synth.GLOBAL_SCALE)
            down = host.Nvfp4Sm100Weight.repack_device_planes(
                ctx.stream, abi.LAYOUT_STREAM, HIDDEN, shard, dc, ds, synth.GLOBAL_SCALE)
        if index == 0 and keep_first_planes:
            first = tuple((c.cpu().numpy(), s.cpu().numpy(), synth.GLOBAL_SCALE) for c, s in ((gc, gs), (uc, us), (dc, ds)))
        built.append((gate_up, down))
        del gc, gs, uc, us, dc, ds
    return built, first


def bits(t):
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rel_error(y_bits, y64):
    """max |y - y64| / max(|y64|, 1e-3 rms(y64)): the bound of one GEMM output against the fp64 oracle."""
    from augur_v100_b200 import synth
    y = synth.bf16_bits_to_f32(y_bits).astype(np.float64).reshape(y64.shape)
    rms = float(np.sqrt(np.mean(y64 * y64))) or 1.0
    return float(np.max(np.abs(y - y64) / np.maximum(np.abs(y64), 1e-3 * rms)))


def rms_error(y_bits, y64):
    """max |y - y64| / rms(y64)."""
    from augur_v100_b200 import synth
    y = synth.bf16_bits_to_f32(y_bits).astype(np.float64).reshape(y64.shape)
    rms = float(np.sqrt(np.mean(y64 * y64))) or 1.0
    return float(np.max(np.abs(y - y64)) / rms)


def config0_probe(ctx):
    """Configuration 0: the single 17408 x 5120 linear at M=8, eight distinct weights in rotation (400 MB, more than L2)."""
    import oracle
    from augur_v100_b200 import synth
    torch, host, abi = ctx.torch, ctx.host, ctx.abi
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(99)
    rows, cols, count = INTER, HIDDEN, 8
    plan = host.Plan(ctx.stream, host.gemv_scratch_bytes(rows, cols, TOKENS))
    x = torch.randn((TOKENS, cols), device=ctx.device, generator=generator).to(torch.bfloat16)
    projections, first = [], None
    for index in range(count):
        codes, scales = device_planes(torch, generator, rows, cols, ctx.device)
        weight = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_STREAM, rows, cols, codes, scales, synth.GLOBAL_SCALE)
        if index == 0:
            first = (codes.cpu().numpy(), scales.cpu().numpy())
        projections.append(host.Nvfp4Sm100Projection.bind(plan, weight, x))
        del codes, scales

    def sweep():
        for projection in projections:
            projection.submit_for_plan()

    for _ in range(3):
        sweep()
    rounds = 50
    ms = ctx.timed(sweep, rounds) / (rounds * count)
    entry = ctx.hbm_entry(linear_bytes(rows, cols, TOKENS), linear_bytes(rows, cols, TOKENS), ms)
    entry["workload"] = f"config0: single NVFP4 linear, M={TOKENS}, K={cols}, N={rows}; {count} distinct weights in rotation"
    y64 = oracle.linear_f64(first[0], first[1], synth.GLOBAL_SCALE, rows, cols, bits(x), threads=oracle.max_threads())
    projections[0].submit_for_plan()
    ctx.stream.synchronize()
    entry["parity"] = {"rel_error_vs_fp64_oracle": rel_error(bits(projections[0].out), y64), "bound": 2e-2}
    entry["device_status"] = plan.device_status()
    entry["kernel"] = KERNELS["mma_sync"][0]
    del projections
    plan.close()
    torch.cuda.empty_cache()

    # the same linear on the tensor-memory kernel (weights in the tcgen05 layout)
    generator.manual_seed(99)
    torch.randn((TOKENS, cols), device=ctx.device, generator=generator)   # the same draws as above: x, then the planes
    plan = host.Plan(ctx.stream, host.gemv_tc_scratch_bytes(rows, cols))
    projections = []
    for index in range(count):
        codes, scales = device_planes(torch, generator, rows, cols, ctx.device)
        weight = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_TCGEN05, rows, cols, codes, scales, synth.GLOBAL_SCALE)
        projections.append(host.Nvfp4Sm100TcProjection.bind(plan, weight, x))
        del codes, scales
    for _ in range(3):
        sweep()
    other = ctx.hbm_entry(linear_bytes(rows, cols, TOKENS), linear_bytes(rows, cols, TOKENS), ctx.timed(sweep, rounds) / (rounds * count))
    projections[0].submit_for_plan()
    ctx.stream.synchronize()
    other["parity"] = {"rel_error_vs_fp64_oracle": rel_error(bits(projections[0].out), y64), "bound": 2e-2}
    other["device_status"] = plan.device_status()
    other["kernel"] = KERNELS["tensor_memory"][0]
    entry["tensor_memory_kernel"] = other
    del projections
    plan.close()
    return entry


def other_kernel_probe(ctx, kernel):
    """Configuration 1 on the small-token kernel the headline does not use: eight distinct layers in rotation (1.2 GB
    of weights); parity of the first against the CPU oracle."""
    import oracle
    torch, host = ctx.torch, ctx.host
    count = 8
    layers, first = build_mlp_layers(ctx, count, keep_first_planes=True, kernel=kernel, seed=2024)
    tensor_memory = kernel == "tensor_memory"
    plan = host.Plan(ctx.stream, host.mlp_tc_scratch_bytes(HIDDEN, INTER) if tensor_memory else host.mlp_scratch_bytes(HIDDEN, INTER))
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(77)
    x = torch.randn((TOKENS, HIDDEN), device=ctx.device, generator=generator).mul_(8.0).to(torch.bfloat16)
    program_type = host.Nvfp4Sm100TcFfnProgram if tensor_memory else host.Nvfp4Sm100FfnProgram
    programs = [program_type.bind(plan, gate_up, down, x) for gate_up, down in layers]

    def sweep():
        for program in programs:
            program.submit_for_plan()

    for _ in range(3):
        sweep()
    reps = 40
    launches_before = host.launch_count()
    ms = ctx.timed(sweep, reps) / (reps * count)
    launches = (host.launch_count() - launches_before) // (reps * count)
    entry = ctx.hbm_entry(layer_bytes(), layer_bytes(), ms)
    entry.update({"workload": f"config1 on {KERNELS[kernel][0]}: the MLP block, M={TOKENS}; {count} distinct layers in rotation; ms per layer",
                  "kernel": KERNELS[kernel][0], "launches_per_layer": launches, "device_status": plan.device_status()})
    entry["roofline"]["traffic"] = recorded_traffic(KERNELS[kernel][2])
    gate, up, down = first
    programs[0].submit_for_plan()
    ctx.stream.synchronize()
    h64, _ = oracle.mlp_f64(gate, up, down, HIDDEN, INTER, bits(x), threads=oracle.max_threads())
    h_bits = bits(programs[0].intermediate)
    y64_from_h = oracle.linear_f64(down[0], down[1], down[2], HIDDEN, INTER, h_bits, threads=oracle.max_threads())
    entry["parity"] = {"gate_up_rel_error_vs_fp64_oracle": rel_error(h_bits, h64),
                       "down_rel_error_vs_fp64_oracle": rel_error(bits(programs[0].out), y64_from_h), "bound": 2e-2}
    del programs, layers
    plan.close()
    return entry


def head_probe(ctx):
    """The BF16 vocabulary head (248320 x 5120, F32 activations and logits) at 8 token rows: 2.54 GB of weights per
    call, far more than L2. Bytes: weights once, activations and logits."""
    import oracle
    torch, host = ctx.torch, ctx.host
    rows, cols = 248320, 5120
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(31)
    weight = (torch.randn((rows, cols), device=ctx.device, generator=generator) * 0.02).to(torch.bfloat16)
    x = torch.randn((TOKENS, cols), device=ctx.device, generator=generator)
    head = host.Bf16Head.bind(ctx.stream, weight, x)
    for _ in range(3):
        head.submit()
    reps = 20
    ms = ctx.timed(head.submit, reps) / reps
    nbytes = rows * cols * 2 + TOKENS * cols * 4 + TOKENS * rows * 4
    entry = ctx.hbm_entry(nbytes, nbytes, ms)
    entry["workload"] = f"BF16 vocabulary head {rows} x {cols}, M={TOKENS}, F32 activations and logits"
    pick = np.sort(np.random.default_rng(8).choice(rows, size=512, replace=False))
    index = torch.from_numpy(pick).to(ctx.device)
    w_bits = weight[index].view(torch.int16).cpu().numpy().view(np.uint16)
    x_host = x.cpu().numpy()
    want = oracle.bf16_head_f64(w_bits, x_host)
    w64 = (w_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    scale = np.linalg.norm(w64, axis=1)[None, :] * np.linalg.norm(x_host.astype(np.float64), axis=1)[:, None]
    got = head.out[:, index].cpu().numpy().astype(np.float64)
    entry["parity"] = {"sampled_rows": int(pick.size), "max_error_over_norm_product_vs_fp64": float(np.max(np.abs(got - want) / scale)),
                       "bound": 1e-7}
    return entry


def prefill_probe(ctx):
    """Configuration 2 on one GPU: the M=4096 GEMMs through the tcgen05 path. Per shape: the mode that is
    accurate against the BF16-activation reference (three residual activation terms; the rate counts the
    useful 2*M*N*K once although three times as many MMAs run) and the plain W4A4 mode (one term), each
    with a roofline object and a parity check on sampled token rows outside the timed region."""
    import oracle
    from augur_v100_b200 import synth
    torch, host, abi = ctx.torch, ctx.host, ctx.abi
    out = {}
    plan = host.Plan(ctx.stream, host.gemm_plan_scratch_bytes())   # room to cut the leftover tiles along k
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(77)
    tokens, sampled, g_a = 4096, 16, 2.0 ** -8
    pick = np.sort(np.random.default_rng(7).choice(tokens, size=sampled, replace=False))
    threads = oracle.max_threads()
    for name, rows, cols in (("up_17408x5120", INTER, HIDDEN), ("down_5120x17408", HIDDEN, INTER)):
        codes, scales = device_planes(torch, generator, rows, cols, ctx.device)
        weight = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_TCGEN05, rows, cols, codes, scales,
                                                            synth.GLOBAL_SCALE)
        codes_host, scales_host = codes.cpu().numpy(), scales.cpu().numpy()
        del codes, scales
        x = torch.randn((tokens, cols), device=ctx.device, generator=generator).to(torch.bfloat16)
        x_bits = bits(x)[pick]
        y64_reference = oracle.linear_f64(codes_host, scales_host, synth.GLOBAL_SCALE, rows, cols, x_bits, threads=threads)
        flops = 2.0 * tokens * rows * cols
        shape = {"tokens": tokens, "rows": rows, "cols": cols}
        for key, terms in (("bf16_accurate", 3), ("w4a4", 1)):
            lin = host.Nvfp4Sm100PrefillLinear.bind(plan, weight, x, terms=terms, activation_global_scale=g_a)
            lin.submit_for_plan()
            ctx.stream.synchronize()
            status = plan.device_status()
            reps = 10
            ms_gemm = ctx.timed(lin.submit_gemm, reps) / reps
            ms_all = ctx.timed(lin.submit_for_plan, reps) / reps
            a_codes, a_scales = lin.staged_planes()
            a64 = oracle.act_dequant_f64(np.ascontiguousarray(a_codes[:, pick]), np.ascontiguousarray(a_scales[:, pick]),
                                         g_a, sampled, cols, terms)
            y64 = oracle.linear_f64_xf64(codes_host, scales_host, synth.GLOBAL_SCALE, rows, cols, a64, threads=threads)
            got = bits(lin.out[torch.from_numpy(pick).to(ctx.device)])
            tflops = flops / ms_all / 1e9
            shape[key] = {
                "activation_terms": terms, "ms": ms_all, "ms_gemm_only": ms_gemm, "tflops": tflops,
                "tflops_gemm_only": flops / ms_gemm / 1e9,
                "note": "useful 2*M*N*K per second, activation quantiser launch included" + (
                    "; the tensor pipe runs three MMAs per useful one" if terms == 3 else
                    "; plain W4A4: about 10 % rms from the BF16-activation reference, reported as the kernel's raw rate only"),
                "roofline": {"bound": "tensor", "achieved": tflops, "peak": DATASHEET_FP4_TFLOPS, "unit": "TFLOP/s",
                             "frac": tflops / DATASHEET_FP4_TFLOPS,
                             "peak_source": "datasheet dense NVFP4 (no measured FP4 peak on this pool)",
                             "frac_of_measured_bf16_peak": tflops / ctx.bf16_peak, "traffic": None},
                "parity": {"sampled_token_rows": sampled,
                           "rel_error_vs_fp64_oracle_same_staged_activations": rel_error(got, y64),
                           "max_error_over_rms_vs_bf16_activation_oracle": rms_error(got, y64_reference),
                           "bound": 2e-2},
                "device_status": status,
            }
            del lin
        out[name] = shape
        del weight, x
    plan.close()
    return out


def prefill_mlp_probe(ctx, tokens, chunk, terms):
    """Configuration 4 (long-prefill chunked MLP, tensor-parallel): whole-job TFLOP/s of the useful 2*M*N*K."""
    from augur_v100_b200 import synth, tp
    torch, host, abi = ctx.torch, ctx.host, ctx.abi
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(4321 + ctx.rank)
    shard = INTER // ctx.world
    gc, gs = device_planes(torch, generator, shard, HIDDEN, ctx.device)
    uc, us = device_planes(torch, generator, shard, HIDDEN, ctx.device)

    def interleave(gate_plane, up_plane):   # 16 gate rows, then the matching 16 up rows
        width = gate_plane.shape[1]
        return torch.stack([gate_plane.view(shard // 16, 16, width), up_plane.view(shard // 16, 16, width)], dim=1).reshape(2 * shard, width).contiguous()

    gate_up = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_TCGEN05, 2 * shard, HIDDEN, interleave(gc, uc),
                                                         interleave(gs, us), synth.GLOBAL_SCALE)
    gate_up.global_scale_b = synth.GLOBAL_SCALE
    dc, ds = device_planes(torch, generator, HIDDEN, shard, ctx.device)
    down = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_TCGEN05, HIDDEN, shard, dc, ds, synth.GLOBAL_SCALE)
    del gc, gs, uc, us, dc, ds
    plan = host.Plan(ctx.stream, host.gemm_plan_scratch_bytes())   # room to cut the leftover tiles along k
    x = torch.randn((tokens, HIDDEN), device=ctx.device, generator=generator).to(torch.bfloat16)
    block = tp.TensorParallelPrefillMlp(plan, gate_up, down, x, ctx.world, chunk_tokens=chunk, terms=terms,
                                        input_global_scale=2.0 ** -8, intermediate_global_scale=2.0 ** -6)
    block.submit()
    ctx.stream.synchronize()
    status = plan.device_status()
    reps = 3
    ms = ctx.timed(block.submit, reps) / reps
    flops = 2.0 * tokens * 3 * HIDDEN * INTER
    result = {"ms": ms, "tflops_useful": flops / ms / 1e9, "activation_terms": terms, "device_status": status,
              "finite": bool(torch.isfinite(block.out.float()).all())}
    del block
    plan.close()
    return result


SWEEP_LAYERS = 64
SWEEP_SHAPES = ((10240, 5120, "column"), (5120, 5120, "column"), (5120, 10240, "row"))   # rows, cols, how it shards


def norm_group_probe(ctx):
    """The GDN-input group at M=8: RMSNorm -> BF16 stage -> four projections of the same input (10240, 6144 and two
    48-row gates held as 64 weight rows), eight distinct groups in rotation (381 MB of weights, more than L2). Timed
    as the grouped program (norm stage + one grid for all members: 2 launches) and as the norm stage with one launch
    per projection (5 launches), which is how the members run when they are not grouped."""
    import oracle
    from augur_v100_b200 import synth
    torch, host, abi = ctx.torch, ctx.host, ctx.abi
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(4242)
    cols, count = HIDDEN, 8
    shapes, stored = [(10240, cols), (6144, cols), (64, cols), (64, cols)], [0, 0, 48, 48]
    plan = host.Plan(ctx.stream, 64 << 20)   # the group's members take their partial-sum regions side by side
    norm_weight = 1.0 + 0.1 * torch.randn((cols,), device=ctx.device, generator=generator)
    x = 3.0 * torch.randn((TOKENS, cols), device=ctx.device, generator=generator)
    grouped, separate, first = [], [], None
    for index in range(count):
        weights = []
        for rows, _ in shapes:
            codes, scales = device_planes(torch, generator, rows, cols, ctx.device)
            weights.append(host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, abi.LAYOUT_STREAM, rows, cols, codes, scales,
                                                                      synth.GLOBAL_SCALE))
            if index == 0 and rows == shapes[0][0]:
                first = (codes.cpu().numpy(), scales.cpu().numpy())
            del codes, scales
        grouped.append(host.Nvfp4Sm100NormGroupProgram.bind(plan, weights, x, norm_weight, stored_rows=stored))
        lone = host.Nvfp4Sm100NormGroupProgram.bind(plan, weights[:1], x, norm_weight)
        separate.append([lone] + [host.Nvfp4Sm100Projection.bind(plan, weight, lone.staged) for weight in weights[1:]])

    def run_grouped():
        for program in grouped:
            program.submit_for_plan()

    def run_separate():
        for members in separate:
            for member in members:
                member.submit_for_plan()

    weight_bytes = sum(rows * cols * 9 // 16 for rows, _ in shapes)
    rounds, results = 50, {}
    for label, body in (("grouped", run_grouped), ("one_launch_per_projection", run_separate)):
        for _ in range(3):
            body()
        launches_before = host.launch_count()
        ms = ctx.timed(body, rounds) / (rounds * count)
        results[label] = ctx.hbm_entry(weight_bytes, weight_bytes, ms)
        results[label]["launches"] = (host.launch_count() - launches_before) // (rounds * count)
    entry = results["grouped"]
    entry["one_launch_per_projection"] = results["one_launch_per_projection"]
    entry["workload"] = (f"norm group (GDN input): RMSNorm + BF16 stage + projections {[rows for rows, _ in shapes]} x {cols} "
                         f"(gates stored as 48 rows), M={TOKENS}; {count} distinct groups in rotation; bytes = weight bytes")
    grouped[0].submit_for_plan()
    ctx.stream.synchronize()
    y64 = oracle.linear_f64(first[0], first[1], synth.GLOBAL_SCALE, shapes[0][0], cols, bits(grouped[0].staged), threads=oracle.max_threads())
    entry["parity"] = {"first_member_rel_error_vs_fp64_oracle_same_staged_activations": rel_error(bits(grouped[0].outputs[0]), y64),
                       "bound": 2e-2}
    entry["device_status"] = plan.device_status()
    del grouped, separate
    plan.close()
    return entry


def sweep_probe(ctx, exchange, kernel):
    """Configuration 3: 64 layers, each the MLP block plus the projections 5120 -> 10240, 5120 -> 5120 and
    10240 -> 5120, all NVFP4 at M=8. With N > 1 the first two are column-parallel (row slices, outputs stay
    sharded), the third is row-parallel (k slices) with the all-reduce inside its launch, the MLP as in the
    headline. Reports the weight bytes streamed per verify pass, whole job."""
    from augur_v100_b200 import synth, tp
    torch, host, abi = ctx.torch, ctx.host, ctx.abi
    world = ctx.world
    generator = torch.Generator(device=ctx.device)
    generator.manual_seed(555 + ctx.rank)
    scratch = max([host.mlp_scratch_bytes(HIDDEN, INTER // world)] +
                  [2 * host.gemv_scratch_bytes(rows // world if how == "column" else rows,
                                               cols if how == "column" else cols // world, TOKENS) for rows, cols, how in SWEEP_SHAPES])
    plan = host.Plan(ctx.stream, scratch)
    x = torch.randn((TOKENS, HIDDEN), device=ctx.device, generator=generator).to(torch.bfloat16)
    wide = torch.randn((TOKENS, 10240 // world), device=ctx.device, generator=generator).to(torch.bfloat16)
    # On one GPU every launch of the pass is on the chosen kernel. (Mixed, the one-launch tensor-memory block between
    # attention-shaped launches of the mma.sync kernel measured 5.58 ms per pass against 5.48 all mma.sync and 5.31 all
    # tensor-memory: a launch starts its prologue under the tail of a neighbour of its own kind only.)
    tensor_memory = kernel == "tensor_memory" and world == 1
    mlp_layers, _ = build_mlp_layers(ctx, SWEEP_LAYERS, kernel="tensor_memory" if tensor_memory else "mma_sync")
    mlp_plan = plan
    if tensor_memory:
        mlp_plan = host.Plan(ctx.stream, max([host.mlp_tc_scratch_bytes(HIDDEN, INTER)] +
                                             [host.gemv_tc_scratch_bytes(rows, cols) for rows, cols, _ in SWEEP_SHAPES]))
    program_type = host.Nvfp4Sm100TcFfnProgram if tensor_memory else host.Nvfp4Sm100FfnProgram
    outs = [torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16, device=ctx.device) for _ in range(2)]
    programs = []
    for index, (gate_up, down) in enumerate(mlp_layers):
        layer = []
        for rows, cols, how in SWEEP_SHAPES:
            r, c = (rows // world, cols) if how == "column" else (rows, cols // world)
            codes, scales = device_planes(torch, generator, r, c, ctx.device)
            layout = abi.LAYOUT_TCGEN05 if tensor_memory else abi.LAYOUT_STREAM
            weight = host.Nvfp4Sm100Weight.repack_device_planes(ctx.stream, layout, r, c, codes, scales, synth.GLOBAL_SCALE)
            del codes, scales
            if tensor_memory:
                projection = host.Nvfp4Sm100TcProjection.bind(mlp_plan, weight, x if how == "column" else wide)
            else:
                projection = host.Nvfp4Sm100Projection.bind(plan, weight, x if how == "column" else wide)
            if how == "row" and exchange is not None:
                projection = tp.RowParallelLinear(projection, exchange)
            layer.append(projection)
        program = program_type.bind(mlp_plan, gate_up, down, x, out=outs[index % 2])
        if exchange is not None:
            program = tp.FusedExchangeProgram(program, exchange)
        layer.append(program)
        programs.append(layer)
    use_nccl = world > 1 and exchange is None

    def verify_pass():
        for layer in programs:
            for member in layer:
                member.submit_for_plan()
                if use_nccl and member is not layer[0] and member is not layer[1]:
                    ctx.dist.all_reduce(member.out)

    for _ in range(3):
        verify_pass()
    reps = 10
    launches_before = host.launch_count()
    ms = ctx.timed(verify_pass, reps) / reps
    launches = (host.launch_count() - launches_before) // reps
    weights_total = SWEEP_LAYERS * (3 * HIDDEN * INTER + sum(rows * cols for rows, cols, _ in SWEEP_SHAPES)) * 9 // 16
    entry = ctx.hbm_entry(weights_total // world, weights_total, ms)
    entry.update({"workload": f"config3: {SWEEP_LAYERS} layers x (MLP 5120 -> 2x17408 -> 5120, 5120 -> 10240, 5120 -> 5120, 10240 -> 5120), "
                              f"M={TOKENS}, tp{world}", "weight_bytes_per_verify_pass": weights_total,
                  "weight_bytes_per_gpu": weights_total // world, "launches_per_pass": launches,
                  "kernel": KERNELS["tensor_memory" if tensor_memory else "mma_sync"][0],
                  "device_status": plan.device_status() | mlp_plan.device_status()})
    del programs, mlp_layers
    if mlp_plan is not plan:
        mlp_plan.close()
    plan.close()
    return entry


def run_library(args):
    import torch
    import torch.distributed as dist

    from augur_v100_b200 import abi, host

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if INTER % (world * 128) != 0:
        raise SystemExit("intermediate size does not shard over this many GPUs")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        # NCCL writes its version / debug lines to stdout by default; stdout carries the one JSON line only
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)

    # Everything runs on one non-default stream, so that a pass can also be captured into a CUDA graph.
    side = torch.cuda.Stream(device)
    torch.cuda.set_stream(side)
    stream = host.Stream(local, side)
    ctx = Context(torch, dist, host, abi, device, stream, side, world, rank)
    # one GPU: the tensor-memory kernel, one launch per block; tensor-parallel: the mma.sync kernel, which carries the exchange
    kernel = args.small_token_kernel if world == 1 else "mma_sync"
    tensor_memory = kernel == "tensor_memory"
    program_type = host.Nvfp4Sm100TcFfnProgram if tensor_memory else host.Nvfp4Sm100FfnProgram
    layers, first_planes = build_mlp_layers(ctx, LAYERS, keep_first_planes=(world == 1 and rank == 0), kernel=kernel)
    plan = host.Plan(stream, host.mlp_tc_scratch_bytes(HIDDEN, INTER) if tensor_memory else host.mlp_scratch_bytes(HIDDEN, INTER // world))
    x_host = torch.randn((TOKENS, HIDDEN), dtype=torch.float32).mul_(8.0).to(torch.bfloat16).pin_memory()
    y_host = torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    outs = [torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16, device=device) for _ in range(2)]
    programs = [program_type.bind(plan, gate_up, down, x, out=outs[index % 2])
                for index, (gate_up, down) in enumerate(layers)]
    x1 = x[:1].contiguous()
    outs1 = [torch.empty((1, HIDDEN), dtype=torch.bfloat16, device=device) for _ in range(2)]
    programs_m1 = [program_type.bind(plan, gate_up, down, x1, out=outs1[index % 2])
                   for index, (gate_up, down) in enumerate(layers)]
    shard_programs = programs    # this rank's shard without any exchange (the same objects the exchange wraps)

    # With more than one rank the all-reduce is fused into the down launch (peer stores over NVLink);
    # --allreduce nccl, or a failed symmetric-memory set-up (reported in the line), uses NCCL instead.
    exchange, exchange_note = None, None
    if world > 1 and args.allreduce == "fused":
        from augur_v100_b200 import tp
        failure = None
        try:
            exchange = tp.ExchangeBuffers(HIDDEN, rank, world)
            fused_programs = [tp.FusedExchangeProgram(program, exchange) for program in programs]
            fused_m1 = [tp.FusedExchangeProgram(program, exchange) for program in programs_m1]
        except Exception as error:  # reported in the line, never hidden
            failure = repr(error)
        agree = torch.tensor([0 if failure else 1], device=device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 1:
            programs, programs_m1 = fused_programs, fused_m1
            exchange_note = ("fused into the down launch: f32 tiles stored to every rank over NVLink, flags, rank-order sum; "
                             "the launches count the exchange sequence on the device")
        else:
            exchange = None
            exchange_note = f"NCCL bf16 8x5120 per layer (fused exchange set-up failed on some rank: {failure})"
    elif world > 1:
        exchange_note = "NCCL bf16 8x5120 per layer"
    use_nccl = world > 1 and exchange is None

    def one_pass():
        for index, program in enumerate(programs):
            program.submit_for_plan()
            if use_nccl:
                dist.all_reduce(outs[index % 2])

    def step():
        for _ in range(PASSES):
            one_pass()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    launches_before = host.launch_count()
    sampler.mark_begin()
    total_ms = ctx.timed(step, args.steps)
    launches = host.launch_count() - launches_before

    # End to end: every pass copies its activations in from pinned host memory and its result back.
    def e2e_pass():
        x.copy_(x_host, non_blocking=True)
        one_pass()
        y_host.copy_(outs[(LAYERS - 1) % 2], non_blocking=True)
        side.synchronize()

    def e2e_step(body):
        def run():
            for _ in range(PASSES):
                body()
        return run

    for _ in range(3):
        e2e_pass()
    e2e_direct_ms = ctx.timed(e2e_step(e2e_pass), args.steps)
    e2e_ms, e2e_submission = e2e_direct_ms, "direct calls of the public API"
    graph_ok = torch.tensor([1], device=device)
    graph = None
    if not use_nccl:
        # The way a serving loop drives it (the reference captures its programs into CUDA graphs,
        # crates/augur-backend/src/cuda_qwen35_prefill_cublas/qpn.rs:507-515): the same calls captured once, replayed per pass.
        try:
            reference_bits = y_host.view(torch.int16).clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                x.copy_(x_host, non_blocking=True)
                one_pass()
                y_host.copy_(outs[(LAYERS - 1) % 2], non_blocking=True)
        except Exception as error:  # reported, never hidden
            graph_ok[0] = 0
            e2e_submission = f"direct calls of the public API (graph capture failed: {error!r})"
    else:
        graph_ok[0] = 0
    if world > 1:
        dist.all_reduce(graph_ok, op=dist.ReduceOp.MIN)
    if int(graph_ok.item()) == 1:
        def e2e_graph_pass():
            graph.replay()
            side.synchronize()

        y_host.zero_()
        for _ in range(3):
            e2e_graph_pass()
        same = torch.tensor([1 if torch.equal(y_host.view(torch.int16), reference_bits) else 0], device=device)
        if world > 1:
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if int(same.item()) == 1:
            e2e_ms = ctx.timed(e2e_step(e2e_graph_pass), args.steps)
            e2e_submission = "CUDA graph replay of one pass's public-API calls (H2D copy, all launches, D2H copy), one replay per pass"
        else:
            e2e_submission = "direct calls of the public API (graph replay and direct calls disagreed)"
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    status = plan.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status:#x}")

    extras = {}
    # M=1 on the same layers (decode), all ranks
    def m1_pass():
        for index, program in enumerate(programs_m1):
            program.submit_for_plan()
            if use_nccl:
                dist.all_reduce(outs1[index % 2])

    for _ in range(3):
        m1_pass()
    reps = 50
    m1_ms = ctx.timed(m1_pass, reps) / (reps * LAYERS)
    per_gpu_m1 = 3 * HIDDEN * (INTER // world) * 9 // 16 + 2 * HIDDEN * 2
    extras["config1_m1"] = ctx.hbm_entry(per_gpu_m1, layer_bytes(1), m1_ms)
    extras["config1_m1"]["workload"] = f"config1 at M=1: the same {LAYERS} layers, one token row; ms per layer"

    if world > 1:
        # What the exchange costs: the same layers with every rank running its shard alone (no exchange, outputs are
        # partial sums), beside the headline's time per layer, which has the exchange and the wait for the slowest rank.
        def shard_pass():
            for program in shard_programs:
                program.submit_for_plan()

        for _ in range(3):
            shard_pass()
        shard_ms = ctx.timed(shard_pass, reps) / (reps * LAYERS)
        with_exchange_ms = total_ms / (args.steps * PASSES * LAYERS)
        extras["config1_shard_without_exchange"] = {
            "ms_per_layer": shard_ms, "ms_per_layer_with_exchange": with_exchange_ms,
            "exchange_and_rank_skew_ms": with_exchange_ms - shard_ms, "device_status": plan.device_status(),
            "workload": f"config1, tp{world}: each rank's shard of the {LAYERS} layers with no exchange (max over ranks), "
                        "beside the headline's time per layer"}

    # parity of the timed programs against the CPU oracle (one GPU: the first layer, both token counts)
    parity = None
    if first_planes is not None:
        import oracle
        gate, up, down = first_planes
        parity = {"bound": 2e-2}
        for label, program, source in (("m8", programs[0], x), ("m1", programs_m1[0], x1)):
            program.submit_for_plan()
            stream.synchronize()
            h64, y64 = oracle.mlp_f64(gate, up, down, HIDDEN, INTER, bits(source), threads=oracle.max_threads())
            h_bits = bits(program.intermediate)
            y64_from_h = oracle.linear_f64(down[0], down[1], down[2], HIDDEN, INTER, h_bits, threads=oracle.max_threads())
            parity[label] = {"gate_up_rel_error_vs_fp64_oracle": rel_error(h_bits, h64),
                             "down_rel_error_vs_fp64_oracle": rel_error(bits(program.out), y64_from_h),
                             "block_max_error_over_rms": rms_error(bits(program.out), y64)}
        worst = max(max(v.values()) for k, v in parity.items() if k != "bound")
        if worst > 2e-2:
            raise SystemExit(f"parity of the timed MLP programs failed: {parity}")

    del programs, programs_m1, layers, graph
    torch.cuda.empty_cache()
    if not args.headline_only:
        try:
            extras["config3_sweep"] = sweep_probe(ctx, exchange, kernel)
        except Exception as error:  # reported, never hidden
            extras["config3_sweep"] = {"error": repr(error)}
        torch.cuda.empty_cache()
        try:
            extras["config4_prefill_mlp"] = {
                "workload": f"config4: chunked MLP, M={args.prefill_mlp_tokens} in chunks of 4096, hidden {HIDDEN}, intermediate {INTER}, "
                            f"tp{world}, per-chunk NCCL all-reduce overlapped with the next chunk",
                "bf16_accurate": prefill_mlp_probe(ctx, args.prefill_mlp_tokens, 4096, 3),
                "w4a4": prefill_mlp_probe(ctx, args.prefill_mlp_tokens, 4096, 1)}
        except Exception as error:
            extras["config4_prefill_mlp"] = {"error": repr(error)}
        torch.cuda.empty_cache()
        if world == 1:
            other = "mma_sync" if tensor_memory else "tensor_memory"
            for key, probe in (("config0", config0_probe), ("config1_other_kernel", lambda c: other_kernel_probe(c, other)),
                               ("config2_prefill", prefill_probe), ("head_bf16", head_probe), ("norm_group", norm_group_probe)):
                try:
                    extras[key] = probe(ctx)
                except Exception as error:
                    extras[key] = {"error": repr(error)}
                torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pass_bytes = LAYERS * layer_bytes()
    ms_per_step = total_ms / args.steps
    ms_per_pass = ms_per_step / PASSES
    value = pass_bytes / (ms_per_pass * 1e-3) / 1e9
    e2e_pass_ms = e2e_ms / args.steps / PASSES
    # Per GPU, per layer: the launches of the block (one, or two) read this rank's weight shard once.
    per_gpu_layer_bytes = 3 * HIDDEN * (INTER // world) * 9 // 16 + 2 * TOKENS * HIDDEN * 2
    launch_pair_ms = ms_per_pass / LAYERS
    kernel_name, launches_per_block, summary, dtype_line = KERNELS[kernel]
    achieved = per_gpu_layer_bytes / (launch_pair_ms * 1e-3) / 1e9
    line = {
        "metric": "nvfp4_linear_m8_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": dtype_line,
        "data": "synthetic",
        "config": {"workload": f"config1: NVFP4 MLP block (gate|up+SwiGLU, down), M={TOKENS}, hidden {HIDDEN}, "
                               f"intermediate {INTER}; one step = {PASSES} passes over {LAYERS} distinct layers",
                   "passes_per_step": PASSES, "layers_per_pass": LAYERS, "ms_per_pass": ms_per_pass,
                   "l2": f"inputs larger than L2: {LAYERS * 3 * HIDDEN * INTER * 9 // 16 // world} weight bytes per GPU per pass",
                   "parallelism": f"tp{world}" if world > 1 else "single", "all_reduce": exchange_note,
                   "small_token_kernel": f"{kernel_name}, {launches_per_block} launch(es) per block"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": ctx.hbm_peak, "unit": "GB/s", "frac": achieved / ctx.hbm_peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of the launches of one block (single GPU, full
                     # shapes) as recorded in the tracked ncu summary of this kernel
                     "traffic": recorded_traffic(summary) if world == 1 else None, "traffic_unit": "bytes per block (ncu)",
                     "peak_source": ctx.peak_source,
                     "kernel": f"{kernel_name} ({launches_per_block} launch(es) per block; with N>1 the interval also holds the all-reduce)",
                     "bytes_per_block": per_gpu_layer_bytes, "ms_per_block": launch_pair_ms},
        "e2e": {"value": pass_bytes / (e2e_pass_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": PASSES * TOKENS * HIDDEN * 2, "d2h_bytes_per_step": PASSES * TOKENS * HIDDEN * 2,
                "ms_per_step": e2e_ms / args.steps, "submission": e2e_submission,
                "direct_calls_value": pass_bytes / (e2e_direct_ms / args.steps / PASSES * 1e-3) / 1e9},
        "gpu_launches": launches, "clocks": clocks, "parity": parity,
    }
    line.update(extras)
    if world == 1:
        cpu_value, _, sample, threads = cpu_reference_run(1, 5, 20.0)
        line["cpu_baseline"] = {"value": cpu_value, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": sample + "; C restatement of the reference CPU path"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["library", "reference"], default="library")
    parser.add_argument("--headline-only", action="store_true",
                        help="time configuration 1 only (skips the other configurations' entries)")
    parser.add_argument("--prefill-mlp-tokens", type=int, default=32768)
    parser.add_argument("--small-token-kernel", choices=sorted(KERNELS), default="tensor_memory",
                        help="the kernel of the headline on one GPU (tensor-parallel runs use mma_sync, which carries the exchange)")
    parser.add_argument("--allreduce", choices=["fused", "nccl"], default="fused",
                        help="N>1: all-reduce inside the down launch over peer memory, or NCCL on the BF16 partials")
    parser.add_argument("--layers", type=int, default=LAYERS,
                        help="distinct layers streamed per pass (smaller values are for profiler captures only)")
    parser.add_argument("--passes", type=int, default=PASSES, help="passes over the layers per step")
    args = parser.parse_args()
    globals()["LAYERS"] = args.layers
    globals()["PASSES"] = args.passes
    if args.impl == "reference":
        run_reference(args)
    else:
        run_library(args)


if __name__ == "__main__":
    main()
