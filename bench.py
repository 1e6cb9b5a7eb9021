#!/usr/bin/env python
"""Benchmark of the NVFP4 quantized-linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (sm_100a kernels)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path, timed on host cores

Workload (configuration 1 of the benchmark definition): the 27B-class NVFP4 MLP block at the fixed 8-row
verify batch — gate|up 5120 -> 2x17408 fused with SiLU(gate)*up, then down
17408 -> 5120 — with synthetic weights of the benchmark's value distributions.
One step streams LAYERS distinct layers (2.4 GB of weights at N=1, far more than
L2), so every weight byte of a step comes from HBM. With N > 1 the block is
tensor-parallel: column-parallel gate|up, row-parallel down, one NCCL all-reduce
of the 8 x 5120 BF16 output per layer.

Prints one JSON line (rank 0). `value` is whole-job GB/s of algorithmic bytes
with inputs resident in HBM; `e2e` is the same through the public host API with
the activations copied from pinned host memory and the result read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

HIDDEN, INTER, TOKENS, LAYERS = 5120, 17408, 8, 16
ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def layer_bytes() -> int:
    """Algorithmic bytes of one MLP layer: every weight byte once + the input + the output (whole job)."""
    weights = 3 * HIDDEN * INTER * 9 // 16          # 0.5 B code + 1/16 B scale per element
    return weights + 2 * TOKENS * HIDDEN * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return float(data["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


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
# reference arm: the CPU path (C restatement of the reference's Rust, all host threads)
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = oracle.max_threads()
    # A step is one pass over a slice of the layer (the first `inter` intermediate columns of gate, up and
    # down: the same arithmetic per byte), sized so that warm-up plus timed steps fit the budget.
    probe_inter = 1024
    probe = min(cpu_layer_seconds(threads, 2, probe_inter))
    per_step = REFERENCE_BUDGET_SECONDS / max(args.warmup + args.steps, 1)
    inter = int(min(INTER, max(128, per_step / probe * probe_inter))) // 128 * 128
    times = cpu_layer_seconds(threads, args.warmup + args.steps, inter)[args.warmup:]
    seconds = sum(times) / len(times)
    value = mlp_bytes(inter) / seconds / 1e9
    sample = (f"one MLP layer (M=8, 5120 -> 2x{inter} -> 5120) per step"
              + ("" if inter == INTER else f": the first {inter} of {INTER} intermediate columns, to fit {args.warmup}+{args.steps} steps in "
                 f"{REFERENCE_BUDGET_SECONDS:.0f} s"))
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


def build_layers(torch, host, abi, stream, device, world, rank, layers):
    from augur_v100_b200 import synth
    generator = torch.Generator(device=device)
    generator.manual_seed(1234 + rank)
    inter_shard = INTER // world
    built = []
    for _ in range(layers):
        gc, gs = device_planes(torch, generator, inter_shard, HIDDEN, device)
        uc, us = device_planes(torch, generator, inter_shard, HIDDEN, device)
        gate_up = host.Nvfp4Sm100Weight.repack_device_planes(
            stream, abi.LAYOUT_STREAM_PAIR, inter_shard, HIDDEN, gc, gs, synth.GLOBAL_SCALE, uc, us, synth.GLOBAL_SCALE)
        dc, ds = device_planes(torch, generator, HIDDEN, inter_shard, device)
        down = host.Nvfp4Sm100Weight.repack_device_planes(
            stream, abi.LAYOUT_STREAM, HIDDEN, inter_shard, dc, ds, synth.GLOBAL_SCALE)
        built.append((gate_up, down))
        del gc, gs, uc, us, dc, ds
    return built


def prefill_probe(torch, host, abi, stream, device):
    """Config 2 on one GPU: M=4096 GEMMs through the tcgen05 path; returns TFLOP/s or an error string."""
    from augur_v100_b200 import synth
    out = {}
    try:
        plan = host.Plan(stream, host.gemm_plan_scratch_bytes())   # room to cut the leftover tiles along k
        generator = torch.Generator(device=device)
        generator.manual_seed(77)
        tokens = 4096
        for name, rows, cols in (("up_5120x17408", INTER, HIDDEN), ("down_17408x5120", HIDDEN, INTER)):
            codes, scales = device_planes(torch, generator, rows, cols, device)
            weight = host.Nvfp4Sm100Weight.repack_device_planes(stream, abi.LAYOUT_TCGEN05, rows, cols, codes, scales,
                                                                synth.GLOBAL_SCALE)
            x = torch.randn((tokens, cols), device=device, generator=generator).to(torch.bfloat16)
            lin = host.Nvfp4Sm100PrefillLinear.bind(plan, weight, x, terms=1, activation_global_scale=2.0 ** -8)
            lin.submit_for_plan()
            stream.synchronize()
            if plan.device_status() != 0:
                out[name] = {"error": f"device status {plan.device_status():#x}"}
                continue
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            start.record()
            for _ in range(reps):
                lin.submit_gemm()
            end.record()
            end.synchronize()
            ms = start.elapsed_time(end) / reps
            out[name] = {"ms": ms, "tflops": 2.0 * tokens * rows * cols / ms / 1e9, "tokens": tokens,
                         "activation_terms": 1, "finite": bool(torch.isfinite(lin.out.float()).all())}
            # Three residual activation terms bring the result within 2e-2 of the BF16-activation oracle;
            # the rate below counts the useful 2*M*N*K once, although three times as many MMAs run.
            del lin
            lin3 = host.Nvfp4Sm100PrefillLinear.bind(plan, weight, x, terms=3, activation_global_scale=2.0 ** -8)
            lin3.submit_for_plan()
            stream.synchronize()
            start.record()
            for _ in range(reps):
                lin3.submit_gemm()
            end.record()
            end.synchronize()
            ms3 = start.elapsed_time(end) / reps
            out[name]["three_terms"] = {"ms": ms3, "tflops_useful": 2.0 * tokens * rows * cols / ms3 / 1e9}
            del weight, lin3, x, codes, scales
        plan.close()
    except Exception as error:  # reported, never hidden
        out["error"] = repr(error)
    return out


def prefill_mlp_probe(torch, host, abi, stream, device, world, rank, tokens, chunk, terms):
    """Config 4 (long-prefill chunked MLP, tensor-parallel): returns whole-job TFLOP/s of useful 2*M*N*K."""
    import torch.distributed as dist

    from augur_v100_b200 import synth, tp
    generator = torch.Generator(device=device)
    generator.manual_seed(4321 + rank)
    shard = INTER // world
    gc, gs = device_planes(torch, generator, shard, HIDDEN, device)
    uc, us = device_planes(torch, generator, shard, HIDDEN, device)

    def interleave(gate_plane, up_plane):   # 16 gate rows, then the matching 16 up rows
        width = gate_plane.shape[1]
        return torch.stack([gate_plane.view(shard // 16, 16, width), up_plane.view(shard // 16, 16, width)], dim=1).reshape(2 * shard, width).contiguous()

    gate_up = host.Nvfp4Sm100Weight.repack_device_planes(stream, abi.LAYOUT_TCGEN05, 2 * shard, HIDDEN, interleave(gc, uc),
                                                         interleave(gs, us), synth.GLOBAL_SCALE)
    gate_up.global_scale_b = synth.GLOBAL_SCALE
    dc, ds = device_planes(torch, generator, HIDDEN, shard, device)
    down = host.Nvfp4Sm100Weight.repack_device_planes(stream, abi.LAYOUT_TCGEN05, HIDDEN, shard, dc, ds, synth.GLOBAL_SCALE)
    del gc, gs, uc, us, dc, ds
    plan = host.Plan(stream, host.gemm_plan_scratch_bytes())   # room to cut the leftover tiles along k
    x = torch.randn((tokens, HIDDEN), device=device, generator=generator).to(torch.bfloat16)
    block = tp.TensorParallelPrefillMlp(plan, gate_up, down, x, world, chunk_tokens=chunk, terms=terms,
                                        input_global_scale=2.0 ** -8, intermediate_global_scale=2.0 ** -6)
    block.submit()
    stream.synchronize()
    if plan.device_status() != 0:
        return {"error": f"device status {plan.device_status():#x}"}
    if world > 1:
        dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    start.record()
    for _ in range(reps):
        block.submit()
    end.record()
    end.synchronize()
    ms = torch.tensor([start.elapsed_time(end) / reps], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    flops = 2.0 * tokens * 3 * HIDDEN * INTER
    result = {"workload": f"chunked MLP, M={tokens} in chunks of {chunk}, hidden {HIDDEN}, intermediate {INTER}, tp{world}, "
                          "per-chunk NCCL all-reduce overlapped with the next chunk",
              "ms": ms, "tflops_useful": flops / ms / 1e9, "activation_terms": terms,
              "finite": bool(torch.isfinite(block.out.float()).all())}
    plan.close()
    return result


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
        dist.init_process_group("nccl", device_id=device)

    # Everything runs on one non-default stream, so that a step can also be captured into a CUDA graph.
    side = torch.cuda.Stream(device)
    torch.cuda.set_stream(side)
    stream = host.Stream(local, side)
    layers = build_layers(torch, host, abi, stream, device, world, rank, LAYERS)
    plan = host.Plan(stream, host.mlp_scratch_bytes(HIDDEN, INTER // world))
    x_host = torch.randn((TOKENS, HIDDEN), dtype=torch.float32).mul_(8.0).to(torch.bfloat16).pin_memory()
    y_host = torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    outs = [torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16, device=device) for _ in range(2)]
    programs = [host.Nvfp4Sm100FfnProgram.bind(plan, gate_up, down, x, out=outs[index % 2])
                for index, (gate_up, down) in enumerate(layers)]

    # With more than one rank the all-reduce is fused into the down launch (peer stores over NVLink);
    # --allreduce nccl, or a failed symmetric-memory set-up (reported in the line), uses NCCL instead.
    exchange_note = None
    if world > 1 and args.allreduce == "fused":
        from augur_v100_b200 import tp
        failure = None
        try:
            exchange = tp.ExchangeBuffers(HIDDEN, rank, world)
            fused_programs = [tp.FusedExchangeProgram(program, exchange) for program in programs]
        except Exception as error:  # reported in the line, never hidden
            failure = repr(error)
        agree = torch.tensor([0 if failure else 1], device=device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 1:
            programs = fused_programs
            exchange_note = "fused into the down launch: f32 tiles stored to every rank over NVLink, flags, rank-order sum"
        else:
            exchange_note = f"NCCL bf16 8x5120 per layer (fused exchange set-up failed on some rank: {failure})"
    elif world > 1:
        exchange_note = "NCCL bf16 8x5120 per layer"
    use_nccl = world > 1 and not (exchange_note or "").startswith("fused")

    def step():
        for index, program in enumerate(programs):
            program.submit_for_plan()
            if use_nccl:
                dist.all_reduce(outs[index % 2])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(body, steps):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            body()
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    launches_before = host.launch_count()
    sampler.mark_begin()
    total_ms = timed(step, args.steps)
    launches = host.launch_count() - launches_before

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        step()
        y_host.copy_(outs[(LAYERS - 1) % 2], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps)
    e2e_submission, e2e_direct_ms = "direct calls of the public API", None
    if world == 1:
        # The way a serving loop drives it (the reference captures its programs into CUDA graphs,
        # crates/augur-backend/src/cuda_qwen35_prefill_cublas/qpn.rs:507-515): the same calls captured once, replayed per step.
        try:
            reference_bits = y_host.view(torch.int16).clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                x.copy_(x_host, non_blocking=True)
                step()
                y_host.copy_(outs[(LAYERS - 1) % 2], non_blocking=True)

            def e2e_graph_step():
                graph.replay()
                side.synchronize()

            y_host.zero_()
            for _ in range(3):
                e2e_graph_step()
            if not torch.equal(y_host.view(torch.int16), reference_bits):
                raise RuntimeError("graph replay and direct calls disagree")
            graph_ms = timed(e2e_graph_step, args.steps)
            e2e_direct_ms, e2e_ms = e2e_ms, graph_ms
            e2e_submission = "CUDA graph replay of the step's public-API calls (H2D copy, all launches, D2H copy)"
        except Exception as error:  # reported, never hidden
            e2e_submission = f"direct calls of the public API (graph capture failed: {error!r})"
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    status = plan.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status:#x}")

    prefill_mlp = None
    if args.prefill_mlp:
        # every rank takes part (collectives inside); the decode layers are released first
        del programs, layers
        torch.cuda.empty_cache()
        prefill_mlp = {}
        for terms in (1, 3):
            prefill_mlp[f"terms_{terms}"] = prefill_mlp_probe(torch, host, abi, stream, device, world, rank,
                                                              args.prefill_mlp_tokens, 4096, terms)
        programs, layers = [], []

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    step_bytes = LAYERS * layer_bytes()
    ms_per_step = total_ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
    peak, peak_source = measured_peaks()
    # Per GPU, per layer: the two launches of the streaming kernel read this rank's weight shard once.
    per_gpu_layer_bytes = 3 * HIDDEN * (INTER // world) * 9 // 16 + 2 * TOKENS * HIDDEN * 2
    launch_pair_ms = ms_per_step / LAYERS
    achieved = per_gpu_layer_bytes / (launch_pair_ms * 1e-3) / 1e9
    line = {
        "metric": "nvfp4_linear_m8_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 x bf16 -> f32 (E2M1 codes as BF16 fragments on mma.sync, E4M3 block scales applied in f32)",
        "data": "synthetic",
        "config": {"workload": f"config1: NVFP4 MLP block (gate|up+SwiGLU, down), M={TOKENS}, hidden {HIDDEN}, "
                               f"intermediate {INTER}, {LAYERS} distinct layers per step",
                   "l2": f"inputs larger than L2: {LAYERS * 3 * HIDDEN * INTER * 9 // 16 // world} weight bytes per GPU per step",
                   "parallelism": f"tp{world}" if world > 1 else "single", "all_reduce": exchange_note},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one gate|up launch plus one down launch
                     # (single GPU, full shapes), from the ncu capture summarised under profiles/
                     "traffic": 155.05e6 if world == 1 else None, "traffic_unit": "bytes per launch pair (ncu)",
                     "peak_source": peak_source,
                     "kernel": "gemv_kernel (gate|up launch + down launch per layer; with N>1 the interval also holds the all-reduce)",
                     "bytes_per_launch_pair": per_gpu_layer_bytes, "ms_per_launch_pair": launch_pair_ms},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": TOKENS * HIDDEN * 2,
                "d2h_bytes_per_step": TOKENS * HIDDEN * 2, "ms_per_step": e2e_ms / args.steps,
                "submission": e2e_submission,
                "direct_calls_value": None if e2e_direct_ms is None else step_bytes / (e2e_direct_ms / args.steps * 1e-3) / 1e9},
        "gpu_launches": launches, "clocks": clocks,
    }
    if world == 1:
        import oracle
        threads = oracle.max_threads()
        seconds = min(cpu_layer_seconds(threads, 2))
        line["cpu_baseline"] = {"value": layer_bytes() / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": "one full MLP layer (M=8), best of 2, C restatement of the reference CPU path"}
        if not args.no_prefill:
            del programs, layers
            torch.cuda.empty_cache()
            line["prefill"] = prefill_probe(torch, host, abi, stream, device)
    if prefill_mlp is not None:
        line["prefill_mlp"] = prefill_mlp
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=1000)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["library", "reference"], default="library")
    parser.add_argument("--no-prefill", action="store_true", help="skip the M=4096 tcgen05 probe at N=1")
    parser.add_argument("--prefill-mlp", action="store_true",
                        help="also time the chunked tensor-parallel prefill MLP (reported under prefill_mlp)")
    parser.add_argument("--prefill-mlp-tokens", type=int, default=32768)
    parser.add_argument("--allreduce", choices=["fused", "nccl"], default="fused",
                        help="N>1: all-reduce inside the down launch over peer memory, or NCCL on the BF16 partials")
    parser.add_argument("--layers", type=int, default=LAYERS,
                        help="distinct layers streamed per step (smaller values are for profiler captures only)")
    args = parser.parse_args()
    globals()["LAYERS"] = args.layers
    if args.impl == "reference":
        run_reference(args)
    else:
        run_library(args)


if __name__ == "__main__":
    main()
