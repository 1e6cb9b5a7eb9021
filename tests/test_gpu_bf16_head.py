"""GPU parity of the BF16 vocabulary head (1..8 token rows, F32 activations, F32 logits) through the C ABI.

The reference's own test of this kernel (`f32_rw4_head_matches_mmvf8_and_f64_reference`, described in
docs/AUGUR_SHARED_HEAD_RW4_20261016.md) uses the full-vocabulary geometry with outlier activations, compares
sampled rows with an FP64 reference, checks the Top-20 sets of every token row, rejects misaligned input at
bind and verifies output guard bytes and zero hot allocations; the same checks are made here.
Bound: max |logit - fp64| / (||w_row|| * ||x_token||) <= 2e-7. Products are exact, as in the reference's FP32
kernel (which measures 4.8e-8 on this metric); the tensor core adds into its accumulator without rounding to
nearest, so every 64-k block is summed in registers of its own and added to the running sum with ordinary F32
additions (one long MMA chain measured 7.6e-7; the reference's discarded FP16 tensor-core variant 4.9e-7).
"""
from ctypes import byref

import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    yield {"torch": torch, "host": host, "stream": stream, "device": torch.device("cuda", 0)}
    stream.close()


def _normalised_error(got, want, w64, x64):
    scale = np.linalg.norm(w64, axis=1)[None, :] * np.linalg.norm(x64, axis=1)[:, None]
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(scale, 1e-300)))


@pytest.mark.parametrize("rows,cols,tokens", [(16, 64, 8), (48, 192, 3), (256, 5120, 8), (4096, 1024, 1), (1008, 2176, 5)])
def test_head_matches_fp64_reference(ctx, rows, cols, tokens):
    torch, host = ctx["torch"], ctx["host"]
    rng = np.random.default_rng(rows + cols + tokens)
    w = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32) * 0.05).to(ctx["device"]).to(torch.bfloat16)
    x_host = rng.standard_normal((tokens, cols)).astype(np.float32)
    x_host[0, ::97] *= 64.0                    # outlier activations
    x = torch.from_numpy(x_host).to(ctx["device"])
    guard = torch.full(((tokens + 2) * rows,), float("nan"), dtype=torch.float32, device=ctx["device"])
    out = guard[rows:(tokens + 1) * rows].view(tokens, rows)
    head = host.Bf16Head.bind(ctx["stream"], w, x, out)
    before = host.allocation_snapshot(), torch.cuda.memory_stats()["allocation.all.allocated"]
    head.submit()
    ctx["stream"].synchronize()
    assert (host.allocation_snapshot(), torch.cuda.memory_stats()["allocation.all.allocated"]) == before
    assert bool(torch.isnan(guard[:rows]).all()) and bool(torch.isnan(guard[(tokens + 1) * rows:]).all())
    w_bits = w.view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.bf16_head_f64(w_bits, x_host)
    w64 = (w_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert _normalised_error(out.cpu().numpy(), want, w64, x_host.astype(np.float64)) <= 2e-7


def test_head_full_vocabulary_geometry(ctx):
    # 248320 x 5120, 8 token rows with outliers: sampled rows against fp64, Top-20 sets of every token row
    torch, host = ctx["torch"], ctx["host"]
    rows, cols, tokens = 248320, 5120, 8
    generator = torch.Generator(device=ctx["device"])
    generator.manual_seed(5)
    w = (torch.randn((rows, cols), device=ctx["device"], generator=generator) * 0.02).to(torch.bfloat16)
    x = torch.randn((tokens, cols), device=ctx["device"], generator=generator)
    x[:, ::61] *= 32.0
    head = host.Bf16Head.bind(ctx["stream"], w, x)
    head.submit()
    ctx["stream"].synchronize()
    pick = np.sort(np.random.default_rng(6).choice(rows, size=2048, replace=False))
    pick[0], pick[-1] = 0, rows - 1
    index = torch.from_numpy(pick).to(ctx["device"])
    w_bits = w[index].view(torch.int16).cpu().numpy().view(np.uint16)
    x_host = x.cpu().numpy()
    want = oracle.bf16_head_f64(w_bits, x_host)
    w64 = (w_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    got = head.out[:, index].cpu().numpy()
    assert _normalised_error(got, want, w64, x_host.astype(np.float64)) <= 2e-7
    # Top-20 of every token row against an fp64 product on the device (torch: plumbing for the comparison only)
    full = (x.double() @ w.double().T)
    assert torch.equal(torch.topk(full, 20, dim=1).indices.sort(dim=1).values, torch.topk(head.out.double(), 20, dim=1).indices.sort(dim=1).values)


def test_head_rejections(ctx):
    torch, host = ctx["torch"], ctx["host"]
    rows, cols, tokens = 64, 128, 8
    w = torch.zeros((rows, cols), dtype=torch.bfloat16, device=ctx["device"])
    x = torch.zeros((tokens + 1, cols), dtype=torch.float32, device=ctx["device"])
    out = torch.zeros((tokens, rows), dtype=torch.float32, device=ctx["device"])
    lib, s = abi.lib(), ctx["stream"]

    def args(**changes):
        a = abi.header(abi.Bf16HeadArgs)
        a.weight, a.weight_len_bytes = w.data_ptr(), w.numel() * 2
        a.input, a.input_len_bytes = x.data_ptr(), tokens * cols * 4
        a.output, a.output_len_bytes = out.data_ptr(), out.numel() * 4
        a.rows, a.cols = rows, cols
        for key, value in changes.items():
            setattr(a, key, value)
        return a

    assert lib.augur_cuda_nvfp4_sm100_bf16_head_preflight_v1(s.ordinal, s.handle, byref(args())).status == abi.STATUS_OK
    launches = host.launch_count()
    for bad in (args(input=x.data_ptr() + 4), args(weight=w.data_ptr() + 2), args(rows=rows + 8), args(cols=cols + 32),
                args(input_len_bytes=9 * cols * 4), args(output_len_bytes=out.numel() * 4 - 4), args(output=x.data_ptr()),
                args(abi_version=2), args(struct_size=72)):
        for entry in (lib.augur_cuda_nvfp4_sm100_bf16_head_preflight_v1, lib.augur_cuda_nvfp4_sm100_bf16_head_prevalidated_submit_v1):
            assert entry(s.ordinal, s.handle, byref(bad)).status in (abi.STATUS_INVALID_ARGUMENT, abi.STATUS_ABI_VERSION_MISMATCH)
    assert host.launch_count() == launches
