"""Checkpoint-format adapters end to end: planes of either scale convention -> device repack -> values."""
import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, checkpoint as ck

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import torch
    from augur_v100_b200 import host
    torch.cuda.set_device(0)
    stream = host.Stream(0)
    yield {"host": host, "stream": stream}
    stream.close()


@pytest.mark.parametrize("kind,scalar", [("compressed-tensors", 3.0), ("compressed-tensors", 448.0), ("modelopt", 0.37),
                                         ("modelopt-w4a16", 1.0 / 448.0)])
@pytest.mark.parametrize("layout", [abi.LAYOUT_STREAM, abi.LAYOUT_TCGEN05])
def test_checkpoint_planes_dequantise_to_the_reference_values(ctx, kind, scalar, layout):
    host = ctx["host"]
    rows, cols = 128, 320 if layout == abi.LAYOUT_TCGEN05 else 384
    rng = np.random.default_rng(11)
    packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(0, 127, size=(rows, cols // 16), dtype=np.uint8)
    if kind == "compressed-tensors":
        m = ck.CheckpointNvfp4Matrix.from_compressed_tensors(packed, scales, scalar, 2.0)
    else:
        m = ck.CheckpointNvfp4Matrix.from_modelopt(packed, scales, scalar, 2.0 if kind == "modelopt" else None)
    codes, block_scales, global_scale = m.planes()
    weight = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], layout, rows, cols, codes, block_scales, global_scale)
    got = weight.dequant_f32().cpu().numpy()
    # bit-exact against the reference's two-rounding f32 decode with the converted scalar ...
    want = oracle.dequant_planes_f32(codes, block_scales, global_scale, rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # ... and within f32 rounding of the format's own f64 statement (divide or multiply)
    e2m1 = np.array([oracle.decode_e2m1(c) for c in range(16)], dtype=np.float64)
    e4m3 = np.array([oracle.decode_e4m3fn(b) for b in range(127)], dtype=np.float64)
    values = np.stack([packed & 15, packed >> 4], axis=-1).reshape(rows, cols)
    exact = m.scale.apply_f64(e2m1[values] * np.repeat(e4m3[scales], 16, axis=1))
    assert np.all(np.abs(got.astype(np.float64) - exact) <= 3 * 2.0 ** -24 * np.abs(exact))


def test_ggml36_import_feeds_the_same_weight(ctx):
    host = ctx["host"]
    rows, cols = 64, 256
    rng = np.random.default_rng(12)
    packed = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(0, 127, size=(rows, cols // 16), dtype=np.uint8)
    direct = ck.CheckpointNvfp4Matrix.from_modelopt(packed, scales, 0.5, 1.0)
    imported = ck.CheckpointNvfp4Matrix.from_ggml36(rows, cols, direct.to_ggml36(), direct.scale)
    a = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, *direct.planes())
    b = host.Nvfp4Sm100Weight.upload_checkpoint_nvfp4(ctx["stream"], abi.LAYOUT_STREAM, rows, cols, *imported.planes())
    assert np.array_equal(a.dequant_f32().cpu().numpy().view(np.uint32), b.dequant_f32().cpu().numpy().view(np.uint32))
