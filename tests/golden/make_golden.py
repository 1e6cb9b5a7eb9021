"""Writes tests/golden/nvfp4_golden.npz: small seeded inputs with the CPU oracle's outputs.

The reference's own implementation of this path is Rust and cannot be run in the build
image, so these vectors come from the C restatement in oracle/ AFTER it has been pinned to
the reference's known-answer tests (tests/test_oracle_kat.py). Re-run with
    python tests/golden/make_golden.py
and commit the result whenever the oracle changes; tests/test_golden_cpu.py fails if the
committed file and the oracle ever disagree.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from augur_v100_b200 import synth  # noqa: E402


def build():
    out = {}
    # linear: 96 x 384 weight, 8 tokens
    rows, cols, tokens = 96, 384, 8
    codes, scales, glob = synth.make_weight(0, 90, "linear.w", rows, cols)
    x = synth.make_activation(0, 90, "linear.x", tokens, cols)
    y_bits, y_f32 = oracle.linear_bf16(codes, scales, glob, rows, cols, x, want_f32=True)
    out.update({"lin_codes": codes, "lin_scales": scales, "lin_global": np.float32(glob), "lin_x": x,
                "lin_dequant_bits": oracle.dequant_planes_f32(codes, scales, glob, rows, cols).view(np.uint32),
                "lin_y_bf16": y_bits, "lin_y_f32_bits": y_f32.view(np.uint32),
                "lin_y_f64": oracle.linear_f64(codes, scales, glob, rows, cols, x)})
    # the reference's own 2 x 64 case (crates/augur-reference/tests/m46_fp4.rs:37-50)
    act = ((np.arange(64, dtype=np.float32) - np.float32(31.0)) / np.float32(17.0)).astype(np.float32)
    blocks = oracle.make_blocks([[(0x5C + i) & 0xFF] * 8 for i in range(8)], [0x30 + i for i in range(8)], [0.125] * 8)
    out["m46_expected_bits"] = oracle.qmatvec_nvfp4_f32_ref(blocks, 2, 64, act).view(np.uint32)
    # MLP: hidden 128, intermediate 256, 8 tokens
    hidden, inter = 128, 256
    gate = synth.make_weight(0, 91, "mlp.gate", inter, hidden)
    up = synth.make_weight(0, 91, "mlp.up", inter, hidden)
    down = synth.make_weight(0, 91, "mlp.down", hidden, inter)
    xm = synth.f32_to_bf16_bits(np.random.default_rng(91).standard_normal((tokens, hidden)).astype(np.float32) * 8)
    h_bits, ym_bits = oracle.mlp_bf16(gate, up, down, hidden, inter, xm)
    h64, y64 = oracle.mlp_f64(gate, up, down, hidden, inter, xm)
    for name, (c, s, _) in (("gate", gate), ("up", up), ("down", down)):
        out[f"mlp_{name}_codes"], out[f"mlp_{name}_scales"] = c, s
    out.update({"mlp_x": xm, "mlp_h_bf16": h_bits, "mlp_y_bf16": ym_bits, "mlp_h_f64": h64, "mlp_y_f64": y64})
    # activation quantiser: 128 tokens x 64 columns, 2 residual terms
    xa = synth.make_activation(0, 92, "quant.x", 128, 64)
    qc, qs = oracle.act_quant(xa, 128, 64, 2.0 ** -8, 2)
    out.update({"quant_x": xa, "quant_codes": qc, "quant_scales": qs})
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nvfp4_golden.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
