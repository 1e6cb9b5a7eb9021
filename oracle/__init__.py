"""CPU oracle for the NVFP4 linear path — TEST INFRASTRUCTURE ONLY.

Loads the plain-C restatement of the reference's CPU arithmetic
(``oracle/nvfp4_oracle.c``) through ctypes. Only the test-suite, the smoke
check and the benchmark's CPU-baseline legs may import this package; the
shipped library never does. Parity status: pinned against the reference's own
known-answer vectors (``tests/test_oracle_kat.py``).

There is no ``oracle/_ref``: the reference's implementation of this path is
Rust (crates augur-formats / augur-repack / augur-kernels / augur-reference)
and no Rust toolchain exists in the build image, so it cannot be compiled.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libnvfp4_oracle.so"

OK = 0
NON_FINITE_VALUE = 1
OUTPUT_TOO_SMALL = 2
BAD_WEIGHT_SHAPE = 3
BAD_ACTIVATION_LENGTH = 4
BAD_OUTPUT_LENGTH = 5
BAD_WEIGHT_BLOCK_COUNT = 6
BAD_WEIGHT = 7


class CompactBlock(ctypes.Structure):
    """Nvfp4CompactBlock (crates/augur-formats/src/fp4.rs:91-96)."""

    _fields_ = [
        ("qs", ctypes.c_uint8 * 8),
        ("scale_e4m3", ctypes.c_uint8),
        ("pad", ctypes.c_uint8 * 3),
        ("global_scale", ctypes.c_float),
    ]


class HotBlock(ctypes.Structure):
    """Nvfp4HotCpuBlock (crates/augur-kernel-api/src/hot/fp4_portable.rs:15-19)."""

    _fields_ = [("scale", ctypes.c_float), ("qs", ctypes.c_uint8 * 8)]


def build(force: bool = False) -> Path:
    """Compile the C oracle with gcc (no FMA contraction)."""
    source = _HERE / "nvfp4_oracle.c"
    header = _HERE / "nvfp4_oracle.h"
    stale = (
        force
        or not _LIB_PATH.exists()
        or _LIB_PATH.stat().st_mtime < max(source.stat().st_mtime, header.stat().st_mtime)
    )
    if stale:
        _LIB_PATH.parent.mkdir(exist_ok=True)
        compiler = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.run(
            [compiler, "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-std=c11", "-shared",
             "-o", str(_LIB_PATH), str(source), "-lm", "-lpthread"],
            check=True,
        )
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        handle = ctypes.CDLL(str(build()))
        handle.augur_oracle_decode_e2m1.restype = ctypes.c_float
        handle.augur_oracle_decode_e2m1.argtypes = [ctypes.c_uint8]
        handle.augur_oracle_decode_e4m3fn.argtypes = [ctypes.c_uint8, ctypes.POINTER(ctypes.c_float)]
        handle.augur_oracle_bf16_round.restype = ctypes.c_float
        handle.augur_oracle_bf16_round.argtypes = [ctypes.c_float]
        _lib = handle
    return _lib


def _p(array: np.ndarray, ctype):
    return array.ctypes.data_as(ctypes.POINTER(ctype))


def _u8(array) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=np.uint8)


def _u16(array) -> np.ndarray:
    return np.ascontiguousarray(array, dtype=np.uint16)


class OracleError(Exception):
    def __init__(self, code: int):
        super().__init__(f"oracle error {code}")
        self.code = code


def _check(code: int) -> None:
    if code != OK:
        raise OracleError(code)


def decode_e2m1(value: int) -> float:
    return float(lib().augur_oracle_decode_e2m1(value & 0xFF))


def decode_e4m3fn(value: int) -> float:
    out = ctypes.c_float()
    _check(lib().augur_oracle_decode_e4m3fn(value & 0xFF, ctypes.byref(out)))
    return float(out.value)


def bf16_round(value: float) -> float:
    return float(lib().augur_oracle_bf16_round(ctypes.c_float(value)))


def make_blocks(qs_list, scale_list, global_list):
    blocks = (CompactBlock * len(qs_list))()
    for index, (qs, scale, glob) in enumerate(zip(qs_list, scale_list, global_list)):
        for lane in range(8):
            blocks[index].qs[lane] = qs[lane]
        blocks[index].scale_e4m3 = scale
        blocks[index].global_scale = glob
    return blocks


def block_decode_ref(qs, scale: int, global_scale: float) -> np.ndarray:
    blocks = make_blocks([qs], [scale], [global_scale])
    out = np.zeros(16, dtype=np.float32)
    _check(lib().augur_oracle_nvfp4_block_decode_ref(blocks, _p(out, ctypes.c_float), ctypes.c_size_t(16)))
    return out


def qmatvec_nvfp4_f32_ref(blocks, rows: int, cols: int, activation: np.ndarray, out_len=None) -> np.ndarray:
    activation = np.ascontiguousarray(activation, dtype=np.float32)
    out = np.zeros(rows if out_len is None else out_len, dtype=np.float32)
    _check(lib().augur_oracle_qmatvec_nvfp4_f32_ref(
        blocks, ctypes.c_size_t(len(blocks)), ctypes.c_size_t(rows), ctypes.c_size_t(cols),
        _p(activation, ctypes.c_float), ctypes.c_size_t(activation.size),
        _p(out, ctypes.c_float), ctypes.c_size_t(out.size)))
    return out


def repack_nvfp4_tensor_cpu(blocks, rows: int, cols: int):
    hot = (HotBlock * len(blocks))()
    _check(lib().augur_oracle_repack_nvfp4_tensor_cpu(
        blocks, ctypes.c_size_t(len(blocks)), ctypes.c_size_t(rows), ctypes.c_size_t(cols), hot))
    return hot


def qmatvec_nvfp4_f32_cpu_portable(hot, rows: int, cols: int, activation: np.ndarray) -> np.ndarray:
    activation = np.ascontiguousarray(activation, dtype=np.float32)
    out = np.zeros(rows, dtype=np.float32)
    _check(lib().augur_oracle_qmatvec_nvfp4_f32_cpu_portable(
        hot, ctypes.c_size_t(len(hot)), ctypes.c_size_t(rows), ctypes.c_size_t(cols),
        _p(activation, ctypes.c_float), ctypes.c_size_t(activation.size),
        _p(out, ctypes.c_float), ctypes.c_size_t(out.size)))
    return out


def planes_to_blocks(codes, scales, global_scale: float, rows: int, cols: int):
    codes, scales = _u8(codes), _u8(scales)
    blocks = (CompactBlock * (rows * cols // 16))()
    _check(lib().augur_oracle_planes_to_blocks(
        _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(global_scale),
        ctypes.c_size_t(rows), ctypes.c_size_t(cols), blocks))
    return blocks


def dequant_planes_f32(codes, scales, global_scale: float, rows: int, cols: int) -> np.ndarray:
    codes, scales = _u8(codes), _u8(scales)
    out = np.zeros((rows, cols), dtype=np.float32)
    _check(lib().augur_oracle_dequant_planes_f32(
        _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(global_scale),
        ctypes.c_size_t(rows), ctypes.c_size_t(cols), _p(out, ctypes.c_float)))
    return out


def linear_bf16(codes, scales, global_scale: float, rows: int, cols: int, x_bf16_bits, threads: int = 1,
                want_f32: bool = False):
    """y[m][n] = bf16_round(sequential f32 sum); x and y are BF16 bit patterns (uint16)."""
    codes, scales, x = _u8(codes), _u8(scales), _u16(x_bf16_bits)
    tokens = x.size // cols
    y = np.zeros((tokens, rows), dtype=np.uint16)
    y32 = np.zeros((tokens, rows), dtype=np.float32) if want_f32 else None
    _check(lib().augur_oracle_linear_bf16(
        _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(global_scale),
        ctypes.c_size_t(rows), ctypes.c_size_t(cols), _p(x, ctypes.c_uint16), ctypes.c_size_t(tokens),
        _p(y, ctypes.c_uint16), _p(y32, ctypes.c_float) if want_f32 else None, ctypes.c_int(threads)))
    return (y, y32) if want_f32 else y


def linear_f64(codes, scales, global_scale: float, rows: int, cols: int, x_bf16_bits, threads: int = 1):
    codes, scales, x = _u8(codes), _u8(scales), _u16(x_bf16_bits)
    tokens = x.size // cols
    y = np.zeros((tokens, rows), dtype=np.float64)
    _check(lib().augur_oracle_linear_f64(
        _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(global_scale),
        ctypes.c_size_t(rows), ctypes.c_size_t(cols), _p(x, ctypes.c_uint16), ctypes.c_size_t(tokens),
        _p(y, ctypes.c_double), ctypes.c_int(threads)))
    return y


def linear_f64_xf64(codes, scales, global_scale: float, rows: int, cols: int, x_f64, threads: int = 1):
    codes, scales = _u8(codes), _u8(scales)
    x = np.ascontiguousarray(x_f64, dtype=np.float64)
    tokens = x.size // cols
    y = np.zeros((tokens, rows), dtype=np.float64)
    _check(lib().augur_oracle_linear_f64_xf64(
        _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(global_scale),
        ctypes.c_size_t(rows), ctypes.c_size_t(cols), _p(x, ctypes.c_double), ctypes.c_size_t(tokens),
        _p(y, ctypes.c_double), ctypes.c_int(threads)))
    return y


def _mlp_args(gate, up, down):
    args = []
    keep = []
    for codes, scales, glob in (gate, up, down):
        codes, scales = _u8(codes), _u8(scales)
        keep += [codes, scales]
        args += [_p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(glob)]
    return args, keep


def mlp_bf16(gate, up, down, hidden: int, intermediate: int, x_bf16_bits, threads: int = 1):
    """gate/up/down are (codes, scales, global) triples. Returns (h_bf16, y_bf16) bit patterns."""
    x = _u16(x_bf16_bits)
    tokens = x.size // hidden
    h = np.zeros((tokens, intermediate), dtype=np.uint16)
    y = np.zeros((tokens, hidden), dtype=np.uint16)
    args, _keep = _mlp_args(gate, up, down)
    _check(lib().augur_oracle_mlp_bf16(
        *args, ctypes.c_size_t(hidden), ctypes.c_size_t(intermediate), _p(x, ctypes.c_uint16),
        ctypes.c_size_t(tokens), _p(h, ctypes.c_uint16), _p(y, ctypes.c_uint16), ctypes.c_int(threads)))
    return h, y


def mlp_f64(gate, up, down, hidden: int, intermediate: int, x_bf16_bits, threads: int = 1):
    x = _u16(x_bf16_bits)
    tokens = x.size // hidden
    h = np.zeros((tokens, intermediate), dtype=np.float64)
    y = np.zeros((tokens, hidden), dtype=np.float64)
    args, _keep = _mlp_args(gate, up, down)
    _check(lib().augur_oracle_mlp_f64(
        *args, ctypes.c_size_t(hidden), ctypes.c_size_t(intermediate), _p(x, ctypes.c_uint16),
        ctypes.c_size_t(tokens), _p(h, ctypes.c_double), _p(y, ctypes.c_double), ctypes.c_int(threads)))
    return h, y


def act_quant(x_bf16_bits, tokens: int, cols: int, global_scale: float, terms: int = 1):
    x = _u16(x_bf16_bits)
    codes = np.zeros((terms, tokens, cols // 2), dtype=np.uint8)
    scales = np.zeros((terms, tokens, cols // 16), dtype=np.uint8)
    _check(lib().augur_oracle_act_quant(
        _p(x, ctypes.c_uint16), ctypes.c_size_t(tokens), ctypes.c_size_t(cols),
        ctypes.c_float(global_scale), ctypes.c_int(terms), _p(codes, ctypes.c_uint8),
        _p(scales, ctypes.c_uint8)))
    return codes, scales


def act_dequant_f64(codes, scales, global_scale: float, tokens: int, cols: int, terms: int = 1):
    codes, scales = _u8(codes), _u8(scales)
    out = np.zeros((tokens, cols), dtype=np.float64)
    _check(lib().augur_oracle_act_dequant_f64(
        _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), ctypes.c_float(global_scale),
        ctypes.c_size_t(tokens), ctypes.c_size_t(cols), ctypes.c_int(terms), _p(out, ctypes.c_double)))
    return out


def rmsnorm_stage(input_f32, weight_f32, epsilon: float, add_a=None, add_b=None):
    """[residual add] -> RMSNorm -> (input actually normalised, F32 output, BF16 staged bits)."""
    weight = np.ascontiguousarray(weight_f32, dtype=np.float32)
    residual = add_a is not None
    if residual:
        a, b = np.ascontiguousarray(add_a, dtype=np.float32), np.ascontiguousarray(add_b, dtype=np.float32)
        x = np.zeros_like(a)
    else:
        a = b = None
        x = np.array(input_f32, dtype=np.float32, order="C", copy=True)
    tokens, cols = x.shape
    out = np.zeros((tokens, cols), dtype=np.float32)
    staged = np.zeros((tokens, cols), dtype=np.uint16)
    fp = ctypes.POINTER(ctypes.c_float)
    _check(lib().augur_oracle_rmsnorm_stage(
        a.ctypes.data_as(fp) if residual else None, b.ctypes.data_as(fp) if residual else None,
        x.ctypes.data_as(fp), weight.ctypes.data_as(fp), ctypes.c_size_t(tokens), ctypes.c_size_t(cols),
        ctypes.c_float(epsilon), ctypes.c_int(1 if residual else 0), out.ctypes.data_as(fp),
        staged.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))))
    return x, out, staged


def bf16_head_f64(weight_bf16_bits, x_f32) -> np.ndarray:
    """logits[token][row] = sum_k w[row][k] * x[token][k] in fp64: the FP64 reference the shared-head GPU test of
    the reference compares sampled rows with (docs/AUGUR_SHARED_HEAD_RW4_20261016.md, "Configuration and checks";
    products of a BF16 weight and an F32 activation are exact in fp64, so only the summation rounds)."""
    w = (np.ascontiguousarray(weight_bf16_bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    return np.ascontiguousarray(x_f32, dtype=np.float32).astype(np.float64) @ w.T


def max_threads() -> int:
    return int(lib().augur_oracle_max_threads())


# ---- independent numpy restatement (cross-check of the C file) -------------

E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32)


def e4m3_table_numpy() -> np.ndarray:
    """All 256 E4M3FN values as f32 (NaN for 0x7f/0xff); fp4.rs:46-59."""
    value = np.arange(256)
    sign = np.where(value & 0x80, -1.0, 1.0).astype(np.float32)
    exponent = (value >> 3) & 0x0F
    mantissa = (value & 0x07).astype(np.float32)
    sub = np.float32(2.0 ** -6) * (mantissa / np.float32(8.0))
    normal = np.exp2(exponent.astype(np.float32) - 7).astype(np.float32) * (np.float32(1.0) + mantissa / np.float32(8.0))
    out = sign * np.where(exponent == 0, sub, normal).astype(np.float32)
    out[(exponent == 0x0F) & ((value & 7) == 7)] = np.nan
    return out.astype(np.float32)


def dequant_planes_numpy(codes, scales, global_scale: float, rows: int, cols: int) -> np.ndarray:
    """Vectorised two-rounding dequant: fl(e2m1 * fl(e4m3 * global)); fp4.rs:105-125."""
    codes = _u8(codes).reshape(rows, cols // 2)
    scales = _u8(scales).reshape(rows, cols // 16)
    nibbles = np.empty((rows, cols), dtype=np.uint8)
    nibbles[:, 0::2] = codes & 0x0F
    nibbles[:, 1::2] = codes >> 4
    scale = (e4m3_table_numpy()[scales] * np.float32(global_scale)).astype(np.float32)
    return (E2M1_VALUES[nibbles] * np.repeat(scale, 16, axis=1)).astype(np.float32)
