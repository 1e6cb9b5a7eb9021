"""CPU-side checks of the C ABI: exports, struct sizes, host repack, descriptor rejection.

None of these touches a GPU: they exercise the checks that run before any CUDA call.
"""
import ctypes
import re
from ctypes import byref, c_void_p
from pathlib import Path

import numpy as np
import pytest

import oracle
from augur_v100_b200 import abi, host, synth

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "augur_cuda_nvfp4_sm100.h").read_text()
    declared = set(re.findall(r"AUGUR_CUDA_CALL\s+(augur_cuda_nvfp4_sm100_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(abi.EXPORTS), declared ^ set(abi.EXPORTS)
    raw = ctypes.CDLL(str(abi.library_path()))
    for name in declared:
        assert getattr(raw, name) is not None
    lib = abi.lib()
    assert lib.augur_cuda_nvfp4_sm100_abi_version() == 1
    assert lib.augur_cuda_nvfp4_sm100_build_capability_v1() == 100


def test_struct_sizes_match_the_static_asserts():
    assert ctypes.sizeof(abi.RepackArgs) == 104
    assert ctypes.sizeof(abi.DequantArgs) == 80
    assert ctypes.sizeof(abi.GemvArgs) == 88
    assert ctypes.sizeof(abi.MlpArgs) == 184
    assert ctypes.sizeof(abi.MlpTpArgs) == 272
    assert ctypes.sizeof(abi.NormGroupArgs) == 472
    assert ctypes.sizeof(abi.ActQuantArgs) == 56
    assert ctypes.sizeof(abi.GemmArgs) == 80
    assert ctypes.sizeof(abi.GemmSwigluArgs) == 88
    assert ctypes.sizeof(abi.GemmSwigluQuantArgs) == 112
    assert ctypes.sizeof(abi.Result) == 8


@pytest.mark.parametrize("layout,rows,cols", [
    (abi.LAYOUT_STREAM, 64, 256), (abi.LAYOUT_STREAM, 32, 128), (abi.LAYOUT_STREAM_PAIR, 48, 384),
    (abi.LAYOUT_TCGEN05, 128, 256), (abi.LAYOUT_TCGEN05, 200, 192)])
def test_host_repack_is_a_lossless_permutation(layout, rows, cols):
    # permutation generators in the style of crates/augur-model-qwen35/src/checkpoint_quant.rs:349-372
    idx = np.arange(rows * cols // 2)
    codes = ((idx * 73 + idx // 17 + 11) % 256).astype(np.uint8).reshape(rows, cols // 2)
    sidx = np.arange(rows * cols // 16)
    scales = (sidx % 127).astype(np.uint8).reshape(rows, cols // 16)
    pair = layout == abi.LAYOUT_STREAM_PAIR
    codes_b = ((idx * 31 + 5) % 256).astype(np.uint8).reshape(rows, cols // 2) if pair else None
    scales_b = ((sidx * 7 + 3) % 127).astype(np.uint8).reshape(rows, cols // 16) if pair else None
    packed = host.repack_host(layout, rows, cols, codes, scales, codes_b, scales_b)
    assert packed.size == host.repack_extent(layout, rows, cols)
    back = host.unpack_host(layout, rows, cols, packed)
    assert np.array_equal(back[0], codes) and np.array_equal(back[1], scales)
    if pair:
        assert np.array_equal(back[2], codes_b) and np.array_equal(back[3], scales_b)
    if layout != abi.LAYOUT_TCGEN05:
        # a pure bit permutation: same size, same number of set bits, nothing padded
        source = np.concatenate([a.reshape(-1) for a in (codes, scales, codes_b, scales_b) if a is not None])
        assert packed.size == source.size
        assert int(np.unpackbits(packed).sum()) == int(np.unpackbits(source).sum())


WHERE = [(15, 8, 7, 6), (12, 5, 4, 3), (9, 2, 1, 0), (11, 10, 14, 13)]   # (sign, e1, e0, m) per fragment register


def _pack_word(source_bytes):
    word = 0
    for j, byte in enumerate(source_bytes):
        for half in range(2):
            code = (int(byte) >> (4 * half)) & 15
            for bit, at in zip((3, 2, 1, 0), WHERE[j]):
                word |= ((code >> bit) & 1) << (at + 16 * half)
    return word


def test_stream_layout_fragment_order():
    # one block: lane (g, t4), word j holds source bytes (row g + 8*(b&1), byte column 8*kstep + 4*(b>>1) + t4), b = 0..3,
    # bit-permuted so that the kernel's shift/mask/multiply extractions yield e2m1 * 2^-126 as BF16 pairs
    rows, cols = 32, 128
    rng = np.random.default_rng(0)
    tag = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scales = (np.arange(rows * cols // 16) % 127).astype(np.uint8).reshape(rows, cols // 16)
    packed = host.repack_host(abi.LAYOUT_STREAM, rows, cols, tag, scales)
    words = packed[:2048].view(np.uint32)
    e2m1 = oracle.E2M1_VALUES.astype(np.float64)
    mask = 0x81C081C0
    for t in range(2):
        for q in range(2):
            for lane in (0, 5, 31):
                for j in range(4):
                    g, t4 = lane >> 2, lane & 3
                    src = [tag[t * 16 + g + (b & 1) * 8, (q * 4 + j) * 8 + (b >> 1) * 4 + t4] for b in range(4)]
                    w = int(words[((t * 2 + q) * 32 + lane) * 4 + j])
                    assert w == _pack_word(src)
                    regs = [w & mask, (w << 3) & mask & 0xFFFFFFFF, (w << 6) & mask & 0xFFFFFFFF,
                            ((((w >> 10) & 0x001B001B) * 0x4108) & 0xFFFFFFFF) & mask]
                    for b in range(4):
                        for half in range(2):
                            bits = (regs[b] >> (16 * half)) & 0xFFFF
                            value = float(np.array([bits << 16], dtype=np.uint32).view(np.float32)[0]) * 2.0 ** 126
                            code = (int(src[b]) >> (4 * half)) & 15
                            assert value == e2m1[code], (t, q, lane, j, b, half)
    # scales: tile t, row pair g: bytes 2*ks + hi
    for t in range(2):
        for g in range(8):
            for ks in range(8):
                for hi in range(2):
                    assert packed[2048 + (t * 8 + g) * 16 + ks * 2 + hi] == scales[t * 16 + g + 8 * hi, ks]


def test_host_repack_rejects_bad_scales_and_shapes():
    rows, cols = 32, 128
    codes = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    scales[3, 2] = 0x7F  # NaN scale, as in crates/augur-reference/tests/m46_fp4.rs:52-59
    with pytest.raises(host.CudaRuntimeError) as err:
        host.repack_host(abi.LAYOUT_STREAM, rows, cols, codes, scales)
    assert err.value.status == abi.STATUS_INVALID_ARGUMENT
    scales[3, 2] = 0x80  # negative scale
    with pytest.raises(host.CudaRuntimeError):
        host.repack_host(abi.LAYOUT_STREAM, rows, cols, codes, scales)
    with pytest.raises(host.CudaRuntimeError):
        host.repack_extent(abi.LAYOUT_STREAM, 31, 128)      # rows not a multiple of 32
    with pytest.raises(host.CudaRuntimeError):
        host.repack_extent(abi.LAYOUT_STREAM, 32, 64)       # cols not a multiple of 128
    with pytest.raises(host.CudaRuntimeError):
        host.repack_extent(abi.LAYOUT_COMPACT, 32, 128)     # compact is not a repack target


def _fake_stream(ordinal=0):
    handle = c_void_p()
    res = abi.lib().augur_cuda_nvfp4_sm100_stream_adopt_v1(ordinal, c_void_p(0x1000), byref(handle))
    assert res.status == abi.STATUS_OK
    return handle


def _valid_repack_args():
    rows, cols = 64, 256
    args = abi.header(abi.RepackArgs)
    args.codes, args.codes_len_bytes = 0x10000000, rows * cols // 2
    args.scales, args.scales_len_bytes = 0x20000000, rows * cols // 16
    args.destination = 0x30000000
    args.destination_len_bytes = host.repack_extent(abi.LAYOUT_STREAM, rows, cols)
    args.rows, args.cols, args.layout = rows, cols, abi.LAYOUT_STREAM
    return args


REPACK_MUTATIONS = [
    ("abi+1", lambda a: setattr(a, "abi_version", 2), abi.STATUS_ABI_VERSION_MISMATCH),
    ("struct_size-1", lambda a: setattr(a, "struct_size", a.struct_size - 1), abi.STATUS_INVALID_ARGUMENT),
    ("reserved", lambda a: setattr(a, "reserved", 1), abi.STATUS_INVALID_ARGUMENT),
    ("codes null", lambda a: setattr(a, "codes", 0), abi.STATUS_INVALID_ARGUMENT),
    ("codes len-1", lambda a: setattr(a, "codes_len_bytes", a.codes_len_bytes - 1), abi.STATUS_INVALID_ARGUMENT),
    ("scales len+1", lambda a: setattr(a, "scales_len_bytes", a.scales_len_bytes + 1), abi.STATUS_INVALID_ARGUMENT),
    ("dest len-256", lambda a: setattr(a, "destination_len_bytes", a.destination_len_bytes - 256), abi.STATUS_INVALID_ARGUMENT),
    ("dest misaligned", lambda a: setattr(a, "destination", a.destination + 16), abi.STATUS_INVALID_ARGUMENT),
    ("codes misaligned", lambda a: setattr(a, "codes", a.codes + 4), abi.STATUS_INVALID_ARGUMENT),
    ("alias dest=codes", lambda a: setattr(a, "destination", a.codes), abi.STATUS_INVALID_ARGUMENT),
    ("alias scales in codes", lambda a: setattr(a, "scales", a.codes + 64), abi.STATUS_INVALID_ARGUMENT),
    ("rows 0", lambda a: setattr(a, "rows", 0), abi.STATUS_INVALID_ARGUMENT),
    ("rows odd", lambda a: setattr(a, "rows", 63), abi.STATUS_INVALID_ARGUMENT),
    ("cols 64", lambda a: setattr(a, "cols", 64), abi.STATUS_INVALID_ARGUMENT),
    ("layout compact", lambda a: setattr(a, "layout", abi.LAYOUT_COMPACT), abi.STATUS_INVALID_ARGUMENT),
    ("layout 9", lambda a: setattr(a, "layout", 9), abi.STATUS_INVALID_ARGUMENT),
    ("stray codes_b", lambda a: setattr(a, "codes_b", 0x40000000), abi.STATUS_INVALID_ARGUMENT),
    ("overflow address", lambda a: setattr(a, "codes", 2 ** 64 - 16), abi.STATUS_INVALID_ARGUMENT),
]


@pytest.mark.parametrize("name,mutate,expected", REPACK_MUTATIONS, ids=[m[0] for m in REPACK_MUTATIONS])
def test_descriptor_mutations_are_rejected_before_any_cuda_call(name, mutate, expected):
    # crates/augur-backend/src/cuda_nvfp4_sm70.rs:579-610: each single-field mutation must fail
    # both preflight and submit.
    lib = abi.lib()
    stream = _fake_stream()
    args = _valid_repack_args()
    mutate(args)
    for fn in (lib.augur_cuda_nvfp4_sm100_repack_preflight_v1, lib.augur_cuda_nvfp4_sm100_repack_prevalidated_submit_v1):
        res = fn(0, stream, byref(args))
        assert res.status == expected, (name, res.status)
    lib.augur_cuda_nvfp4_sm100_stream_destroy_v1(stream)


def test_null_and_foreign_handles_are_rejected():
    # crates/augur-backend/src/cuda_nvfp4_sm70.rs:508-524,563,626-634
    lib = abi.lib()
    stream = _fake_stream(0)
    args = _valid_repack_args()
    assert lib.augur_cuda_nvfp4_sm100_repack_preflight_v1(0, None, byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_repack_preflight_v1(0, stream, None).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_repack_preflight_v1(1, stream, byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_repack_preflight_v1(-1, stream, byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    gemv = abi.header(abi.GemvArgs)
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(0, stream, None, byref(gemv)).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(0, stream, None, byref(gemv)).status == abi.STATUS_INVALID_ARGUMENT
    mlp = abi.header(abi.MlpArgs)
    assert lib.augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1(0, stream, None, byref(mlp)).status == abi.STATUS_INVALID_ARGUMENT
    gemm = abi.header(abi.GemmArgs)
    assert lib.augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(0, stream, None, byref(gemm)).status == abi.STATUS_INVALID_ARGUMENT
    quant = abi.header(abi.ActQuantArgs)
    assert lib.augur_cuda_nvfp4_sm100_act_quant_preflight_v1(0, stream, byref(quant)).status == abi.STATUS_INVALID_ARGUMENT
    out = ctypes.c_void_p()
    assert lib.augur_cuda_nvfp4_sm100_plan_create_v1(0, None, 1024, byref(out)).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_plan_destroy_v1(None).status == abi.STATUS_INVALID_ARGUMENT
    lib.augur_cuda_nvfp4_sm100_stream_destroy_v1(stream)


def test_exchange_extent_and_tp_argument_checks():
    lib = abi.lib()
    out = ctypes.c_uint64()
    # [2 parities][world][groups] tiles of 256 {value, flag} pairs, then 256 bytes for the device-side sequence counter
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(5120, 8, ctypes.byref(out)).status == abi.STATUS_OK
    assert out.value == 2 * 8 * 160 * 2048 + 256
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(64, 2, ctypes.byref(out)).status == abi.STATUS_OK
    assert out.value == 2 * 2 * 2 * 2048 + 256
    for rows, world in ((5120, 0), (5120, 9), (5100, 2), (0, 2)):
        assert lib.augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(rows, world, ctypes.byref(out)).status == abi.STATUS_INVALID_ARGUMENT
    # without a stream and a plan nothing is looked at, on either entry
    args = abi.header(abi.MlpTpArgs)
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_preflight_v1(0, None, None, ctypes.byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1(0, None, None, ctypes.byref(args)).status == abi.STATUS_INVALID_ARGUMENT
    single = abi.header(abi.GemvTpArgs)
    assert ctypes.sizeof(abi.GemvTpArgs) == 184
    assert lib.augur_cuda_nvfp4_sm100_gemv_tp_preflight_v1(0, None, None, ctypes.byref(single)).status == abi.STATUS_INVALID_ARGUMENT
    assert lib.augur_cuda_nvfp4_sm100_gemv_tp_prevalidated_submit_v1(0, None, None, ctypes.byref(single)).status == abi.STATUS_INVALID_ARGUMENT


def test_scratch_extents():
    assert host.gemv_scratch_bytes(17408, 5120, 8) > 0
    assert host.gemv_scratch_bytes(5120, 17408, 8) > 0
    with pytest.raises(host.CudaRuntimeError):
        host.gemv_scratch_bytes(17408, 5120, 9)       # more than the small-token limit
    with pytest.raises(host.CudaRuntimeError):
        host.gemv_scratch_bytes(17408, 5100, 8)
    # prefill plans: the two counter regions, then one 256 x 256 f32 accumulator slot per CTA pair
    assert host.gemm_plan_scratch_bytes(148) == 2 * 65536 + 74 * 256 * 256 * 4
    assert host.gemm_plan_scratch_bytes(2) == 2 * 65536 + 256 * 256 * 4
    with pytest.raises(host.CudaRuntimeError):
        host.gemm_plan_scratch_bytes(5000)


def test_synthetic_generator_is_deterministic_and_in_range():
    c1, s1, g1 = synth.make_weight(0, 0, "w", 64, 256)
    c2, s2, g2 = synth.make_weight(0, 0, "w", 64, 256)
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2) and g1 == g2 == float(np.float32(1.0) / np.float32(448.0))
    assert s1.min() >= 1 and s1.max() <= 0x7E
    c3, _, _ = synth.make_weight(0, 0, "other", 64, 256)
    assert not np.array_equal(c1, c3)
    # the E4M3 encoder is round-to-nearest-even against the oracle's decoder
    table = np.array([oracle.decode_e4m3fn(c) for c in range(127)])
    assert np.array_equal(synth.e4m3_encode_rne(table), np.arange(127, dtype=np.uint8))
    mid = (table[8:-1] + table[9:]) / 2
    enc = synth.e4m3_encode_rne(mid)
    assert np.all(enc % 2 == 0)
