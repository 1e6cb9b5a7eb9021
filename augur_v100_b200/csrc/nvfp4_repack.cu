// Repack (compact planes -> hot layouts), its host twin and inverse, and the
// bit-exact f32 dequantiser used for verification.
#include <cuda_runtime.h>

#include <cmath>

#include <cstring>

#include "nvfp4_internal.h"
#include "nvfp4_layout.cuh"

namespace augur_sm100 {
namespace {

static_assert(sizeof(augur_cuda_nvfp4_sm100_repack_args_v1) == 104, "repack ABI");
static_assert(sizeof(augur_cuda_nvfp4_sm100_dequant_args_v1) == 80, "dequant ABI");

bool stream_shape_ok(uint32_t layout, uint32_t rows, uint32_t cols) {
    if (!rows || !cols || rows > INT_MAX || cols > INT_MAX) return false;
    if (static_cast<uint64_t>(rows) * cols > UINT32_MAX) return false;
    switch (layout) {
        case AUGUR_NVFP4_SM100_LAYOUT_COMPACT: return cols % 16 == 0;
        case AUGUR_NVFP4_SM100_LAYOUT_STREAM: return rows % 32 == 0 && cols % 128 == 0;
        case AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR: return rows % 16 == 0 && cols % 128 == 0;
        case AUGUR_NVFP4_SM100_LAYOUT_TCGEN05: return cols % 64 == 0;
        default: return false;
    }
}

uint64_t layout_extent(uint32_t layout, uint32_t rows, uint32_t cols) {
    switch (layout) {
        case AUGUR_NVFP4_SM100_LAYOUT_STREAM: return stream_extent_bytes(false, rows, cols);
        case AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR: return stream_extent_bytes(true, rows, cols);
        case AUGUR_NVFP4_SM100_LAYOUT_TCGEN05: return tcgen05_extent_bytes(rows, cols);
        default: return 0;
    }
}

// ---- device repack ----------------------------------------------------------------
// STREAM / STREAM_PAIR: one thread per destination word (coalesced writes, gathered reads).
__global__ void repack_stream_kernel(const uint8_t* __restrict__ codes_a, const uint8_t* __restrict__ scales_a,
                                     const uint8_t* __restrict__ codes_b, const uint8_t* __restrict__ scales_b,
                                     uint8_t* __restrict__ destination, uint32_t rows, uint32_t cols, bool pair) {
    const uint32_t kb_count = cols / kStreamBlockK;
    const uint64_t groups = pair ? rows / 16 : rows / 32;
    const uint64_t words = groups * kb_count * (kStreamBlockBytes / 4);
    const uint64_t index = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= words) return;
    const uint64_t block = index / (kStreamBlockBytes / 4);
    const uint32_t word = static_cast<uint32_t>(index % (kStreamBlockBytes / 4));
    const uint32_t group = static_cast<uint32_t>(block / kb_count);
    const uint32_t kb = static_cast<uint32_t>(block % kb_count);
    uint32_t value = 0;
    if (word < kStreamCodeBytes / 4) {
        const uint32_t j = word & 3, lane = (word >> 2) & 31, q = (word >> 7) & 1, t = word >> 8;
        const uint32_t g = lane >> 2, t4 = lane & 3;
        const uint32_t kstep = kb * 8 + q * 4 + j;
        const uint8_t* source = (pair && t) ? codes_b : codes_a;
        const uint32_t row0 = pair ? group * 16 : group * 32 + t * 16;
        uint32_t bytes[4];
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            const uint32_t row = row0 + g + (b & 1) * 8;
            const uint32_t column = kstep * 8 + (b >> 1) * 4 + t4;
            bytes[b] = source[static_cast<uint64_t>(row) * (cols / 2) + column];
        }
        value = stream_pack_word(bytes[0], bytes[1], bytes[2], bytes[3]);
    } else {
        // scale word sw of the block: tile t, quad-row g, k-steps 2p and 2p+1, each {row g, row g+8}
        const uint32_t sw = word - kStreamCodeBytes / 4;  // 0..63
        const uint32_t p = sw & 3, g = (sw >> 2) & 7, t = sw >> 5;
        const uint8_t* source = (pair && t) ? scales_b : scales_a;
        const uint32_t row0 = (pair ? group * 16 : group * 32 + t * 16) + g;
#pragma unroll
        for (uint32_t b = 0; b < 4; ++b) {
            const uint32_t row = row0 + (b & 1) * 8;
            const uint32_t sc = kb * 8 + p * 2 + (b >> 1);
            value |= static_cast<uint32_t>(source[static_cast<uint64_t>(row) * (cols / 16) + sc]) << (8 * b);
        }
    }
    reinterpret_cast<uint32_t*>(destination)[index] = value;
}

// TCGEN05: codes are copied through; one thread per destination scale word.
__global__ void repack_tcgen05_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                      uint8_t* __restrict__ destination, uint32_t rows, uint32_t cols) {
    const uint64_t code_words = tcgen05_codes_bytes(rows, cols) / 4;
    const uint64_t scale_words = tcgen05_scale_bytes(rows, cols) / 4;
    const uint64_t index = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index < code_words) {
        reinterpret_cast<uint32_t*>(destination)[index] = reinterpret_cast<const uint32_t*>(codes)[index];
        return;
    }
    const uint64_t sw = index - code_words;
    if (sw >= scale_words) return;
    // word sw of the scale region: atom = sw / 128; inside: (r % 32) * 4 + (r / 32) % 4
    const uint64_t atoms_per_row_block = cols / 64;
    const uint64_t atom = sw / 128;
    const uint32_t inner = static_cast<uint32_t>(sw % 128);
    const uint32_t row = static_cast<uint32_t>(atom / atoms_per_row_block) * 128 + (inner & 3) * 32 + (inner >> 2);
    const uint32_t sc0 = static_cast<uint32_t>(atom % atoms_per_row_block) * 4;
    uint32_t value = 0;
    if (row < rows) {
        value = *reinterpret_cast<const uint32_t*>(scales + static_cast<uint64_t>(row) * (cols / 16) + sc0);
    }
    reinterpret_cast<uint32_t*>(destination)[index] = value;
}

// ---- device dequant ------------------------------------------------------------------
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
    const uint32_t exponent = (byte >> 3) & 15, mantissa = byte & 7;
    float magnitude;
    if (exponent == 15 && mantissa == 7) {
        magnitude = __int_as_float(0x7fc00000);
    } else if (exponent == 0) {
        magnitude = static_cast<float>(mantissa) * 0x1p-9f;
    } else {
        magnitude = __uint_as_float(((exponent + 120) << 23) | (mantissa << 20));
    }
    return (byte & 0x80) ? -magnitude : magnitude;
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t nibble) {
    // code 8 decodes to +0.0, as the reference's table does.
    const uint32_t magnitude = nibble & 7;
    const float table[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    const float value = table[magnitude];
    return ((nibble & 8) && magnitude) ? -value : value;
}

// One thread per (row, 16-element group).
__global__ void dequant_kernel(const uint8_t* __restrict__ weight, const uint8_t* __restrict__ scales,
                               float* __restrict__ output, uint32_t rows, uint32_t cols, uint32_t layout,
                               float global_a, float global_b) {
    const uint32_t groups = cols / 16;
    const uint32_t matrices = layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR ? 2 : 1;
    const uint64_t total = static_cast<uint64_t>(matrices) * rows * groups;
    const uint64_t index = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const uint32_t m = static_cast<uint32_t>(index / (static_cast<uint64_t>(rows) * groups));
    const uint64_t rest = index % (static_cast<uint64_t>(rows) * groups);
    const uint32_t row = static_cast<uint32_t>(rest / groups), group = static_cast<uint32_t>(rest % groups);
    uint8_t code_bytes[8];
    uint32_t scale_byte;
    if (layout == AUGUR_NVFP4_SM100_LAYOUT_COMPACT) {
        const uint2 packed = *reinterpret_cast<const uint2*>(weight + static_cast<uint64_t>(row) * (cols / 2) + group * 8);
        memcpy(code_bytes, &packed, 8);
        scale_byte = scales[static_cast<uint64_t>(row) * groups + group];
    } else if (layout == AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) {
        const uint2 packed = *reinterpret_cast<const uint2*>(weight + static_cast<uint64_t>(row) * (cols / 2) + group * 8);
        memcpy(code_bytes, &packed, 8);
        scale_byte = weight[tcgen05_codes_bytes(rows, cols) + tcgen05_scale_offset(row, group, cols)];
    } else {
        const bool pair = layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR;
#pragma unroll
        for (uint32_t b = 0; b < 8; ++b) {
            const StreamCoord at = stream_code_coord(pair, m, row, group * 8 + b, cols);
            const uint32_t word = *reinterpret_cast<const uint32_t*>(weight + at.block * kStreamBlockBytes + at.offset);
            code_bytes[b] = static_cast<uint8_t>(stream_unpack_byte(word, at.slot));
        }
        const StreamCoord at = stream_scale_coord(pair, m, row, group, cols);
        scale_byte = weight[at.block * kStreamBlockBytes + at.offset];
    }
    // Two roundings, exactly as Nvfp4CompactBlock::decode_ref: fl(e4m3*global), then fl(e2m1*scale).
    const float scale = __fmul_rn(e4m3_to_f32(scale_byte), m ? global_b : global_a);
    float* out = output + (static_cast<uint64_t>(m) * rows + row) * cols + group * 16;
#pragma unroll
    for (uint32_t b = 0; b < 8; ++b) {
        float2 pair_out;
        pair_out.x = __fmul_rn(e2m1_to_f32(code_bytes[b] & 15u), scale);
        pair_out.y = __fmul_rn(e2m1_to_f32(code_bytes[b] >> 4), scale);
        *reinterpret_cast<float2*>(out + 2 * b) = pair_out;
    }
}

// ---- validation -------------------------------------------------------------------------
bool check_repack(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_repack_args_v1* a, bool full,
                  augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a) || a->reserved != 0) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (a->layout == AUGUR_NVFP4_SM100_LAYOUT_COMPACT || !stream_shape_ok(a->layout, a->rows, a->cols)) return false;
    const uint64_t elements = static_cast<uint64_t>(a->rows) * a->cols;
    const bool pair = a->layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR;
    if (a->codes_len_bytes != elements / 2 || a->scales_len_bytes != elements / 16) return false;
    if (a->destination_len_bytes != layout_extent(a->layout, a->rows, a->cols)) return false;
    Range r[5] = {{a->codes, a->codes_len_bytes, 16}, {a->scales, a->scales_len_bytes, 4},
                  {a->destination, a->destination_len_bytes, 256}, {}, {}};
    size_t count = 3;
    if (pair) {
        if (a->codes_b_len_bytes != elements / 2 || a->scales_b_len_bytes != elements / 16) return false;
        r[3] = {a->codes_b, a->codes_b_len_bytes, 16};
        r[4] = {a->scales_b, a->scales_b_len_bytes, 4};
        count = 5;
    } else if (a->codes_b || a->codes_b_len_bytes || a->scales_b || a->scales_b_len_bytes) {
        return false;
    }
    if (!all_disjoint(r, count)) return false;
    return !full || inspect_device_ranges(d, r, count, failure);
}

bool check_dequant(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_dequant_args_v1* a, bool full,
                   augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a) || a->reserved != 0) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!stream_shape_ok(a->layout, a->rows, a->cols) || !std::isfinite(a->global_scale)) return false;
    const uint64_t elements = static_cast<uint64_t>(a->rows) * a->cols;
    const bool pair = a->layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR;
    if (pair ? !std::isfinite(a->global_scale_b) : a->global_scale_b != 0.0f) return false;
    if (a->output_len_bytes != elements * 4 * (pair ? 2 : 1)) return false;
    Range r[3];
    size_t count = 2;
    if (a->layout == AUGUR_NVFP4_SM100_LAYOUT_COMPACT) {
        if (a->weight_len_bytes != elements / 2 || a->scales_len_bytes != elements / 16) return false;
        r[0] = {a->weight, a->weight_len_bytes, 8};
        r[1] = {a->output_f32, a->output_len_bytes, 8};
        r[2] = {a->scales, a->scales_len_bytes, 1};
        count = 3;
    } else {
        if (a->weight_len_bytes != layout_extent(a->layout, a->rows, a->cols) || a->scales || a->scales_len_bytes) {
            return false;
        }
        r[0] = {a->weight, a->weight_len_bytes, 16};
        r[1] = {a->output_f32, a->output_len_bytes, 8};
    }
    if (!all_disjoint(r, count)) return false;
    return !full || inspect_device_ranges(d, r, count, failure);
}

void launch_repack(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_repack_args_v1* a) {
    const auto* codes = reinterpret_cast<const uint8_t*>(a->codes);
    const auto* scales = reinterpret_cast<const uint8_t*>(a->scales);
    auto* destination = reinterpret_cast<uint8_t*>(a->destination);
    const uint64_t words = a->destination_len_bytes / 4;
    const uint32_t blocks = static_cast<uint32_t>((words + 255) / 256);
    if (a->layout == AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) {
        repack_tcgen05_kernel<<<blocks, 256, 0, s->stream>>>(codes, scales, destination, a->rows, a->cols);
    } else {
        repack_stream_kernel<<<blocks, 256, 0, s->stream>>>(
            codes, scales, reinterpret_cast<const uint8_t*>(a->codes_b),
            reinterpret_cast<const uint8_t*>(a->scales_b), destination, a->rows, a->cols,
            a->layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR);
    }
    count_launch();
}

void launch_dequant(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_dequant_args_v1* a) {
    const uint32_t matrices = a->layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR ? 2 : 1;
    const uint64_t total = static_cast<uint64_t>(matrices) * a->rows * (a->cols / 16);
    dequant_kernel<<<static_cast<uint32_t>((total + 255) / 256), 256, 0, s->stream>>>(
        reinterpret_cast<const uint8_t*>(a->weight), reinterpret_cast<const uint8_t*>(a->scales),
        reinterpret_cast<float*>(a->output_f32), a->rows, a->cols, a->layout, a->global_scale, a->global_scale_b);
    count_launch();
}

template <class Args, class Check, class Launch>
augur_cuda_result_v1 submit_entry(int32_t d, augur_cuda_stream_t s, const Args* a, Check check, Launch launch) {
    augur_cuda_result_v1 failure;
    if (!check(d, s, a, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    launch(s, a);
    return submitted();
}

}  // namespace
}  // namespace augur_sm100

using namespace augur_sm100;

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_extent_host_v1(
    uint32_t layout, uint32_t rows, uint32_t cols, uint64_t* out_bytes) {
    if (!out_bytes || layout == AUGUR_NVFP4_SM100_LAYOUT_COMPACT || !stream_shape_ok(layout, rows, cols)) {
        return invalid();
    }
    *out_bytes = layout_extent(layout, rows, cols);
    return ok();
}

// Host twin of the device repack: the same coordinate functions, applied source-first.
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_host_v1(
    uint32_t layout, uint32_t rows, uint32_t cols, const uint8_t* codes, const uint8_t* scales,
    const uint8_t* codes_b, const uint8_t* scales_b, uint8_t* destination, uint64_t destination_len_bytes) {
    if (layout == AUGUR_NVFP4_SM100_LAYOUT_COMPACT || !stream_shape_ok(layout, rows, cols) || !codes || !scales ||
        !destination || destination_len_bytes != layout_extent(layout, rows, cols)) {
        return invalid();
    }
    const bool pair = layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR;
    if (pair && (!codes_b || !scales_b)) return invalid();
    const uint32_t matrices = pair ? 2 : 1;
    // Block scales must be finite and non-negative, as the reference loader demands
    // (crates/augur-backend/src/cuda_qwen35_qpn.rs:67-69).
    for (uint32_t m = 0; m < matrices; ++m) {
        const uint8_t* plane = m ? scales_b : scales;
        for (uint64_t i = 0; i < static_cast<uint64_t>(rows) * (cols / 16); ++i) {
            if (plane[i] >= 127) return invalid();
        }
    }
    if (layout == AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) {
        const uint64_t code_bytes = tcgen05_codes_bytes(rows, cols);
        memcpy(destination, codes, code_bytes);
        memset(destination + code_bytes, 0, tcgen05_scale_bytes(rows, cols));
        for (uint32_t r = 0; r < rows; ++r) {
            for (uint32_t sc = 0; sc < cols / 16; ++sc) {
                destination[code_bytes + tcgen05_scale_offset(r, sc, cols)] = scales[static_cast<uint64_t>(r) * (cols / 16) + sc];
            }
        }
        return ok();
    }
    // Each destination word holds four source bytes, bit-permuted: gather them first.
    memset(destination, 0, destination_len_bytes);
    for (uint32_t m = 0; m < matrices; ++m) {
        const uint8_t* code_plane = m ? codes_b : codes;
        const uint8_t* scale_plane = m ? scales_b : scales;
        for (uint32_t r = 0; r < rows; ++r) {
            for (uint32_t c = 0; c < cols / 2; ++c) {
                const StreamCoord at = stream_code_coord(pair, m, r, c, cols);
                // staged as plain bytes in slot order; permuted word by word below
                destination[at.block * kStreamBlockBytes + at.offset + at.slot] = code_plane[static_cast<uint64_t>(r) * (cols / 2) + c];
            }
            for (uint32_t sc = 0; sc < cols / 16; ++sc) {
                const StreamCoord at = stream_scale_coord(pair, m, r, sc, cols);
                destination[at.block * kStreamBlockBytes + at.offset] = scale_plane[static_cast<uint64_t>(r) * (cols / 16) + sc];
            }
        }
    }
    for (uint64_t block = 0; block < destination_len_bytes / kStreamBlockBytes; ++block) {
        uint8_t* words = destination + block * kStreamBlockBytes;
        for (uint32_t w = 0; w < kStreamCodeBytes; w += 4) {
            const uint32_t packed = stream_pack_word(words[w], words[w + 1], words[w + 2], words[w + 3]);
            memcpy(words + w, &packed, 4);
        }
    }
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_unpack_host_v1(
    uint32_t layout, uint32_t rows, uint32_t cols, const uint8_t* source, uint64_t source_len_bytes,
    uint8_t* codes, uint8_t* scales, uint8_t* codes_b, uint8_t* scales_b) {
    if (layout == AUGUR_NVFP4_SM100_LAYOUT_COMPACT || !stream_shape_ok(layout, rows, cols) || !codes || !scales ||
        !source || source_len_bytes != layout_extent(layout, rows, cols)) {
        return invalid();
    }
    const bool pair = layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR;
    if (pair && (!codes_b || !scales_b)) return invalid();
    if (layout == AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) {
        const uint64_t code_bytes = tcgen05_codes_bytes(rows, cols);
        memcpy(codes, source, code_bytes);
        for (uint32_t r = 0; r < rows; ++r) {
            for (uint32_t sc = 0; sc < cols / 16; ++sc) {
                scales[static_cast<uint64_t>(r) * (cols / 16) + sc] = source[code_bytes + tcgen05_scale_offset(r, sc, cols)];
            }
        }
        return ok();
    }
    for (uint32_t m = 0; m < (pair ? 2u : 1u); ++m) {
        uint8_t* code_plane = m ? codes_b : codes;
        uint8_t* scale_plane = m ? scales_b : scales;
        for (uint32_t r = 0; r < rows; ++r) {
            for (uint32_t c = 0; c < cols / 2; ++c) {
                const StreamCoord at = stream_code_coord(pair, m, r, c, cols);
                uint32_t word;
                memcpy(&word, source + at.block * kStreamBlockBytes + at.offset, 4);
                code_plane[static_cast<uint64_t>(r) * (cols / 2) + c] = static_cast<uint8_t>(stream_unpack_byte(word, at.slot));
            }
            for (uint32_t sc = 0; sc < cols / 16; ++sc) {
                const StreamCoord at = stream_scale_coord(pair, m, r, sc, cols);
                scale_plane[static_cast<uint64_t>(r) * (cols / 16) + sc] = source[at.block * kStreamBlockBytes + at.offset];
            }
        }
    }
    return ok();
}

// ---- checkpoint formats ----------------------------------------------------------------------------
// A checkpoint hands NVFP4 weights over as the COMPACT planes plus one typed scalar
// (crates/augur-model-qwen35/src/checkpoint_quant.rs:10-58): compressed-tensors stores
// weight_global_scale and DIVIDES by it, ModelOpt stores weight_scale_2 and MULTIPLIES by it.
// The kernels of this library multiply, so the scalar is converted once at load time.
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_checkpoint_global_scale_host_v1(
    uint32_t convention, float checkpoint_scalar, float* out_global_scale) {
    if (!out_global_scale || !std::isfinite(checkpoint_scalar) || checkpoint_scalar <= 0.0f) return invalid();
    float multiplier;
    if (convention == AUGUR_NVFP4_SM100_SCALE_COMPRESSED_TENSORS) {
        multiplier = 1.0f / checkpoint_scalar;
    } else if (convention == AUGUR_NVFP4_SM100_SCALE_MODELOPT) {
        multiplier = checkpoint_scalar;
    } else {
        return invalid();
    }
    if (!scale_ok(multiplier)) return invalid();
    *out_global_scale = multiplier;
    return ok();
}

// The same validation the reference applies to checkpoint planes before anything is uploaded
// (checkpoint_quant.rs:113-133): non-empty shape, cols % 16, exact plane extents, no negative or
// NaN block scale.
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_checkpoint_validate_host_v1(
    uint64_t rows, uint64_t cols, const uint8_t* codes, uint64_t codes_len_bytes, const uint8_t* scales,
    uint64_t scales_len_bytes) {
    if (!rows || !cols || cols % 16 != 0 || !codes || !scales) return invalid();
    if (rows > UINT64_MAX / cols) return invalid();
    const uint64_t count = rows * cols;
    if (codes_len_bytes != count / 2 || scales_len_bytes != count / 16) return invalid();
    for (uint64_t i = 0; i < scales_len_bytes; ++i) {
        if (scales[i] >= 127) return invalid();
    }
    return ok();
}

// GGML36 wire blocks (checkpoint_quant.rs:157-189): 64 elements = 4 scale bytes, then four
// 8-byte groups; byte j of a group holds element j of the group's 16 in its low nibble and
// element j + 8 in its high nibble. Lossless in both directions; the global scalar stays apart.
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_planes_to_ggml36_host_v1(
    uint64_t rows, uint64_t cols, const uint8_t* codes, const uint8_t* scales, uint8_t* wire, uint64_t wire_len_bytes) {
    if (!rows || !cols || cols % 64 != 0 || !codes || !scales || !wire || rows > UINT64_MAX / cols) return invalid();
    const uint64_t blocks = rows * cols / 64;
    if (wire_len_bytes != blocks * 36) return invalid();
    for (uint64_t b = 0; b < blocks; ++b) {
        uint8_t* out = wire + b * 36;
        memcpy(out, scales + b * 4, 4);
        for (uint32_t group = 0; group < 4; ++group) {
            const uint8_t* src = codes + b * 32 + group * 8;   // 16 elements, two per byte, even element low
            for (uint32_t j = 0; j < 8; ++j) {
                const uint32_t first = (src[j / 2] >> ((j & 1) * 4)) & 15u;               // element j
                const uint32_t second = (src[(j + 8) / 2] >> (((j + 8) & 1) * 4)) & 15u;  // element j + 8
                out[4 + group * 8 + j] = static_cast<uint8_t>(first | (second << 4));
            }
        }
    }
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_ggml36_to_planes_host_v1(
    uint64_t rows, uint64_t cols, const uint8_t* wire, uint64_t wire_len_bytes, uint8_t* codes, uint8_t* scales) {
    if (!rows || !cols || cols % 64 != 0 || !codes || !scales || !wire || rows > UINT64_MAX / cols) return invalid();
    const uint64_t blocks = rows * cols / 64;
    if (wire_len_bytes != blocks * 36) return invalid();
    for (uint64_t b = 0; b < blocks; ++b) {
        const uint8_t* in = wire + b * 36;
        for (uint32_t i = 0; i < 4; ++i) {
            if (in[i] >= 127) return invalid();   // negative or NaN block scale
        }
        memcpy(scales + b * 4, in, 4);
        for (uint32_t group = 0; group < 4; ++group) {
            uint8_t* dst = codes + b * 32 + group * 8;
            for (uint32_t byte = 0; byte < 8; ++byte) {
                uint32_t value = 0;
                for (uint32_t half = 0; half < 2; ++half) {
                    const uint32_t element = byte * 2 + half;   // 0..15 inside the group
                    const uint32_t code = (in[4 + group * 8 + (element & 7)] >> ((element >> 3) * 4)) & 15u;
                    value |= code << (half * 4);
                }
                dst[byte] = static_cast<uint8_t>(value);
            }
        }
    }
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_interleave_gate_up_host_v1(
    uint32_t rows, uint32_t cols, const uint8_t* gate_codes, const uint8_t* gate_scales, const uint8_t* up_codes,
    const uint8_t* up_scales, uint8_t* out_codes, uint8_t* out_scales) {
    if (!rows || !cols || rows % 16 != 0 || cols % 16 != 0 || rows > INT_MAX / 2 || !gate_codes || !gate_scales || !up_codes ||
        !up_scales || !out_codes || !out_scales) {
        return invalid();
    }
    const uint64_t code_row = cols / 2, scale_row = cols / 16;
    for (uint32_t r = 0; r < rows; ++r) {
        const uint64_t gate_at = static_cast<uint64_t>(r / 16) * 32 + r % 16, up_at = gate_at + 16;
        memcpy(out_codes + gate_at * code_row, gate_codes + r * code_row, code_row);
        memcpy(out_codes + up_at * code_row, up_codes + r * code_row, code_row);
        memcpy(out_scales + gate_at * scale_row, gate_scales + r * scale_row, scale_row);
        memcpy(out_scales + up_at * scale_row, up_scales + r * scale_row, scale_row);
    }
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_preflight_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_repack_args_v1* a) {
    augur_cuda_result_v1 failure;
    return check_repack(d, s, a, true, &failure) ? ok() : failure;
}
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_repack_args_v1* a) {
    return submit_entry(d, s, a, check_repack, launch_repack);
}
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_dequant_f32_preflight_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_dequant_args_v1* a) {
    augur_cuda_result_v1 failure;
    return check_dequant(d, s, a, true, &failure) ? ok() : failure;
}
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_dequant_f32_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_dequant_args_v1* a) {
    return submit_entry(d, s, a, check_dequant, launch_dequant);
}
