// Index arithmetic of the hot layouts; shared by host repack, device repack and the kernels.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define AUGUR_HD __host__ __device__ __forceinline__
#else
#define AUGUR_HD inline
#endif

namespace augur_sm100 {

// ---- STREAM / STREAM_PAIR -------------------------------------------------------
// The tensor is cut into blocks of 32 weight rows x 128 k (8 k-steps of 16). A block
// is 2304 bytes: 2048 code bytes in mma.m16n8k16 A-fragment order, then 256 scale bytes.
//   codes : [tile t:2][quad q:2][lane:32][16 bytes]; the 16 bytes of a lane are 4 words,
//           word j = k-step 4q+j. A word carries the 8 codes of the lane's four fragment
//           registers (g = lane>>2, t4 = lane&3):
//             a0 (row g,   k 2t4, 2t4+1)   a1 (row g+8, same k)
//             a2 (row g,   k 2t4+8, +9)    a3 (row g+8, same k)
//           bit-permuted so that each register falls out of the word with at most a shift
//           and a mask, already positioned as the low exponent bits and top mantissa bit
//           of two BF16 numbers (see stream_pack_word). The even-k code of a register
//           sits in the low 16 bits, the odd-k code in the high 16 bits.
//   scales: [tile t:2][g:8][16 bytes] = k-steps 0..7, each {row g, row g+8}.
// STREAM:      block row-group s holds rows 32s..32s+31, tile t = rows 32s+16t..+15.
// STREAM_PAIR: block row-group s holds gate rows 16s..16s+15 (tile 0) and the
//              matching up rows (tile 1).
// Blocks are stored row-group major: index = s * (cols/128) + kb.
constexpr uint32_t kStreamBlockBytes = 2304;
constexpr uint32_t kStreamCodeBytes = 2048;
constexpr uint32_t kStreamBlockK = 128;

// An E2M1 code (s e1 e0 m) placed at BF16 bits (15; 8 7 6) reads as e2m1 * 2^-126 (the
// subnormal 0.5 included), so a register of two codes needs no arithmetic to become two
// BF16 values. Within each 16-bit half of a word the four registers' codes live at
//   a0: s15 e8 e7 m6     -> a0 =  w        & 0x81C081C0
//   a1: s12 e5 e4 m3     -> a1 = (w << 3)  & 0x81C081C0
//   a2: s9  e2 e1 m0     -> a2 = (w << 6)  & 0x81C081C0
//   a3: s11 e1@10 e0@14 m13 -> a3 = (((w >> 10) & 0x001B001B) * 0x4108) & 0x81C081C0
// `bytes` are the four source bytes of a0..a3 (low nibble = even k).
AUGUR_HD uint32_t stream_pack_word(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
    const uint32_t bytes[4] = {b0, b1, b2, b3};
    // destination bit of (sign, e1, e0, m) for each register, inside a 16-bit half
    const uint32_t where[4][4] = {{15, 8, 7, 6}, {12, 5, 4, 3}, {9, 2, 1, 0}, {11, 10, 14, 13}};
    uint32_t word = 0;
    for (uint32_t j = 0; j < 4; ++j) {
        for (uint32_t half = 0; half < 2; ++half) {
            const uint32_t code = (bytes[j] >> (4 * half)) & 15u;
            word |= ((code >> 3) & 1u) << (where[j][0] + 16 * half);
            word |= ((code >> 2) & 1u) << (where[j][1] + 16 * half);
            word |= ((code >> 1) & 1u) << (where[j][2] + 16 * half);
            word |= (code & 1u) << (where[j][3] + 16 * half);
        }
    }
    return word;
}

// Inverse of stream_pack_word: source byte of register j.
AUGUR_HD uint32_t stream_unpack_byte(uint32_t word, uint32_t j) {
    const uint32_t where[4][4] = {{15, 8, 7, 6}, {12, 5, 4, 3}, {9, 2, 1, 0}, {11, 10, 14, 13}};
    uint32_t byte = 0;
    for (uint32_t half = 0; half < 2; ++half) {
        const uint32_t code = (((word >> (where[j][0] + 16 * half)) & 1u) << 3) |
                              (((word >> (where[j][1] + 16 * half)) & 1u) << 2) |
                              (((word >> (where[j][2] + 16 * half)) & 1u) << 1) |
                              ((word >> (where[j][3] + 16 * half)) & 1u);
        byte |= code << (4 * half);
    }
    return byte;
}

struct StreamCoord {
    uint64_t block;    // block index
    uint32_t offset;   // byte offset inside the block: of the WORD for codes, of the byte for scales
    uint32_t slot;     // codes only: which register (0..3) of the word holds the source byte
};

// Where source code byte (matrix m, row r, byte column c) goes.
AUGUR_HD StreamCoord stream_code_coord(bool pair, uint32_t m, uint32_t r, uint32_t c, uint32_t cols) {
    const uint32_t kb_count = cols / kStreamBlockK;
    const uint32_t kstep = c >> 3, cb = c & 7;
    const uint32_t t4 = cb & 3, half = cb >> 2;
    const uint32_t kb = kstep >> 3, ks = kstep & 7, q = ks >> 2, j = ks & 3;
    const uint32_t group = pair ? (r >> 4) : (r >> 5);
    const uint32_t t = pair ? m : ((r >> 4) & 1);
    const uint32_t rr = r & 15, g = rr & 7, hi = rr >> 3;
    const uint32_t lane = g * 4 + t4;
    StreamCoord out;
    out.block = static_cast<uint64_t>(group) * kb_count + kb;
    out.offset = ((t * 2 + q) * 32 + lane) * 16 + j * 4;
    out.slot = hi + 2 * half;
    return out;
}

// Where source scale byte (matrix m, row r, k-step sc) goes.
AUGUR_HD StreamCoord stream_scale_coord(bool pair, uint32_t m, uint32_t r, uint32_t sc, uint32_t cols) {
    const uint32_t kb_count = cols / kStreamBlockK;
    const uint32_t kb = sc >> 3, ks = sc & 7;
    const uint32_t group = pair ? (r >> 4) : (r >> 5);
    const uint32_t t = pair ? m : ((r >> 4) & 1);
    const uint32_t rr = r & 15, g = rr & 7, hi = rr >> 3;
    StreamCoord out;
    out.block = static_cast<uint64_t>(group) * kb_count + kb;
    out.offset = kStreamCodeBytes + (t * 8 + g) * 16 + ks * 2 + hi;
    out.slot = 0;
    return out;
}

AUGUR_HD uint64_t stream_extent_bytes(bool pair, uint32_t rows, uint32_t cols) {
    const uint64_t groups = pair ? rows / 16 : rows / 32;
    return groups * (cols / kStreamBlockK) * kStreamBlockBytes;
}

// ---- TCGEN05 ---------------------------------------------------------------------
// Codes stay [rows][cols/2] (K-major, even k in the low nibble): exactly what a TMA
// tensor map of packed 4-bit data and the UMMA K-major descriptor consume. The block
// scales follow, re-tiled into 512-byte atoms of 128 rows x 4 scales (64 k): byte
//   (r % 32) * 16 + ((r / 32) % 4) * 4 + (sc % 4)
// of atom [r / 128][sc / 4]; atoms are stored row-block major, so one 128-row x 256-k
// tile of scales (4 atoms) is 2048 contiguous bytes. This is the arrangement
// tcgen05.cp (32x128b, warpx4) moves into tensor memory for scale_vec::4X.
// rows are padded up to a multiple of 128 in the scale region (padding bytes are 0).
constexpr uint32_t kSfAtomBytes = 512;

AUGUR_HD uint64_t tcgen05_codes_bytes(uint32_t rows, uint32_t cols) {
    return static_cast<uint64_t>(rows) * (cols / 2);
}
AUGUR_HD uint64_t tcgen05_scale_bytes(uint32_t rows, uint32_t cols) {
    const uint64_t row_blocks = (static_cast<uint64_t>(rows) + 127) / 128;
    return row_blocks * (cols / 64) * kSfAtomBytes;
}
AUGUR_HD uint64_t tcgen05_extent_bytes(uint32_t rows, uint32_t cols) {
    return tcgen05_codes_bytes(rows, cols) + tcgen05_scale_bytes(rows, cols);
}
// Byte offset of scale (row r, k-step sc) inside the scale region.
AUGUR_HD uint64_t tcgen05_scale_offset(uint32_t r, uint32_t sc, uint32_t cols) {
    const uint64_t atoms_per_row_block = cols / 64;
    const uint64_t atom = static_cast<uint64_t>(r / 128) * atoms_per_row_block + sc / 4;
    return atom * kSfAtomBytes + (r % 32) * 16 + ((r / 32) % 4) * 4 + (sc % 4);
}

}  // namespace augur_sm100
