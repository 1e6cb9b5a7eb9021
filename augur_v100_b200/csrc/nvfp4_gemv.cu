// Small-token (1..8) NVFP4 linear for sm_100a: a bandwidth-bound dequantising GEMV.
//
// Data path per weight block (32 rows x 128 k, 2304 bytes, already in mma fragment order with
// the codes bit-placed as BF16 fields): one bulk asynchronous copy into a per-warp ring in
// shared memory -> per k-step a shift and a mask per fragment register (the register is then
// two BF16 numbers e2m1 * 2^-126) -> mma.sync.m16n8k16 with the 8 token rows on the MMA n
// dimension, f32 result -> four f32 FMAs that apply the block scales of the two rows a lane
// holds. An FP32 SIMT inner product cannot keep up with HBM at 8 tokens (8 FMA per weight
// element), so the inner product is on the tensor cores and the ALU work is the decoding only.
//
// Activations are BF16 B fragments in shared memory, multiplied per token by an exact power of
// two so that every product with a 2^-126-scaled weight is a normal f32; partial sums are
// scaled back before they leave the warp, so CTAs need not agree on the exponent. A plain
// input is staged by each CTA for its own k-slab; an intermediate produced by the SwiGLU
// epilogue of this kernel is written staged (fixed exponent) and bulk-copied in.
//
// Work split (balanced over any grid): the block space of a k-slab is cut into equal
// contiguous spans, one per CTA, and each CTA's span into equal contiguous spans, one
// per warp. Row groups that straddle a warp boundary are combined in shared memory in
// warp order; row groups that straddle a CTA or slab boundary are combined through
// plan scratch with an arrival counter, the last arriver summing the slots in a fixed
// order. Nothing spins on another CTA, and the result does not depend on scheduling.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "nvfp4_internal.h"
#include "nvfp4_layout.cuh"

namespace augur_sm100 {
namespace {

static_assert(sizeof(augur_cuda_nvfp4_sm100_gemv_args_v1) == 88, "gemv ABI");
static_assert(sizeof(augur_cuda_nvfp4_sm100_mlp_args_v1) == 184, "mlp ABI");

constexpr uint32_t kWarps = 16;
constexpr uint32_t kDepth = 3;             // ring slots (weight blocks in flight) per warp
constexpr uint32_t kScaleScratchBytes = 1024;   // per warp: the f32 block scales of the block being consumed
constexpr uint32_t kWaitLimit = 1u << 18;   // bounded polls of a ring slot before the kernel gives up
constexpr uint32_t kMaxSlabBlocks = 40;    // 40 * 128 k = 5120 activations columns per slab (80 KB)
constexpr uint32_t kSlotFloats = 256;      // one partial tile: 32 lanes x 8 f32
constexpr uint32_t kCombineBlocks = 48;    // weight blocks a CTA streams in the time of one cross-CTA combine

struct GemvParams {
    const uint8_t* weight;
    const uint16_t* x;
    void* out;
    float* partials;
    uint32_t* counters;
    uint32_t* status_word;
    const uint8_t* staged;     // activations already staged by the producing launch (fixed exponent), or unused
    float fixed_factor;        // non-zero: input is `staged`, and both rescale factors are this constant
    uint16_t* staged_out;      // SwiGLU epilogue: also write the result as staged fragments (or null)
    uint32_t groups, kb_count, slabs, ctas_per_slab, max_contrib, unit;
    uint32_t rows, cols, tokens, epilogue;
    uint32_t store_rows;       // rows that are written (the output is [tokens][store_rows]); the rest of the weight rows is padding
    float global_a, global_b;
    // Tensor-parallel exchange (tp_world == 0: none): every rank's exchange buffer as mapped here.
    uint64_t exchange[AUGUR_NVFP4_SM100_MAX_TP_RANKS];
    uint32_t tp_world, tp_rank;
    uint32_t tp_sequence;      // host-counted sequence, or 0: the launch takes it from `tp_counter`
    uint32_t* tp_counter;      // {launches counted so far, CTAs of the running launch that are done}, in this rank's exchange buffer
};

struct GemvGeometry {
    uint32_t groups, kb_count, slabs, ctas_per_slab, max_contrib, unit;
    uint64_t partial_bytes;   // partial-sum slots
    uint64_t staged_bytes;    // staged activations + factors
};

// Host-side geometry; `sm_count` CTAs at most.
GemvGeometry geometry(uint32_t rows, uint32_t cols, bool pair, uint32_t sm_count) {
    GemvGeometry g{};
    g.groups = pair ? rows / 16 : rows / 32;
    g.kb_count = cols / kStreamBlockK;
    g.slabs = (g.kb_count + kMaxSlabBlocks - 1) / kMaxSlabBlocks;
    const uint32_t min_kbs = g.kb_count / g.slabs;
    // CTAs never wait on one another, so the grid may exceed the SM count when slabs > SMs.
    uint64_t per_slab = sm_count / g.slabs ? sm_count / g.slabs : 1;
    // With one k-slab, spans may be cut at row-group boundaries: every group is then finished inside
    // one CTA (no scratch, no fences, no atomics) at the price of whole groups of imbalance; cutting at
    // single blocks balances perfectly but ends every launch with the cross-CTA combine. The first wins
    // while the imbalance, in blocks per CTA, stays below what that combine costs (about 3 us, the time
    // a CTA streams kCombineBlocks blocks in).
    bool aligned = false;
    if (g.slabs == 1) {
        const uint64_t ctas = per_slab < g.groups ? per_slab : g.groups;
        const uint64_t most = (g.groups + ctas - 1) / ctas;                  // groups of the busiest CTA
        // imbalance = most - groups / sm_count groups, compared in blocks and scaled by sm_count to stay in integers
        aligned = (most * sm_count - g.groups) * min_kbs <= static_cast<uint64_t>(kCombineBlocks) * sm_count;
    }
    g.unit = aligned ? min_kbs : 1;
    const uint64_t least_units = static_cast<uint64_t>(g.groups) * min_kbs / g.unit;
    if (per_slab > least_units) per_slab = least_units;  // every CTA owns at least one unit
    g.ctas_per_slab = static_cast<uint32_t>(per_slab);
    g.max_contrib = g.slabs * ((g.ctas_per_slab + g.groups - 1) / g.groups + 1);
    g.partial_bytes = static_cast<uint64_t>(g.groups) * g.max_contrib * kSlotFloats * 4;
    g.staged_bytes = static_cast<uint64_t>(cols) * 16 + 256;
    return g;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- per-warp weight ring: bulk async copies (TMA engine) into shared memory ------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Issues the copy of one 2304-byte weight block into a ring slot (one lane calls this).
__device__ __forceinline__ void issue_block(uint32_t slot_addr, uint32_t bar, const uint8_t* block) {
    // order this warp's earlier generic-proxy reads of the slot before the async-proxy write
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_expect_tx(bar, kStreamBlockBytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(slot_addr), "l"(block), "r"(kStreamBlockBytes), "r"(bar)
                 : "memory");
}

constexpr uint32_t kCodeMask = 0x81C081C0u;   // BF16 sign + two low exponent bits + top mantissa bit, twice

// Eight E4M3 bytes -> eight f32 values.
__device__ __forceinline__ void cvt_e4m3x8(uint2 bytes, float (&out)[8]) {
    uint32_t h[4];
    asm("{\n"
        ".reg .b16 a, b, c, d;\n"
        "mov.b32 {a, b}, %4;\n"
        "mov.b32 {c, d}, %5;\n"
        "cvt.rn.f16x2.e4m3x2 %0, a;\n"
        "cvt.rn.f16x2.e4m3x2 %1, b;\n"
        "cvt.rn.f16x2.e4m3x2 %2, c;\n"
        "cvt.rn.f16x2.e4m3x2 %3, d;\n"
        "}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(bytes.x), "r"(bytes.y));
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
        out[2 * i] = pair.x;
        out[2 * i + 1] = pair.y;
    }
}

// The 256 block scales of a weight block are needed as f32 by every lane of a quad alike.
// Instead of each lane converting the bytes it needs (four times redundantly), the warp
// converts them once - 8 bytes per lane - into a per-warp 1 KB scratch laid out so that one
// 16-byte load gives a lane the {row g, row g+8} pairs of two consecutive k-steps:
//   [tile t:2][k-step pair kp:4][g:8][k-step parity:2][row g / row g+8].
__device__ __forceinline__ void convert_block_scales(const uint8_t* slot, float* scratch, uint32_t lane) {
    // lane L owns source bytes [8L, 8L+8): tile L/16, row pair g = (L%16)/2, k-steps 4*(L%2)..+3
    const uint2 bytes = *reinterpret_cast<const uint2*>(slot + kStreamCodeBytes + lane * 8);
    float v[8];
    cvt_e4m3x8(bytes, v);
    const uint32_t t = lane >> 4, g = (lane >> 1) & 7, half = lane & 1;
    float4* dst = reinterpret_cast<float4*>(scratch) + ((t * 4 + half * 2) * 8 + g);
    dst[0] = make_float4(v[0], v[1], v[2], v[3]);      // k-step pair 2*half
    dst[8] = make_float4(v[4], v[5], v[6], v[7]);      // k-step pair 2*half + 1
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// One k-step (16 k) of one 16-row tile: the code word becomes the four A-fragment registers
// with shifts and masks only (each register is two BF16 numbers equal to e2m1 * 2^-126; the
// tensor core takes the subnormal 0.5 * 2^-126 exactly), one MMA against the staged
// activations, then the block scales of rows g and g+8 are applied to the 16 x 8 partial
// product in f32.
__device__ __forceinline__ void tile_step(float (&acc)[4], uint32_t w, float sg, float sh, uint32_t b0, uint32_t b1) {
    uint32_t a[4];
    a[0] = w & kCodeMask;
    a[1] = (w << 3) & kCodeMask;
    a[2] = (w << 6) & kCodeMask;
    a[3] = (((w >> 10) & 0x001B001Bu) * 0x4108u) & kCodeMask;
    float d[4];
    mma_bf16(d, a, b0, b1);
    acc[0] = fmaf(sg, d[0], acc[0]);
    acc[1] = fmaf(sg, d[1], acc[1]);
    acc[2] = fmaf(sh, d[2], acc[2]);
    acc[3] = fmaf(sh, d[3], acc[3]);
}

// Four k-steps: one 16-byte code vector of this lane, two scale quads (k-step pairs), two
// B-fragment quads.
__device__ __forceinline__ void tile_quad(float (&acc)[4], const uint4& codes, const float4& s01, const float4& s23,
                                          const uint4& b01, const uint4& b23) {
    tile_step(acc, codes.x, s01.x, s01.y, b01.x, b01.y);
    tile_step(acc, codes.y, s01.z, s01.w, b01.z, b01.w);
    tile_step(acc, codes.z, s23.x, s23.y, b23.x, b23.y);
    tile_step(acc, codes.w, s23.z, s23.w, b23.z, b23.w);
}

// acc[t*4 + i] += block (32 rows x 128 k, in a ring slot) * activations (this block's B fragments).
__device__ __forceinline__ void compute_block(float (&acc)[8], const uint8_t* slot, const uint4* act, float* scale_scratch,
                                              uint32_t lane) {
    convert_block_scales(slot, scale_scratch, lane);
    __syncwarp();
    const uint4* codes = reinterpret_cast<const uint4*>(slot);
    const float4* scales = reinterpret_cast<const float4*>(scale_scratch) + (lane >> 2);
    const uint4 b0 = act[lane], b1 = act[32 + lane], b2 = act[64 + lane], b3 = act[96 + lane];
    float(&d0)[4] = *reinterpret_cast<float(*)[4]>(&acc[0]);
    float(&d1)[4] = *reinterpret_cast<float(*)[4]>(&acc[4]);
    const uint4 c00 = codes[lane], c01 = codes[32 + lane], c10 = codes[64 + lane], c11 = codes[96 + lane];
    tile_quad(d0, c00, scales[0], scales[8], b0, b1);          // tile 0, k-step pairs 0, 1
    tile_quad(d1, c10, scales[32], scales[40], b0, b1);        // tile 1
    tile_quad(d0, c01, scales[16], scales[24], b2, b3);        // tile 0, k-step pairs 2, 3
    tile_quad(d1, c11, scales[48], scales[56], b2, b3);
    __syncwarp();   // the scratch is rewritten for the next block
}

// Which of `parts` equal contiguous spans of [0, total) holds index `at`.
// All block indices fit 32 bits with room for this product: rows*cols <= 2^32 makes
// groups*blocks-per-group <= 2^21, and `parts` is at most a few hundred.
__device__ __forceinline__ uint32_t span_of(uint32_t at, uint32_t total, uint32_t parts) {
    return ((at + 1) * parts - 1) / total;
}

// An intermediate produced inside a program (SiLU(gate)*up) is staged for the next projection
// by the epilogue that computes it, with this fixed exponent shift instead of a per-token one
// (no pass over the finished tensor is needed): exact for magnitudes in [2^-60, 2^62],
// saturating above, flushing below.
constexpr int kFixedStageShift = 64;

// BF16 bits times 2^shift by exponent arithmetic: exact; zeros and subnormals become zero,
// and anything that would leave the normal range on the way down is flushed to zero
// (it is more than 2^200 below the row's largest magnitude). Infinities and NaNs pass through.
__device__ __forceinline__ uint32_t shift_bf16(uint32_t bits, int shift) {
    const int field = static_cast<int>((bits >> 7) & 0xff);
    if (field == 0xff) return bits;
    const int moved = field + shift;
    if (field == 0 || moved < 1) return bits & 0x8000u;
    return (bits & 0x807fu) | (static_cast<uint32_t>(moved > 254 ? 254 : moved) << 7);
}

// ---- tensor-parallel exchange ------------------------------------------------------------------
// Row-parallel down projection over `tp_world` GPUs: every rank holds a k-slice and produces a
// full-width partial sum; the all-reduce is done inside this kernel instead of by a collective
// launched afterwards. Exchange buffer of a rank (same layout on all):
//   [sequence parity][source rank][row group][32 lanes][4 lines of 16 bytes]
// where a line is {value, sequence, value, sequence}: every 8-byte half carries its own flag, an
// aligned 8-byte store becomes visible as a whole, so a reader needs no fence - it polls the
// lines themselves until both flags show the sequence it is waiting for.
//   push   : the warp that finishes a row group stores its tile (256 f32 as 128 lines) into the
//            slot [parity][own rank][group] of EVERY rank's buffer, its own included (peer
//            stores over NVLink), and goes on;
//   reduce : at the end of the kernel every row group is taken by one warp of the grid (static
//            assignment, independent of who finished it), which reads the tiles of all ranks
//            for that group from its own rank's buffer - waiting, bounded, for lines that have
//            not arrived - adds them in rank order and writes the BF16 result.
// Every rank adds the same values in the same order, so all ranks hold bit-identical results.
// Two parities suffice: a source can only overwrite a slot two sequences later, and it cannot
// start the next sequence before this rank has delivered all of its tiles of the current one,
// i.e. after this rank has finished the one before. The reduce step waits for tiles that other
// CTAs of the same grid produce, so the grid must be co-resident (the entry point checks that it
// does not exceed the SM count).
constexpr uint32_t kExchangeWaitLimit = 1u << 20;   // polls of about a microsecond: gives up after about a second
constexpr uint32_t kExchangeTileBytes = kSlotFloats * 8;

// The tiles of both parities, then 256 bytes that hold the device-side sequence counter of this rank.
__host__ __device__ constexpr uint64_t exchange_tiles_bytes(uint32_t world, uint32_t groups) {
    return 2ull * world * groups * kExchangeTileBytes;
}
__host__ __device__ constexpr uint64_t exchange_extent(uint32_t world, uint32_t groups) {
    return exchange_tiles_bytes(world, groups) + 256;
}

// Sequence of a launch that counts on the device: launches 0, 1, 2, ... map to 1, 2, ..., 0xFFFFFFFE, 1, ...
// (never 0, the value of a fresh buffer; the parity alternates across the wrap). Every rank runs the same
// launches in the same order, so the ranks' counters agree without talking to each other, and a captured
// CUDA graph can be replayed: nothing about the sequence is baked into the launch parameters.
__device__ __forceinline__ uint32_t sequence_of(uint32_t launches) { return launches % 0xFFFFFFFEu + 1u; }

// exchange[r] by a chain of selects: a run-time index into kernel parameters would put the table on the stack.
__device__ __forceinline__ uint64_t exchange_base(const GemvParams& p, uint32_t r) {
    uint64_t base = p.exchange[0];
#pragma unroll
    for (uint32_t i = 1; i < AUGUR_NVFP4_SM100_MAX_TP_RANKS; ++i) {
        if (r == i) base = p.exchange[i];
    }
    return base;
}
__device__ __forceinline__ uint64_t exchange_slot(const GemvParams& p, uint32_t seq, uint32_t src, uint32_t group, uint32_t lane) {
    return ((static_cast<uint64_t>(seq & 1) * p.tp_world + src) * p.groups + group) * kExchangeTileBytes + lane * 64;
}

__device__ __forceinline__ void exchange_push(const GemvParams& p, uint32_t seq, uint32_t group, const float (&v)[8], uint32_t lane) {
    const uint64_t offset = exchange_slot(p, seq, p.tp_rank, group, lane);
#pragma unroll
    for (uint32_t d = 0; d < AUGUR_NVFP4_SM100_MAX_TP_RANKS; ++d) {
        if (d < p.tp_world) {
            const uint64_t dst = p.exchange[d] + offset;
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};"
                             ::"l"(dst + j * 16), "r"(__float_as_uint(v[2 * j] * p.global_a)), "r"(seq),
                               "r"(__float_as_uint(v[2 * j + 1] * p.global_a))
                             : "memory");
            }
        }
    }
}

// Whole warps call this once, after everything else the kernel does.
__device__ __forceinline__ void exchange_reduce(const GemvParams& p, uint32_t seq, uint32_t warp, uint32_t lane, uint32_t cta,
                                                uint32_t ctas) {
    const uint32_t world = p.tp_world;
    const uint64_t own = exchange_base(p, p.tp_rank);
    constexpr uint32_t kBatch = 4;   // sources polled together, so that their load latencies overlap
    bool arrived = true;
    for (uint32_t group = cta + ctas * warp; group < p.groups; group += ctas * kWarps) {
        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t first = 0; first < world; first += kBatch) {
            uint32_t line[kBatch][4][4];
            uint32_t spin = 0;
            for (;;) {
                bool ready = true;
#pragma unroll
                for (uint32_t q = 0; q < kBatch; ++q) {
                    if (first + q < world) {
                        const uint64_t from = own + exchange_slot(p, seq, first + q, group, lane);
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(line[q][j][0]), "=r"(line[q][j][1]), "=r"(line[q][j][2]), "=r"(line[q][j][3])
                                         : "l"(from + j * 16)
                                         : "memory");
                        }
                    }
                }
#pragma unroll
                for (uint32_t q = 0; q < kBatch; ++q) {
                    if (first + q < world) {
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) ready = ready && line[q][j][1] == seq && line[q][j][3] == seq;
                    }
                }
                if (ready) break;
                if (++spin > kExchangeWaitLimit) { arrived = false; break; }
            }
#pragma unroll
            for (uint32_t q = 0; q < kBatch; ++q) {
                if (first + q < world) {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        sum[2 * j] += __uint_as_float(line[q][j][0]);
                        sum[2 * j + 1] += __uint_as_float(line[q][j][2]);
                    }
                }
            }
        }
        const uint32_t g = lane >> 2, t4 = lane & 3;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t token = 2 * t4 + (i & 1);
            const uint32_t row = group * 32 + (i >> 2) * 16 + g + ((i >> 1) & 1) * 8;
            if (token < p.tokens) {
                static_cast<__nv_bfloat16*>(p.out)[static_cast<uint64_t>(token) * p.rows + row] = __float2bfloat16_rn(sum[i]);
            }
        }
    }
    if (!__all_sync(0xffffffffu, arrived) && lane == 0) atomicCAS(p.status_word, 0u, 0x203u);   // a tile never arrived
}

__device__ __forceinline__ void epilogue(const GemvParams& p, uint32_t seq, uint32_t group, const float (&v)[8], uint32_t lane) {
    if (p.tp_world) {
        exchange_push(p, seq, group, v, lane);   // the sum over ranks is written by exchange_reduce
        return;
    }
    const uint32_t g = lane >> 2, t4 = lane & 3;
    if (p.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t token = 2 * t4 + (i & 1);
            const uint32_t row = group * 16 + g + (i >> 1) * 8;
            if (token < p.tokens) {
                const float gate = v[i] * p.global_a;
                const float up = v[4 + i] * p.global_b;
                const __nv_bfloat16 h = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                out[static_cast<uint64_t>(token) * p.rows + row] = h;
                if (p.staged_out) {
                    // The same value as the next projection's B fragment: k = row, so k-step = group,
                    // fragment register i>>1 (rows g / g+8 are k%16 = g / g+8), pair g/2, half g%2;
                    // shifted by the fixed staging exponent instead of a per-token one.
                    const uint32_t word = ((group >> 1) * 32 + token * 4 + (g >> 1)) * 4 + (group & 1) * 2 + (i >> 1);
                    p.staged_out[word * 2 + (g & 1)] =
                        static_cast<uint16_t>(shift_bf16(__bfloat16_as_ushort(h), kFixedStageShift));
                }
            }
        }
        return;
    }
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t token = 2 * t4 + (i & 1);
        const uint32_t row = group * 32 + (i >> 2) * 16 + g + ((i >> 1) & 1) * 8;
        if (token < p.tokens && row < p.store_rows) {
            const float value = v[i] * p.global_a;
            if (p.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) {
                static_cast<float*>(p.out)[static_cast<uint64_t>(token) * p.store_rows + row] = value;
            } else {
                static_cast<__nv_bfloat16*>(p.out)[static_cast<uint64_t>(token) * p.store_rows + row] = __float2bfloat16_rn(value);
            }
        }
    }
}

// ---- activation staging --------------------------------------------------------------------
// Plain BF16 activations are staged by every CTA for its own k-slab: the CTA finds each token
// row's largest magnitude over the slab, picks the exponent shift e that puts it in
// [2^100, 2^101) (so that the 2^-126-scaled weight fragments meet activations large enough to
// keep every product a normal f32), and writes x * 2^e as BF16 into shared memory in the mma
// B-fragment order
//   [k-step pair][lane = token*4 + t4][4 words: b0,b1 of the even k-step, b0,b1 of the odd one].
// The raw rows arrive by bulk copy in the same shared memory the fragments will occupy. A lane
// handles one token (lane/4) and one 16-byte chunk (8 k) of every 16th k-step pair; it takes
// all its chunks into registers before anything is rewritten, and - with the four words of a
// chunk stored in an order rotated by token/2 - the 32 lanes of a store hit 32 different banks.
constexpr uint32_t kStageChunks = kMaxSlabBlocks * 4 / kWarps;   // chunks per lane, at most

// Returns the two factors (product 2^(126 - e)) in `factor_out[2*token], [2*token+1]` (shared).
__device__ __forceinline__ void stage_activations(const GemvParams& p, uint32_t kbs, uint32_t* act_words,
                                                  float* amax_scratch, float* factor_out, uint32_t lane, uint32_t warp) {
    const uint32_t token = lane >> 2, cc = lane & 3;
    const uint32_t pairs = kbs * 4;   // k-step pairs in the slab
    const bool live = token < p.tokens;
    // The slab's columns of every token row were bulk-copied, as they are, to the front of the
    // activation area ([token][kbs*256 bytes]); each lane takes its chunks into registers, and the
    // area is rewritten in fragment order once every lane has (the barrier below).
    const uint4* row = reinterpret_cast<const uint4*>(act_words) + token * kbs * 16;
    uint4 v[kStageChunks];
#pragma unroll
    for (uint32_t j = 0; j < kStageChunks; ++j) {
        const uint32_t q = warp + kWarps * j;
        v[j] = make_uint4(0, 0, 0, 0);
        if (live && q < pairs) v[j] = row[q * 4 + cc];
    }
    // largest magnitude, two BF16 lanes at a time
    __nv_bfloat162 amax2 = __float2bfloat162_rn(0.0f);
#pragma unroll
    for (uint32_t j = 0; j < kStageChunks; ++j) {
        const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) amax2 = __hmax2_nan(amax2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i])));
    }
    float amax = fmaxf(__low2float(amax2), __high2float(amax2));
    if (!(amax == amax)) amax = __int_as_float(0x7f800000);   // a NaN anywhere: the row is staged unshifted
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (cc == 0) amax_scratch[warp * 8 + token] = amax;
    __syncthreads();
    float m = 0.0f;
#pragma unroll
    for (uint32_t w = 0; w < kWarps; ++w) m = fmaxf(m, amax_scratch[w * 8 + token]);
    int e = 0;   // zero or non-finite rows are staged unshifted
    const int field = static_cast<int>((__float_as_uint(m) >> 23) & 0xff);
    if (m > 0.0f && field != 0xff && field != 0) e = 227 - field;
    if (warp == 0 && cc == 0) {
        // partial sums are multiplied by 2^(126 - e), split in two factors that are always finite
        const int q = 126 - e, q0 = q / 2, q1 = q - q0;
        factor_out[2 * token] = __uint_as_float(static_cast<uint32_t>(127 + q0) << 23);
        factor_out[2 * token + 1] = __uint_as_float(static_cast<uint32_t>(127 + q1) << 23);
    }
    // x * 2^e as two exact BF16 multiplications by 2^(e/2) and 2^(e - e/2) (e is in [-27, 226]);
    // the values only move toward the staged row's magnitude, so neither step can overflow.
    const int e0 = e / 2, e1 = e - e0;
    const __nv_bfloat162 f0 = __float2bfloat162_rn(__uint_as_float(static_cast<uint32_t>(127 + e0) << 23));
    const __nv_bfloat162 f1 = __float2bfloat162_rn(__uint_as_float(static_cast<uint32_t>(127 + e1) << 23));
    const uint32_t turn = token >> 1;
#pragma unroll
    for (uint32_t j = 0; j < kStageChunks; ++j) {
        const uint32_t q = warp + kWarps * j;
        if (q >= pairs) break;
        // chunk (q, cc) holds k-step 2q + cc/2, fragment register cc%2; its word i is the pair
        // k%16 = 8(cc%2) + 2i, +1 and belongs to B-fragment lane token*4 + i
        uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        if (turn & 1) { const uint32_t t = w[0]; w[0] = w[1]; w[1] = w[2]; w[2] = w[3]; w[3] = t; }
        if (turn & 2) { uint32_t t = w[0]; w[0] = w[2]; w[2] = t; t = w[1]; w[1] = w[3]; w[3] = t; }
        uint32_t* dst = act_words + q * 128 + token * 16 + cc;
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t word = (i + turn) & 3;
            const __nv_bfloat162 moved = __hmul2(__hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]), f0), f1);
            dst[word * 4] = *reinterpret_cast<const uint32_t*>(&moved);
        }
    }
}

// One CTA's finished share of row group `group` in k-slab `slab` (whole warp calls this).
__device__ __forceinline__ void contribute(const GemvParams& p, uint32_t seq, uint32_t group, uint32_t slab, uint32_t cta_in_slab,
                                           const float (&v)[8], uint32_t lane) {
    // Spans cut at row-group boundaries (one k-slab): the group was finished inside this CTA.
    if (p.unit != 1) {
        epilogue(p, seq, group, v, lane);
        return;
    }
    // How many CTAs hold a share of this group, over all k-slabs, and which of them this one is.
    uint32_t total = 0, mine = 0;
    if (p.kb_count % p.slabs == 0) {
        // every slab is cut alike
        const uint32_t kbs = p.kb_count / p.slabs, units = p.groups * kbs;
        const uint32_t first = span_of(group * kbs, units, p.ctas_per_slab);
        const uint32_t count = span_of((group + 1) * kbs - 1, units, p.ctas_per_slab) - first + 1;
        total = p.slabs * count;
        mine = slab * count + (cta_in_slab - first);
    } else {
        for (uint32_t s = 0; s < p.slabs; ++s) {
            const uint32_t kbs = (s + 1) * p.kb_count / p.slabs - s * p.kb_count / p.slabs;
            const uint32_t units = p.groups * kbs;
            const uint32_t first = span_of(group * kbs, units, p.ctas_per_slab);
            const uint32_t last = span_of((group + 1) * kbs - 1, units, p.ctas_per_slab);
            if (s == slab) mine = total + (cta_in_slab - first);
            total += last - first + 1;
        }
    }
    if (total == 1) {
        epilogue(p, seq, group, v, lane);
        return;
    }
    float* slots = p.partials + static_cast<uint64_t>(group) * p.max_contrib * kSlotFloats;
    float4* my_slot = reinterpret_cast<float4*>(slots + static_cast<uint64_t>(mine) * kSlotFloats) + lane * 2;
    my_slot[0] = make_float4(v[0], v[1], v[2], v[3]);
    my_slot[1] = make_float4(v[4], v[5], v[6], v[7]);
    __threadfence();
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(&p.counters[group], 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived + 1 != total) return;
    __threadfence();
    // Slots are summed in slot order; four are fetched at a time so that their latencies overlap.
    float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t j0 = 0; j0 < total; j0 += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const float4* slot = reinterpret_cast<const float4*>(slots + static_cast<uint64_t>(j0 + j) * kSlotFloats) + lane * 2;
            a[j] = b[j] = make_float4(0, 0, 0, 0);
            if (j0 + j < total) {
                a[j] = __ldcg(slot);
                b[j] = __ldcg(slot + 1);
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            if (j0 + j < total) {
                sum[0] += a[j].x; sum[1] += a[j].y; sum[2] += a[j].z; sum[3] += a[j].w;
                sum[4] += b[j].x; sum[5] += b[j].y; sum[6] += b[j].z; sum[7] += b[j].w;
            }
        }
    }
    epilogue(p, seq, group, sum, lane);
    if (lane == 0) p.counters[group] = 0;  // leave the counter clean for the next launch
}

// The work of CTA `cta` of the `ctas` that share the linear `p`.
__device__ __forceinline__ void gemv_body(const GemvParams& p, uint32_t cta, uint32_t ctas, uint8_t* smem) {
    // Let the next kernel in the stream become resident on SMs as this grid drains; every
    // kernel of this library defers its global reads of produced data, and all of its global
    // writes, until its own griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint4* act = reinterpret_cast<uint4*>(smem);                              // [kbs*4][32] x 16 B
    uint8_t* ring = smem + kMaxSlabBlocks * 4 * 512;                          // [warps][kDepth] x 2304 B
    uint8_t* scale_area = ring + kWarps * kDepth * kStreamBlockBytes;         // [warps] x 1 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(scale_area + kWarps * kScaleScratchBytes);   // ring slots, then one for act
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t slab = cta / p.ctas_per_slab, cta_in_slab = cta % p.ctas_per_slab;
    const uint32_t kb_lo = slab * p.kb_count / p.slabs;
    const uint32_t kbs = (slab + 1) * p.kb_count / p.slabs - kb_lo;
    const uint32_t units = p.groups * kbs / p.unit;
    const uint32_t c0 = cta_in_slab * units / p.ctas_per_slab * p.unit, c1 = (cta_in_slab + 1) * units / p.ctas_per_slab * p.unit;
    const uint32_t len = c1 - c0;
    const uint32_t w0 = c0 + warp * len / kWarps, w1 = c0 + (warp + 1) * len / kWarps;

    // A cursor over this warp's blocks: (row group, block inside the slab, address). Stepping it
    // costs an add and a compare; no division in the streaming loop.
    struct Cursor {
        uint32_t group, kbi;
        const uint8_t* ptr;
    };
    const uint32_t group_skip = (p.kb_count - kbs) * kStreamBlockBytes;   // bytes of other slabs between row groups
    auto cursor_at = [&](uint32_t at) {
        Cursor c;
        c.group = at / kbs;
        c.kbi = at - c.group * kbs;
        c.ptr = p.weight + (static_cast<uint64_t>(c.group) * p.kb_count + kb_lo + c.kbi) * kStreamBlockBytes;
        return c;
    };
    auto step = [&](Cursor& c) {
        c.ptr += kStreamBlockBytes;
        if (++c.kbi == kbs) {
            c.kbi = 0;
            ++c.group;
            c.ptr += group_skip;
        }
    };
    Cursor fetch = cursor_at(w0);
    uint8_t* my_ring = ring + warp * kDepth * kStreamBlockBytes;
    const uint32_t my_bars = smem_u32(bars + warp * kDepth);

    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i <= kWarps * kDepth; ++i) mbar_init(smem_u32(bars + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Weight copies go out first so that HBM is busy while the activations are staged.
    if (lane == 0) {
        for (uint32_t d = 0; d < kDepth; ++d) {
            if (w0 + d < w1) {
                issue_block(smem_u32(my_ring + d * kStreamBlockBytes), my_bars + 8 * d, fetch.ptr);
                step(fetch);
            }
        }
    }

    // ---- activations of this k-slab ----
    // Everything above touched only this CTA's shared memory and read-only weights, so it may
    // run while the kernel before this one is still in flight; from here on its output is needed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Tensor-parallel launches that count their sequence on the device read the counter here: the launch
    // before this one is complete, and nobody advances the counter before every CTA of this grid is done.
    uint32_t seq = p.tp_sequence;
    uint32_t launches_before = 0;
    if (p.tp_world && seq == 0) {
        launches_before = *reinterpret_cast<volatile uint32_t*>(p.tp_counter);
        seq = sequence_of(launches_before);
    }
    float* stage_scratch = reinterpret_cast<float*>(scale_area);   // free until the streaming loop starts
    const bool plain = p.fixed_factor == 0.0f;
    {
        // Plain BF16 input: the slab's columns of each token row, copied as they are and staged
        // below. Otherwise the producing launch's epilogue staged them (fixed exponent) and they
        // are copied in ready for use.
        const uint32_t act_bar = smem_u32(bars + kWarps * kDepth);
        const uint32_t row_bytes = kbs * 256;
        const uint32_t act_bytes = plain ? p.tokens * row_bytes : kbs * 2048;   // staged: 4 k-step pairs x 512 bytes per block
        if (threadIdx.x == 0) mbar_expect_tx(act_bar, act_bytes);
        __syncthreads();
        // one copy per warp, issued in parallel
        const uint8_t* src;
        uint32_t begin, bytes = 0;
        if (plain) {
            src = reinterpret_cast<const uint8_t*>(p.x) + (static_cast<uint64_t>(warp) * p.cols + kb_lo * kStreamBlockK) * 2;
            begin = warp * row_bytes;
            if (warp < p.tokens) bytes = row_bytes;
        } else {
            const uint32_t per_warp = (kbs + kWarps - 1) / kWarps * 2048;
            begin = warp * per_warp;
            src = p.staged + static_cast<uint64_t>(kb_lo) * 2048 + begin;
            if (begin < act_bytes) bytes = act_bytes - begin < per_warp ? act_bytes - begin : per_warp;
        }
        if (lane == 0 && bytes) {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(smem + begin)), "l"(src), "r"(bytes), "r"(act_bar)
                         : "memory");
        }
        uint32_t spin = 0;
        bool arrived = true;
        while (!mbar_try_wait(act_bar, 0)) {
            if (++spin > kWaitLimit) { arrived = false; break; }
        }
        if (!arrived && threadIdx.x == 0) atomicCAS(p.status_word, 0u, 0x202u);   // the activations never arrived
    }
    if (plain) {
        stage_activations(p, kbs, reinterpret_cast<uint32_t*>(smem), stage_scratch, stage_scratch + kWarps * 8, lane, warp);
        __syncthreads();
    }

    const uint32_t t4 = lane & 3;
    float inv0a = p.fixed_factor, inv0b = p.fixed_factor, inv1a = p.fixed_factor, inv1b = p.fixed_factor;
    if (plain) {
        const float* factors = stage_scratch + kWarps * 8;
        inv0a = factors[4 * t4]; inv0b = factors[4 * t4 + 1];         // token 2*t4
        inv1a = factors[4 * t4 + 2]; inv1b = factors[4 * t4 + 3];     // token 2*t4 + 1
        __syncthreads();   // the scratch becomes the block-scale area of the streaming loop
    }
    Cursor now = cursor_at(w0);
    const uint32_t first_group = now.group;

    // ---- stream this warp's span of blocks ----
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint32_t seg_group = first_group;
    uint32_t seg_first_kbi = now.kbi;

    // A segment that covers its row group completely is finished here; a partial one is kept
    // (head in registers, tail in the accumulators) until this warp's ring is free to hold it.
    float head[8];
    bool have_head = false, have_tail = false;
    auto flush = [&](uint32_t group, uint32_t first_kbi, uint32_t last_kbi, bool last_segment) {
        float v[8];
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) v[i] = acc[i] * ((i & 1) ? inv1a : inv0a) * ((i & 1) ? inv1b : inv0b);
        if (first_kbi == 0 && last_kbi + 1 == kbs) {
            contribute(p, seq, group, slab, cta_in_slab, v, lane);
        } else if (group == first_group) {
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) head[i] = v[i];
            have_head = true;
        } else {
            // only the last segment of a span can be a partial that is not the head
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) acc[i] = v[i];
            have_tail = last_segment;
            return;
        }
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) acc[i] = 0.0f;
    };

    bool ring_ok = true;
    uint32_t slot = 0, parity = 0;
    for (uint32_t at = w0; at < w1; ++at) {
        const uint32_t kbi = now.kbi;
        if (now.group != seg_group) {
            flush(seg_group, seg_first_kbi, kbs - 1, false);
            seg_group = now.group;
            seg_first_kbi = 0;
        }
        uint32_t spin = 0;
        while (!mbar_try_wait(my_bars + 8 * slot, parity)) {
            if (++spin > kWaitLimit) { ring_ok = false; break; }
        }
        if (!ring_ok) break;
        compute_block(acc, my_ring + slot * kStreamBlockBytes, act + kbi * 128,
                      reinterpret_cast<float*>(scale_area + warp * kScaleScratchBytes), lane);
        __syncwarp();
        if (lane == 0 && at + kDepth < w1) {
            issue_block(smem_u32(my_ring + slot * kStreamBlockBytes), my_bars + 8 * slot, fetch.ptr);
            step(fetch);
        }
        step(now);
        if (++slot == kDepth) {
            slot = 0;
            parity ^= 1;
        }
    }
    if (!ring_ok && lane == 0) atomicCAS(p.status_word, 0u, 0x201u);   // a weight copy never arrived
    if (w1 > w0) flush(seg_group, seg_first_kbi, (w1 - 1) % kbs, true);
    // This warp's ring is idle now (every copy it issued has landed and been read): park the
    // partial segments in its first slot for the CTA-level combination below.
    float* warp_partial = reinterpret_cast<float*>(ring);
    constexpr uint32_t kWarpPartialFloats = kDepth * kStreamBlockBytes / 4;   // floats per warp ring
    if (have_head) {
        float4* dst = reinterpret_cast<float4*>(warp_partial + warp * kWarpPartialFloats) + lane * 2;
        dst[0] = make_float4(head[0], head[1], head[2], head[3]);
        dst[1] = make_float4(head[4], head[5], head[6], head[7]);
    }
    if (have_tail) {
        float4* dst = reinterpret_cast<float4*>(warp_partial + warp * kWarpPartialFloats + kSlotFloats) + lane * 2;
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    __syncthreads();

    // ---- combine row groups that were split between warps of this CTA ----
    if (len != 0) {
        const uint32_t cta_first_group = c0 / kbs;
        const uint32_t cta_groups = (c1 - 1) / kbs - cta_first_group + 1;
        for (uint32_t index = warp; index < cta_groups; index += kWarps) {
            const uint32_t group = cta_first_group + index;
            const uint32_t lo = group * kbs > c0 ? group * kbs : c0;
            const uint32_t hi = (group + 1) * kbs < c1 ? (group + 1) * kbs : c1;
            const uint32_t w_lo = span_of(lo - c0, len, kWarps), w_hi = span_of(hi - 1 - c0, len, kWarps);
            if (w_lo == w_hi && lo == group * kbs && hi == (group + 1) * kbs) continue;  // one warp had it all
            float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (uint32_t w = w_lo; w <= w_hi; ++w) {
                const uint32_t b0 = c0 + w * len / kWarps, b1 = c0 + (w + 1) * len / kWarps;
                if (b1 == b0) continue;
                const uint32_t slot = (b0 >= group * kbs) ? 0 : 1;   // the span's first row group parks in slot 0
                const float4* src = reinterpret_cast<const float4*>(warp_partial + w * kWarpPartialFloats + slot * kSlotFloats) + lane * 2;
                const float4 a = src[0], b = src[1];
                sum[0] += a.x; sum[1] += a.y; sum[2] += a.z; sum[3] += a.w;
                sum[4] += b.x; sum[5] += b.y; sum[6] += b.z; sum[7] += b.w;
            }
            contribute(p, seq, group, slab, cta_in_slab, sum, lane);
        }
    }
    // ---- tensor-parallel: add the ranks' tiles of the row groups assigned to this warp ----
    if (p.tp_world) {
        exchange_reduce(p, seq, warp, lane, cta, ctas);
        if (p.tp_sequence == 0) {
            // the last CTA to get here advances the counter for the next launch and clears the arrivals
            __syncthreads();
            if (threadIdx.x == 0) {
                __threadfence();
                if (atomicAdd(p.tp_counter + 1, 1u) + 1 == ctas) {
                    p.tp_counter[1] = 0;
                    p.tp_counter[0] = launches_before + 1;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kWarps * 32, 1) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    gemv_body(p, blockIdx.x, gridDim.x, smem);
}

// Up to four linears that read the same staged activations, as one grid (the grouped projections of a norm
// group): CTA b works for the member whose CTA range holds b. The members share nothing but the input; each has
// its own counters and partial-sum slots.
constexpr uint32_t kMaxGroupMembers = 4;
struct GemvGroupParams {
    GemvParams member[kMaxGroupMembers];
    uint32_t first_cta[kMaxGroupMembers + 1];
};
__global__ void __launch_bounds__(kWarps * 32, 1) gemv_group_kernel(const __grid_constant__ GemvGroupParams g) {
    extern __shared__ __align__(128) uint8_t smem[];
    // a chain of compile-time indices: a run-time index into kernel parameters would copy them to the stack
    if (blockIdx.x < g.first_cta[1]) {
        gemv_body(g.member[0], blockIdx.x, g.first_cta[1], smem);
    } else if (blockIdx.x < g.first_cta[2]) {
        gemv_body(g.member[1], blockIdx.x - g.first_cta[1], g.first_cta[2] - g.first_cta[1], smem);
    } else if (blockIdx.x < g.first_cta[3]) {
        gemv_body(g.member[2], blockIdx.x - g.first_cta[2], g.first_cta[3] - g.first_cta[2], smem);
    } else {
        gemv_body(g.member[3], blockIdx.x - g.first_cta[3], g.first_cta[4] - g.first_cta[3], smem);
    }
}

constexpr uint32_t kGemvSmemBytes = kMaxSlabBlocks * 4 * 512 + kWarps * kDepth * kStreamBlockBytes +
                                    kWarps * kScaleScratchBytes + (kWarps * kDepth + 1) * 8;

// ---- validation ---------------------------------------------------------------------------
bool check_gemv_scalars(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, bool* pair) {
    if (a->reserved1 || a->epilogue > AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) return false;
    *pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    if (a->stored_rows && (*pair || a->stored_rows > a->rows)) return false;   // a trimmed store: plain linears only
    if (!a->rows || !a->cols || a->rows > INT_MAX || a->cols > INT_MAX) return false;
    if (static_cast<uint64_t>(a->rows) * a->cols > UINT32_MAX) return false;
    if (a->cols % kStreamBlockK != 0 || a->rows % (*pair ? 16 : 32) != 0) return false;
    if (a->tokens < 1 || a->tokens > AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) return false;
    if (!scale_ok(a->global_scale)) return false;
    if (*pair ? !scale_ok(a->global_scale_b) : a->global_scale_b != 0.0f) return false;
    if (a->weight_len_bytes != stream_extent_bytes(*pair, a->rows, a->cols)) return false;
    if (a->input_len_bytes != static_cast<uint64_t>(a->tokens) * a->cols * 2) return false;
    const uint64_t out_elem = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32 ? 4 : 2;
    return a->output_len_bytes == static_cast<uint64_t>(a->tokens) * (a->stored_rows ? a->stored_rows : a->rows) * out_elem;
}

void gemv_ranges(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, Range (&r)[3]) {
    r[0] = {a->weight, a->weight_len_bytes, 256};
    r[1] = {a->input_bf16, a->input_len_bytes, 16};
    r[2] = {a->output, a->output_len_bytes, 4};
}

// `partial_offset`..`partial_limit` is the part of the plan scratch this launch may use: the staged
// activations come first, the partial-sum slots after them.
bool check_gemv(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint64_t partial_offset, uint64_t partial_limit,
                bool full, augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    bool pair = false;
    if (!plan_ok(plan, d, s) || !check_gemv_scalars(a, &pair)) return false;
    const GemvGeometry g = geometry(a->rows, a->cols, pair, plan->sm_count);
    if (g.ctas_per_slab == 0 || g.groups > kMaxGroups || partial_offset < kCounterBytes ||
        partial_limit < partial_offset || g.staged_bytes + g.partial_bytes > partial_limit - partial_offset) {
        return false;
    }
    Range r[4];
    Range base[3];
    gemv_ranges(a, base);
    r[0] = base[0]; r[1] = base[1]; r[2] = base[2];
    r[3] = plan_scratch_range(plan);
    if (!all_disjoint(r, 4)) return false;
    return !full || inspect_device_ranges(d, r, 3, failure);
}

// The tensor-parallel part of a launch: every rank's exchange buffer as mapped here.
struct ExchangeTable {
    const uint64_t* exchange;
    uint32_t world, rank, sequence;
};

// `staged_out_offset` (non-zero): the SwiGLU result is also written, staged, at that offset of the plan
// scratch. `input_is_staged`: the activations were staged there by the producing launch (fixed
// exponent) and are copied in as they are instead of being staged by the kernel.
// Kernel parameters of one linear. `sm_share`: the SMs this linear may fill (all of them, or its share of a grouped grid);
// `counters`: its arrival counters; `staged` / `partials`: where its staged activations are and where its slots go.
GemvParams make_params(const augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t sm_share,
                       uint32_t* counters, const uint8_t* staged, float* partials, bool input_is_staged, uint32_t* ctas) {
    const bool pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    const GemvGeometry g = geometry(a->rows, a->cols, pair, sm_share);
    GemvParams p{};
    p.weight = reinterpret_cast<const uint8_t*>(a->weight);
    p.x = reinterpret_cast<const uint16_t*>(a->input_bf16);
    p.out = reinterpret_cast<void*>(a->output);
    p.counters = counters;
    p.staged = staged;
    p.partials = partials;
    p.unit = g.unit;
    p.fixed_factor = input_is_staged ? 0x1p31f : 0.0f;      // (2^31)^2 = 2^(126 - kFixedStageShift)
    p.status_word = plan->status_word;
    p.groups = g.groups; p.kb_count = g.kb_count; p.slabs = g.slabs; p.ctas_per_slab = g.ctas_per_slab;
    p.max_contrib = g.max_contrib;
    p.rows = a->rows; p.cols = a->cols; p.tokens = a->tokens; p.epilogue = a->epilogue;
    p.store_rows = a->stored_rows ? a->stored_rows : a->rows;
    p.global_a = a->global_scale; p.global_b = a->global_scale_b;
    *ctas = g.slabs * g.ctas_per_slab;
    return p;
}

void launch_gemv(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                 const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t member, uint64_t partial_offset,
                 uint64_t staged_out_offset = 0, bool input_is_staged = false, const ExchangeTable* tp = nullptr) {
    const bool pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    const GemvGeometry g = geometry(a->rows, a->cols, pair, plan->sm_count);
    uint32_t ctas = 0;
    GemvParams p = make_params(plan, a, plan->sm_count, reinterpret_cast<uint32_t*>(plan->scratch + member * kCounterRegionBytes),
                               plan->scratch + partial_offset, reinterpret_cast<float*>(plan->scratch + partial_offset + g.staged_bytes),
                               input_is_staged, &ctas);
    p.staged_out = staged_out_offset ? reinterpret_cast<uint16_t*>(plan->scratch + staged_out_offset) : nullptr;
    if (tp) {
        for (uint32_t r = 0; r < tp->world; ++r) p.exchange[r] = tp->exchange[r];
        p.tp_world = tp->world; p.tp_rank = tp->rank; p.tp_sequence = tp->sequence;
        p.tp_counter = reinterpret_cast<uint32_t*>(tp->exchange[tp->rank] + exchange_tiles_bytes(tp->world, a->rows / 32));
    }
    // Launched with programmatic stream serialisation: the grid may become resident while its
    // predecessor drains, and waits for it in-kernel (griddepcontrol.wait).
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config{};
    config.stream = s->stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    config.gridDim = dim3(g.slabs * g.ctas_per_slab);
    config.blockDim = dim3(kWarps * 32);
    config.dynamicSmemBytes = kGemvSmemBytes;
    cudaLaunchKernelEx(&config, gemv_kernel, p);
    count_launch();
}

}  // namespace

// Called once per device from plan creation (a bind-time call): raises the kernels'
// dynamic shared-memory limit.
cudaError_t gemv_configure_device() {
    const cudaError_t e = cudaFuncSetAttribute(gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemv_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes);
}

}  // namespace augur_sm100

using namespace augur_sm100;

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_scratch_extent_host_v1(
    uint32_t rows, uint32_t cols, uint32_t tokens, uint64_t* out_bytes) {
    if (!out_bytes || !rows || !cols || rows % 16 != 0 || cols % kStreamBlockK != 0 || tokens < 1 ||
        tokens > AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) {
        return invalid();
    }
    // Upper bound over both row groupings and any SM count up to 512.
    uint64_t worst = 0;
    for (uint32_t pair = 0; pair < 2; ++pair) {
        if (!pair && rows % 32 != 0) continue;
        for (uint32_t sms = 1; sms <= 512; ++sms) {
            const GemvGeometry g = geometry(rows, cols, pair != 0, sms);
            if (g.staged_bytes + g.partial_bytes > worst) worst = g.staged_bytes + g.partial_bytes;
        }
    }
    *out_bytes = kCounterBytes + worst;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    return check_gemv(d, s, plan, a, kCounterBytes, plan ? plan->scratch_bytes : 0, true, &failure) ? ok() : failure;
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_gemv(d, s, plan, a, kCounterBytes, plan ? plan->scratch_bytes : 0, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    launch_gemv(s, plan, a, 0, kCounterBytes);
    return submitted();
}

namespace {
// Both members plus every cross alias, before anything is enqueued. The two members use
// separate counter regions and separate halves of the slot area, so their launches may overlap.
bool check_mlp(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
               const augur_cuda_nvfp4_sm100_mlp_args_v1* a, bool full, uint64_t* down_offset,
               augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!plan_ok(plan, d, s)) return false;
    if (plan->scratch_bytes < kCounterBytes) return false;
    const uint64_t middle = kCounterBytes + (plan->scratch_bytes - kCounterBytes) / 2 / 256 * 256;
    *down_offset = middle;
    if (!check_gemv(d, s, plan, &a->gate_up, kCounterBytes, middle, false, failure)) return false;
    if (!check_gemv(d, s, plan, &a->down, middle, plan->scratch_bytes, false, failure)) return false;
    *failure = invalid();
    if (a->gate_up.epilogue != AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 ||
        a->down.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 || a->down.stored_rows) {
        return false;
    }
    // The intermediate is the one shared range: gate_up writes what down reads.
    if (a->down.input_bf16 != a->gate_up.output || a->down.input_len_bytes != a->gate_up.output_len_bytes ||
        a->down.cols != a->gate_up.rows || a->down.tokens != a->gate_up.tokens || a->down.rows != a->gate_up.cols) {
        return false;
    }
    const Range r[6] = {{a->gate_up.weight, a->gate_up.weight_len_bytes, 256},
                        {a->gate_up.input_bf16, a->gate_up.input_len_bytes, 16},
                        {a->gate_up.output, a->gate_up.output_len_bytes, 16},
                        {a->down.weight, a->down.weight_len_bytes, 256},
                        {a->down.output, a->down.output_len_bytes, 4},
                        plan_scratch_range(plan)};
    if (!all_disjoint(r, 6)) return false;
    return !full || inspect_device_ranges(d, r, 5, failure);
}
}  // namespace

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint64_t down_offset = 0;
    return check_mlp(d, s, plan, a, true, &down_offset, &failure) ? ok() : failure;
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint64_t down_offset = 0;
    if (!check_mlp(d, s, plan, a, false, &down_offset, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    // gate|up stages its own input, and its epilogue stages the intermediate where down expects it.
    launch_gemv(s, plan, &a->gate_up, 0, kCounterBytes, down_offset, false);
    augur_cuda_result_v1 first = submitted();
    if (first.status != AUGUR_CUDA_STATUS_OK) return first;
    launch_gemv(s, plan, &a->down, 1, down_offset, 0, true);
    return submitted();
}

// ---- tensor-parallel MLP program -------------------------------------------------------------------
namespace {
static_assert(sizeof(augur_cuda_nvfp4_sm100_mlp_tp_args_v1) == 272, "mlp_tp ABI");

// The exchange buffers of a row-parallel linear `m`: extent, alignment, no two alike, and a grid that is
// resident as a whole (the reduce step polls for tiles that other CTAs of the same grid deliver).
bool exchange_table_ok(const augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1& m,
                       const uint64_t (&exchange)[AUGUR_NVFP4_SM100_MAX_TP_RANKS], uint64_t exchange_len_bytes, uint32_t world) {
    if (exchange_len_bytes < exchange_extent(world, m.rows / 32)) return false;
    const GemvGeometry g = geometry(m.rows, m.cols, false, plan->sm_count);
    if (g.slabs * g.ctas_per_slab > plan->sm_count) return false;
    for (uint32_t r = 0; r < AUGUR_NVFP4_SM100_MAX_TP_RANKS; ++r) {
        if (r >= world) {
            if (exchange[r]) return false;
            continue;
        }
        if (!exchange[r] || exchange[r] % 256 != 0) return false;
        for (uint32_t q = 0; q < r; ++q) {
            if (!disjoint({exchange[r], exchange_len_bytes, 256}, {exchange[q], exchange_len_bytes, 256})) return false;
        }
    }
    return true;
}

bool check_mlp_tp(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                  const augur_cuda_nvfp4_sm100_mlp_tp_args_v1* a, bool full, uint64_t* down_offset,
                  augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    // The two members are checked exactly as a single-GPU program is.
    augur_cuda_nvfp4_sm100_mlp_args_v1 local{};
    local.abi_version = AUGUR_CUDA_ABI_VERSION_V1;
    local.struct_size = sizeof(local);
    local.gate_up = a->gate_up;
    local.down = a->down;
    if (!check_mlp(d, s, plan, &local, full, down_offset, failure)) return false;
    *failure = invalid();
    if (a->reserved || a->world < 1 || a->world > AUGUR_NVFP4_SM100_MAX_TP_RANKS || a->rank >= a->world ||
        a->down.epilogue != AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16) {
        return false;
    }
    if (!exchange_table_ok(plan, a->down, a->exchange, a->exchange_len_bytes, a->world)) return false;
    // This rank's own exchange buffer is local memory like any other range of the program.
    const Range r[7] = {{a->gate_up.weight, a->gate_up.weight_len_bytes, 256},
                        {a->gate_up.input_bf16, a->gate_up.input_len_bytes, 16},
                        {a->gate_up.output, a->gate_up.output_len_bytes, 16},
                        {a->down.weight, a->down.weight_len_bytes, 256},
                        {a->down.output, a->down.output_len_bytes, 4},
                        plan_scratch_range(plan),
                        {a->exchange[a->rank], a->exchange_len_bytes, 256}};
    return all_disjoint(r, 7);
}
}  // namespace

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(
    uint32_t rows, uint32_t world, uint64_t* out_bytes) {
    if (!out_bytes || !rows || rows % 32 != 0 || world < 1 || world > AUGUR_NVFP4_SM100_MAX_TP_RANKS) return invalid();
    *out_bytes = exchange_extent(world, rows / 32);
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tp_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_tp_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint64_t down_offset = 0;
    return check_mlp_tp(d, s, plan, a, true, &down_offset, &failure) ? ok() : failure;
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_tp_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint64_t down_offset = 0;
    if (!check_mlp_tp(d, s, plan, a, false, &down_offset, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    launch_gemv(s, plan, &a->gate_up, 0, kCounterBytes, down_offset, false);
    augur_cuda_result_v1 first = submitted();
    if (first.status != AUGUR_CUDA_STATUS_OK) return first;
    const ExchangeTable table{a->exchange, a->world, a->rank, a->sequence};
    launch_gemv(s, plan, &a->down, 1, down_offset, 0, true, &table);
    return submitted();
}

// ---- a single row-parallel linear with the exchange ------------------------------------------------
namespace {
static_assert(sizeof(augur_cuda_nvfp4_sm100_gemv_tp_args_v1) == 184, "gemv_tp ABI");

bool check_gemv_tp(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                   const augur_cuda_nvfp4_sm100_gemv_tp_args_v1* a, bool full, augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!check_gemv(d, s, plan, &a->linear, kCounterBytes, plan ? plan->scratch_bytes : 0, full, failure)) return false;
    *failure = invalid();
    if (a->reserved || a->world < 1 || a->world > AUGUR_NVFP4_SM100_MAX_TP_RANKS || a->rank >= a->world ||
        a->linear.epilogue != AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16 || a->linear.stored_rows) {
        return false;
    }
    if (!exchange_table_ok(plan, a->linear, a->exchange, a->exchange_len_bytes, a->world)) return false;
    const Range r[5] = {{a->linear.weight, a->linear.weight_len_bytes, 256},
                        {a->linear.input_bf16, a->linear.input_len_bytes, 16},
                        {a->linear.output, a->linear.output_len_bytes, 4},
                        plan_scratch_range(plan),
                        {a->exchange[a->rank], a->exchange_len_bytes, 256}};
    return all_disjoint(r, 5);
}
}  // namespace

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tp_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_tp_args_v1* a) {
    augur_cuda_result_v1 failure;
    return check_gemv_tp(d, s, plan, a, true, &failure) ? ok() : failure;
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tp_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_tp_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_gemv_tp(d, s, plan, a, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    const ExchangeTable table{a->exchange, a->world, a->rank, a->sequence};
    launch_gemv(s, plan, &a->linear, 0, kCounterBytes, 0, false, &table);
    return submitted();
}

// ---- norm group: [residual add] -> RMSNorm -> BF16 stage -> up to four small-token projections ----------------
// The B200 counterpart of the reference's fused norm stage and grouped projections
// (crates/augur-cuda-sys/native/augur_qwen35_gdn_input_b8.cuh:19-49,92 ff.): one validated program,
// 1 + count launches chained by programmatic stream serialisation.
namespace augur_sm100 {
namespace {
static_assert(sizeof(augur_cuda_nvfp4_sm100_norm_group_args_v1) == 472, "norm_group ABI");

constexpr uint32_t kNormThreads = 256;
constexpr uint32_t kNormHeld = 24;       // columns of a row that one thread keeps in registers (rows up to 6144 wide)

// One CTA per token row. The arithmetic order is the reference kernel's, so that the F32 output is
// reproducible on a CPU: lane l accumulates value * value over columns l, l + 256, ... (multiply and
// add, never fused), the 256 partial sums are folded by halving strides, y = (value * scale) * weight.
// scale = 1 / sqrt(mean + epsilon) with correctly rounded operations (the reference's rsqrtf is a
// hardware approximation); the staged copy is BF16.
__global__ void __launch_bounds__(kNormThreads) norm_stage_kernel(const float* __restrict__ add_a, const float* __restrict__ add_b,
                                                                   float* __restrict__ input, const float* __restrict__ weight,
                                                                   float* __restrict__ output, __nv_bfloat16* __restrict__ staged,
                                                                   uint16_t* __restrict__ fragments, uint32_t cols, float epsilon,
                                                                   uint32_t residual) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the inputs may come from the launch before this one
    __shared__ float partial[kNormThreads];
    const uint32_t lane = threadIdx.x;
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * cols;
    // A row of up to 256 * kNormHeld columns is held in registers: all of a thread's loads are in flight at once
    // (each is a round trip to L2), and the second pass reads nothing but the weights, which are fetched with them.
    // The arithmetic and its order are the same on both paths.
    const bool held_row = cols <= kNormThreads * kNormHeld;
    float held[kNormHeld], gain[kNormHeld];
    float sum = 0.0f;
    if (held_row) {
        float other[kNormHeld];
#pragma unroll
        for (uint32_t i = 0; i < kNormHeld; ++i) {
            const uint32_t col = lane + i * kNormThreads;
            held[i] = gain[i] = other[i] = 0.0f;
            if (col < cols) {
                held[i] = residual ? __ldcg(add_a + base + col) : __ldcg(input + base + col);
                if (residual) other[i] = __ldcg(add_b + base + col);
                gain[i] = __ldg(weight + col);
            }
        }
#pragma unroll
        for (uint32_t i = 0; i < kNormHeld; ++i) {
            const uint32_t col = lane + i * kNormThreads;
            if (col < cols) {
                if (residual) {
                    held[i] = __fadd_rn(held[i], other[i]);
                    input[base + col] = held[i];
                }
                sum = __fadd_rn(sum, __fmul_rn(held[i], held[i]));
            }
        }
    } else {
        for (uint32_t col = lane; col < cols; col += kNormThreads) {
            float value;
            if (residual) {
                value = __fadd_rn(__ldcg(add_a + base + col), __ldcg(add_b + base + col));
                input[base + col] = value;
            } else {
                value = __ldcg(input + base + col);
            }
            sum = __fadd_rn(sum, __fmul_rn(value, value));
        }
    }
    partial[lane] = sum;
    __syncthreads();
    for (uint32_t stride = kNormThreads / 2; stride != 0; stride >>= 1) {
        if (lane < stride) partial[lane] = __fadd_rn(partial[lane], partial[lane + stride]);
        __syncthreads();
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial[0], static_cast<float>(cols)), epsilon)));
    auto emit = [&](uint32_t col, float value, float w) {
        const float y = __fmul_rn(__fmul_rn(value, scale), w);
        output[base + col] = y;
        const __nv_bfloat16 rounded = __float2bfloat16_rn(y);
        staged[base + col] = rounded;
        // The same value where the grouped projections read it: their MMA B fragments, shifted by the fixed
        // staging exponent (k-step = col / 16, fragment register (col % 16) / 8, pair (col % 8) / 2, half col % 2),
        // so that none of them has to stage the activations for itself.
        const uint32_t kstep = col >> 4, inner = col & 15;
        const uint32_t word = ((kstep >> 1) * 32 + blockIdx.x * 4 + ((inner & 7) >> 1)) * 4 + (kstep & 1) * 2 + (inner >> 3);
        fragments[word * 2 + (inner & 1)] = static_cast<uint16_t>(shift_bf16(__bfloat16_as_ushort(rounded), kFixedStageShift));
    };
    if (held_row) {
#pragma unroll
        for (uint32_t i = 0; i < kNormHeld; ++i) {
            const uint32_t col = lane + i * kNormThreads;
            if (col < cols) emit(col, held[i], gain[i]);
        }
    } else {
        // this thread wrote input[base + col] itself when there is a residual
        for (uint32_t col = lane; col < cols; col += kNormThreads) emit(col, input[base + col], __ldg(weight + col));
    }
}

// The members of a norm group run as ONE grid: the SMs are dealt out in proportion to the members' weight rows
// (every member at least one), the staged activations sit once behind the counter regions, the members'
// partial-sum slots follow side by side, and members 0/1 and 2/3 share a counter region by halves.
struct GroupLayout {
    uint32_t share[kMaxGroupMembers];
    uint64_t staged_offset, partial_offset[kMaxGroupMembers], end;
};
GroupLayout group_layout(const augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_norm_group_args_v1* a) {
    GroupLayout layout{};
    uint64_t total_rows = 0;
    for (uint32_t i = 0; i < a->count; ++i) total_rows += a->projections[i].rows;
    uint32_t dealt = 0;
    for (uint32_t i = 0; i < a->count; ++i) {
        const uint64_t fair = static_cast<uint64_t>(plan->sm_count) * a->projections[i].rows / (total_rows ? total_rows : 1);
        layout.share[i] = fair ? static_cast<uint32_t>(fair) : 1;
        dealt += layout.share[i];
    }
    // what rounding down left over goes to the largest member; what the minimum of one took too much comes off it
    uint32_t largest = 0;
    for (uint32_t i = 1; i < a->count; ++i) {
        if (a->projections[i].rows > a->projections[largest].rows) largest = i;
    }
    if (dealt < plan->sm_count) layout.share[largest] += plan->sm_count - dealt;
    if (dealt > plan->sm_count && layout.share[largest] > dealt - plan->sm_count) layout.share[largest] -= dealt - plan->sm_count;
    layout.staged_offset = kCounterBytes;
    uint64_t at = kCounterBytes + (static_cast<uint64_t>(a->cols) * 16 + 255) / 256 * 256;
    for (uint32_t i = 0; i < a->count; ++i) {
        layout.partial_offset[i] = at;
        const GemvGeometry g = geometry(a->projections[i].rows, a->projections[i].cols, false, layout.share[i]);
        at += (g.partial_bytes + 255) / 256 * 256;
    }
    layout.end = at;
    return layout;
}

bool check_norm_group(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                      const augur_cuda_nvfp4_sm100_norm_group_args_v1* a, bool full, augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!plan_ok(plan, d, s) || plan->scratch_bytes < kCounterBytes) return false;
    if (a->reserved || a->residual > 1 || a->count < 1 || a->count > 4 || a->tokens < 1 ||
        a->tokens > AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS || !a->cols || a->cols % kNormThreads != 0 || a->cols > INT_MAX ||
        !std::isfinite(a->epsilon) || a->epsilon < 0.0f) {
        return false;
    }
    const uint64_t elements = static_cast<uint64_t>(a->tokens) * a->cols;
    if (a->input_len_bytes != elements * 4 || a->output_len_bytes != elements * 4 || a->staged_len_bytes != elements * 2 ||
        a->weight_len_bytes != static_cast<uint64_t>(a->cols) * 4) {
        return false;
    }
    Range r[16];
    size_t n = 0;
    r[n++] = {a->input_f32, a->input_len_bytes, 16};
    r[n++] = {a->weight_f32, a->weight_len_bytes, 4};
    r[n++] = {a->output_f32, a->output_len_bytes, 16};
    r[n++] = {a->staged_bf16, a->staged_len_bytes, 16};
    if (a->residual) {
        if (a->add_len_bytes != a->input_len_bytes) return false;
        r[n++] = {a->add_a, a->add_len_bytes, 16};
        r[n++] = {a->add_b, a->add_len_bytes, 16};
    } else if (a->add_a || a->add_b || a->add_len_bytes) {
        return false;
    }
    for (uint32_t i = 0; i < 4; ++i) {
        const augur_cuda_nvfp4_sm100_gemv_args_v1& m = a->projections[i];
        if (i >= a->count) {
            // unused members are all zero
            const uint8_t* bytes = reinterpret_cast<const uint8_t*>(&m);
            for (size_t k = 0; k < sizeof(m); ++k) {
                if (bytes[k]) return false;
            }
            continue;
        }
        // each member exactly as a stand-alone small-token linear
        if (!check_gemv(d, s, plan, &m, kCounterBytes, plan->scratch_bytes, false, failure)) return false;
        *failure = invalid();
        if (m.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 || m.input_bf16 != a->staged_bf16 ||
            m.input_len_bytes != a->staged_len_bytes || m.tokens != a->tokens || m.cols != a->cols ||
            m.rows / 32 > kMaxGroups / 2) {   // two members share a counter region
            return false;
        }
        r[n++] = {m.weight, m.weight_len_bytes, 256};
        r[n++] = {m.output, m.output_len_bytes, 4};
    }
    r[n++] = plan_scratch_range(plan);
    if (!all_disjoint(r, n)) return false;
    // the grouped grid: staged activations once, then every member's slots side by side
    const GroupLayout layout = group_layout(plan, a);
    if (layout.end > plan->scratch_bytes) return false;
    return !full || inspect_device_ranges(d, r, n - 1, failure);
}
}  // namespace
}  // namespace augur_sm100

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_norm_group_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_norm_group_args_v1* a) {
    augur_cuda_result_v1 failure;
    return check_norm_group(d, s, plan, a, true, &failure) ? ok() : failure;
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_norm_group_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_norm_group_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_norm_group(d, s, plan, a, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config{};
    config.stream = s->stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    config.gridDim = dim3(a->tokens);
    config.blockDim = dim3(kNormThreads);
    const GroupLayout layout = group_layout(plan, a);
    cudaLaunchKernelEx(&config, norm_stage_kernel, reinterpret_cast<const float*>(a->add_a), reinterpret_cast<const float*>(a->add_b),
                       reinterpret_cast<float*>(a->input_f32), reinterpret_cast<const float*>(a->weight_f32),
                       reinterpret_cast<float*>(a->output_f32), reinterpret_cast<__nv_bfloat16*>(a->staged_bf16),
                       reinterpret_cast<uint16_t*>(plan->scratch + layout.staged_offset), a->cols, a->epsilon, a->residual);
    count_launch();
    augur_cuda_result_v1 result = submitted();
    if (result.status != AUGUR_CUDA_STATUS_OK) return result;
    // all projections of the group in one grid; they copy the staged fragments in and stage nothing themselves
    GemvGroupParams group{};
    uint32_t next = 0;
    for (uint32_t i = 0; i < kMaxGroupMembers; ++i) {
        group.first_cta[i] = next;
        if (i >= a->count) continue;
        uint32_t ctas = 0;
        uint32_t* counters = reinterpret_cast<uint32_t*>(plan->scratch + (i / 2) * kCounterRegionBytes + (i % 2) * (kCounterRegionBytes / 2));
        group.member[i] = make_params(plan, &a->projections[i], layout.share[i], counters, plan->scratch + layout.staged_offset,
                                      reinterpret_cast<float*>(plan->scratch + layout.partial_offset[i]), true, &ctas);
        next += ctas;
    }
    group.first_cta[kMaxGroupMembers] = next;
    for (uint32_t i = a->count; i < kMaxGroupMembers; ++i) group.first_cta[i] = next;   // members that do not exist own no CTA
    config.gridDim = dim3(next);
    config.blockDim = dim3(kWarps * 32);
    config.dynamicSmemBytes = kGemvSmemBytes;
    cudaLaunchKernelEx(&config, gemv_group_kernel, group);
    count_launch();
    return submitted();
}

// ---- one entry point that allocates nothing -------------------------------------------------
// Plan creation calls cudaMalloc. A host that gave every byte of device memory to its own arena
// at start-up, or that runs its serving loop under a no-allocation rule and audits it, cannot
// create a plan once it is running. For such callers the small-token linear is also offered
// with its scratch in this fixed array, which every GPU that loads the library carries from
// load to exit.
namespace {
static __device__ __align__(256) uint8_t g_static_scratch[AUGUR_NVFP4_SM100_STATIC_SCRATCH_BYTES];

struct StaticScratchDevice {
    bool ready = false;
    uint8_t* address = nullptr;   // device address of g_static_scratch on this device
    uint32_t sm_count = 0;
};
StaticScratchDevice g_static_devices[64];
std::mutex g_static_mutex;

// Once per device, with that device current: the array's name is only a host-side handle, the
// kernels need the address the runtime reports for it.
cudaError_t static_scratch_setup(int32_t ordinal, StaticScratchDevice** out) {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticScratchDevice& device = g_static_devices[ordinal];
    if (!device.ready) {
        int major = 0, sms = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal);
        if (e != cudaSuccess) return e;
        if (major != 10) {   // the image holds sm_100a code only; the array does not exist elsewhere
            *out = nullptr;
            return cudaSuccess;
        }
        void* address = nullptr;
        e = cudaGetSymbolAddress(&address, g_static_scratch);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal);
        if (e != cudaSuccess) return e;
        e = gemv_configure_device();
        if (e != cudaSuccess) return e;
        device.address = static_cast<uint8_t*>(address);
        device.sm_count = static_cast<uint32_t>(sms);
        device.ready = true;
    }
    *out = &device;
    return cudaSuccess;
}
}  // namespace

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    if (d < 0 || d >= 64 || !s || s->ordinal != d || !a) return invalid();
    cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    StaticScratchDevice* device = nullptr;
    e = static_scratch_setup(d, &device);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    if (!device) return make_result(AUGUR_CUDA_STATUS_UNSUPPORTED_DEVICE);
    // A plan-shaped view of the fixed array: status word in front, then the same layout a plan has.
    augur_cuda_nvfp4_sm100_plan_v1 view{};
    view.magic = kPlanMagic;
    view.ordinal = d;
    view.owner = s;
    view.owner_stream = s->stream;
    view.status_word = reinterpret_cast<uint32_t*>(device->address);
    view.scratch = device->address + kPlanHeaderBytes;
    view.scratch_bytes = AUGUR_NVFP4_SM100_STATIC_SCRATCH_BYTES - kPlanHeaderBytes - kPlanTrailerBytes;   // the range a plan claims ends with a trailer
    view.sm_count = device->sm_count;
    // The same checks as the plan-based submit; a shape whose scratch need exceeds the fixed
    // array fails here with INVALID_ARGUMENT before anything is enqueued.
    augur_cuda_result_v1 failure;
    if (!check_gemv(d, s, &view, a, kCounterBytes, view.scratch_bytes, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    // The array keeps whatever the last call left. Arrival counters must read zero when the
    // kernel starts, so they are cleared on the caller's stream first (a memset, not an allocation).
    const bool pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    const uint32_t groups = pair ? a->rows / 16 : a->rows / 32;
    e = cudaMemsetAsync(view.scratch, 0, static_cast<size_t>(groups) * 4, s->stream);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_SUBMISSION_FAILURE, e);
    launch_gemv(s, &view, a, 0, kCounterBytes);
    return submitted();
}

// The status word of the fixed array (its first four bytes), for the entry above: what
// plan_device_status_v1 is to a plan. Copies the word back on `s` and waits for the stream; a
// non-zero word is then set back to zero (a memset on the same stream), so every give-up is
// reported once. Like the submit entry it allocates nothing.
extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_static_scratch_status_v1(
    int32_t d, augur_cuda_stream_t s, uint32_t* out_status) {
    if (d < 0 || d >= 64 || !s || s->ordinal != d || !out_status) return invalid();
    cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    StaticScratchDevice* device = nullptr;
    e = static_scratch_setup(d, &device);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    if (!device) return make_result(AUGUR_CUDA_STATUS_UNSUPPORTED_DEVICE);
    e = cudaMemcpyAsync(out_status, device->address, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->stream);
    if (e == cudaSuccess && *out_status != 0) e = cudaMemsetAsync(device->address, 0, sizeof(uint32_t), s->stream);
    return e == cudaSuccess ? ok() : make_result(AUGUR_CUDA_STATUS_COMPLETION_FAILURE, e);
}
