// Small-token (1..8) NVFP4 linear and MLP block for sm_100a on the tensor-memory path: the weights go from HBM to
// the tensor cores without a single per-element instruction on the SMs, and a whole MLP block is ONE launch in
// which the weight stream never stops.
//
//   weights      TCGEN05 layout (codes K-major as in the checkpoint, block scales in 512-byte atoms), the
//                128-row operand of tcgen05.mma kind::mxf4nvf4: TMA brings 128 rows x 256 k (16 KB of codes
//                plus 2 KB of scales) per stage into a ring in shared memory, tcgen05.cp moves the scales on
//                to tensor memory, the MMA reads the codes where the TMA put them;
//   activations  BF16 in global memory. A block-scaled FP4 MMA wants FP4 on both sides, so the launch first
//                splits them - every CTA a slice, once - into kTerms NVFP4 terms: the digits of the value in
//                radix 8 (digits -4..4, i.e. the E2M1 levels 0, 0.5, .., 2 with a sign), all scales powers of
//                two. The terms sit side by side on the MMA n dimension (column = term * 8 + token); their
//                codes and block scales (10 KB per 256 k, L2-resident) ride along with every weight stage.
//                Eight digits hold a BF16 value exactly when it is within 2^-15 of its group's largest magnitude
//                and to 2^-24 of that magnitude otherwise; one MMA per 64 k covers all tokens and all terms;
//   accumulator  128 weight rows x 64 columns of f32 in tensor memory, two buffers; the epilogue warps add
//                the terms of a token with their scales and finish the rows.
//
// A launch runs one phase (a linear) or two (gate|up with SiLU(gate) * up, then down, whose activations are the
// first phase's output). Per phase a CTA owns whole 128-row tiles over the whole k range whenever there are at
// least as many tiles as resident CTAs (two per SM); otherwise every tile is cut along k into equal parts, one
// per CTA: partial sums go to plan scratch with an arrival counter per 32 rows, and the last arriver adds them in
// part order and finishes the rows. Results are bit-reproducible.
//
// Roles of a CTA: one thread streams the weight stages of all its work, both phases back to back, and keeps
// doing so while activations are not ready yet (the ring buffers that time); one thread copies block scales to
// tensor memory; one issues the MMAs; four warps split activations and run the epilogues. The split needs
// every CTA's slice before any CTA can use it, and the second phase needs every CTA's output of the first:
// the grid meets in global memory (all CTAs are resident: the grid never exceeds two CTAs per SM), once in
// the first phase and twice at the phase boundary.
//
// Every wait is bounded; a wait that runs out records a code in the plan's status word, raises a CTA-wide abort
// flag, and all roles fall through to the common exit where tensor memory is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "nvfp4_internal.h"
#include "nvfp4_layout.cuh"
#include "nvfp4_tc.cuh"

namespace augur_sm100 {
namespace {
using namespace tc;

constexpr uint32_t kTerms = 8;                         // radix-8 digits of the activation split
constexpr uint32_t kCols = 8 * kTerms;                 // MMA n: column = term * 8 + token
constexpr uint32_t kStageK = 256;                      // k per ring stage = one 128-byte swizzled row of codes
constexpr uint32_t kStageCodeBytes = kTileM * 128;     // 16 KB of weight codes
constexpr uint32_t kStageSfBytes = 4 * kSfAtomBytes;   // 2 KB: the 4 scale atoms of a stage (weights; activations alike)
constexpr uint32_t kChunkBytes = kCols * 128;          // 8 KB: activation codes of one 256-k chunk, 64 rows x 128 bytes
constexpr uint32_t kStageActCodes = kStageCodeBytes + kStageSfBytes;        // offsets inside a stage
constexpr uint32_t kStageActSf = kStageActCodes + kChunkBytes;
constexpr uint32_t kStageBytes = kStageActSf + kStageSfBytes;               // 28 KB
constexpr uint32_t kStages = 4;                        // per CTA; two CTAs share an SM
constexpr uint32_t kThreads = 224;                     // warp 0 TMA, warp 1 MMA, warps 2..5 split and epilogue, warp 6 scale copies
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 512 /*small state*/;   // the stages start the (1024-byte aligned) window
constexpr uint32_t kCtasPerSm = 2;                     // half of an SM's shared and tensor memory each: a CTA of the next launch
                                                       // moves in (and fills its ring) as soon as one of this launch leaves
constexpr uint32_t kTmemAcc = 0;                       // two accumulators of 64 columns
constexpr uint32_t kTmemSfWeight = 128;                // 16 columns per ring stage
constexpr uint32_t kTmemSfAct = kTmemSfWeight + kStages * 16;
constexpr uint32_t kTmemColumns = 256;
static_assert(kTmemSfAct + kStages * 16 <= kTmemColumns, "tensor memory columns");
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM, a kilobyte each reserved by the system");
static_assert(kTerms == 8, "the digit transposition is 8 lanes x 8 nibbles");
static_assert(kStageBytes % 1024 == 0 && kStageActCodes % 1024 == 0, "swizzled operand tiles are 1024-byte aligned");
constexpr uint32_t kSlotFloats = 256;                  // one partial: 32 rows x 8 tokens
constexpr uint32_t kWorkers = 128;                     // the four split / epilogue warps
constexpr uint32_t kMaxPhases = 2;
constexpr uint32_t kGridWaitLimit = 1u << 22;          // polls of the grid barrier (a fraction of a microsecond each) before giving up

constexpr uint32_t kErrTcProducer = 0x301, kErrTcFull = 0x302, kErrTcAccEmpty = 0x303, kErrTcAccFull = 0x304,
                   kErrTcScalesLanded = 0x305, kErrTcScalesReady = 0x306, kErrTcGridBarrier = 0x307, kErrTcWindow = 0x308;
constexpr uint32_t kHeld = 4;                          // elements a lane keeps in registers between the scan and the split


// The split activations in global memory (plan scratch): the image the ring stages want, chunk by chunk.
//   [chunk = k / 256][64 rows][128 bytes]   codes, rows already in the 128-byte swizzle of a shared-memory operand tile
//   [k / 64][512 bytes]                     block-scale atoms (row n at byte (n % 32) * 16 + (n / 32) * 4 + (k / 16) % 4)
__host__ __device__ constexpr uint64_t split_code_bytes(uint32_t cols) { return static_cast<uint64_t>((cols + kStageK - 1) / kStageK) * kChunkBytes; }
__host__ __device__ constexpr uint64_t split_sf_bytes(uint32_t cols) { return static_cast<uint64_t>((cols + kStageK - 1) / kStageK) * kStageSfBytes; }
__host__ __device__ constexpr uint64_t split_bytes(uint32_t cols) { return split_code_bytes(cols) + split_sf_bytes(cols); }

struct TcPhase {
    const uint8_t* weight_sf;     // scale region of the weight
    const uint16_t* x;            // [tokens][cols] BF16 (second phase: what the first phase wrote)
    uint8_t* split;               // the split activations (layout above)
    void* out;
    float* partials;              // [tile * 4 + quadrant][part][32 rows][8 tokens]
    uint32_t* counters;           // [tile * 4 + quadrant], zero between launches
    uint32_t* row_max;            // [token] bits of the row's largest magnitude, zero between launches
    uint32_t* collect;            // SwiGLU epilogue: the next phase's row_max, or null
    uint32_t rows;                // physical weight rows (SwiGLU: gate and up interleaved by 16)
    uint32_t out_rows;            // output width
    uint32_t cols, epilogue;
    uint32_t tiles, k_blocks, parts;   // `parts` equal k ranges per tile (1: whole tiles)
    uint32_t scan;                // this launch finds row_max itself (else the phase before collected it)
    float global_a, global_b;
};

struct TcParams {
    TcPhase phase[kMaxPhases];
    uint32_t phases, tokens;
    uint32_t* grid_barrier;       // {three arrival counters used in turn, index of the next meeting modulo 3}
    uint32_t* status_word;
};

__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// All CTAs of the grid meet (the four worker warps of each; thread `leader` speaks for its CTA). Everything the
// workers wrote before is visible to every CTA's workers after. Returns false if the wait ran out.
// Meeting number m (counted over all launches of the plan, modulo 3, in `meeting`) uses counter m % 3: one
// release-add per CTA, then acquire-loads until all have arrived. The last arriver clears counter (m - 1) % 3,
// which every CTA has stopped reading (all are at meeting m) and which is not used again before meeting m + 2;
// nobody gets to meeting m + 2 before the last arriver of m, its store behind it, has arrived at m + 1.
__device__ __forceinline__ bool grid_meet(const TcParams& p, bool leader, uint32_t& meeting, volatile uint32_t* abort_flag) {
    workers_sync();
    if (leader) {
        uint32_t* mine = p.grid_barrier + meeting;
        uint32_t arrived;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(mine) : "memory");
        if (arrived + 1 == gridDim.x) {
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.grid_barrier + (meeting + 2) % 3), "r"(0u) : "memory");
        } else {
            uint32_t spin = 0, seen;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
                if (seen >= gridDim.x) break;
                if (++spin > kGridWaitLimit || ((spin & 255u) == 255u && *abort_flag)) {
                    *abort_flag = 1;
                    atomicCAS(p.status_word, 0u, kErrTcGridBarrier);
                    break;
                }
            }
        }
    }
    meeting = (meeting + 1) % 3;
    workers_sync();
    return *abort_flag == 0;
}

// ---- activation split (the four worker warps of every CTA; the grid's worker warps share the groups out) ----
// One lane per element, sixteen neighbouring lanes per 16-element group; warp w of the grid's W worker warps
// takes the group pairs w, w + W, ... With A the exponent field of the token row's largest magnitude and G that
// of the group's, the group's block scale is 2^q, q = G + 8 - A (the row's largest group gets 2^8; E4M3 holds
// powers of two down to 2^-9, smaller groups keep 2^-9 and lose low bits), term t has the global scale
// 2^(A - 135) * 8^-t, and the element is the integer I = |x| / 2^(q + A - 157): at most 255 * 2^15 for the
// group's largest element, exact for every element within 2^-15 of it, rounded to nearest below. I is written
// in radix 8 with digits -4..4 (from the low end: a digit above 4 becomes digit - 8 and carries), digit t being
// the code of term t: level |digit| / 2, sign of digit times sign of x. Eight digits reach 4 * (8^8 - 1) / 7
// > 255 * 2^15. The eight lanes of a half group transpose their digits so that lane t holds the eight codes of
// term t as one word, and store one word each.
__device__ __forceinline__ uint32_t load_element(const TcPhase& ph, uint32_t tokens, uint32_t group_index, uint32_t lane) {
    const uint32_t groups_per_row = ph.cols / 16;
    if (group_index >= tokens * groups_per_row) return 0;
    return __ldcg(ph.x + static_cast<uint64_t>(group_index) * 16 + (lane & 15));   // rows are contiguous: [tokens][cols]
}

__device__ __forceinline__ void split_group(const TcPhase& ph, uint32_t tokens, const uint32_t* anchor, uint32_t group_index, uint32_t bits,
                                            uint32_t lane) {
    const uint32_t groups_per_row = ph.cols / 16;
    const bool active = group_index < tokens * groups_per_row;
    const uint32_t token = active ? group_index / groups_per_row : 0, group = active ? group_index - token * groups_per_row : 0;
    const uint32_t magnitude = bits & 0x7fffu, negative = (bits >> 15) & 1u;
    uint32_t largest = max(magnitude, __shfl_xor_sync(0xffffffffu, magnitude, 8));
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 4));
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 2));
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 1));
    const int a = static_cast<int>(anchor[token]);
    const int g = max(static_cast<int>(largest >> 7), 1);           // a subnormal has the exponent of field 1
    const int q = min(max(g + 8 - a, -9), 8);
    const uint32_t scale_code = q >= -6 ? static_cast<uint32_t>(q + 7) << 3 : 1u << (q + 9);
    const uint32_t field = magnitude >> 7;
    const uint32_t significand = field ? 128u + (magnitude & 127u) : magnitude;
    // |x| = significand * 2^(max(field, 1) - 134); I = |x| * 2^(157 - q - A)
    const int shift = min(max(static_cast<int>(max(field, 1u)) + 23 - a - q, -16), 15);
    uint32_t value = shift >= 0 ? significand << shift : (significand + (1u << (-shift - 1))) >> -shift;
    uint32_t digits = 0;    // code of term t in bits 4t .. 4t + 3
#pragma unroll
    for (int term = static_cast<int>(kTerms) - 1; term >= 0; --term) {
        const uint32_t low = value & 7u;
        const uint32_t carry = low > 4u ? 1u : 0u;
        const uint32_t level = carry ? 8u - low : low;
        value = (value >> 3) + carry;
        digits |= (level | ((level ? (carry ^ negative) : 0u) << 3)) << (4 * term);
    }
    // 8 lanes x 8 nibbles, transposed: lane t of the eight ends up with nibble t of all eight, in lane order
    uint32_t other = __shfl_xor_sync(0xffffffffu, digits, 4);
    digits = (lane & 4) ? (other >> 16) | (digits & 0xffff0000u) : (digits & 0x0000ffffu) | (other << 16);
    other = __shfl_xor_sync(0xffffffffu, digits, 2);
    digits = (lane & 2) ? ((other & 0xff00ff00u) >> 8) | (digits & 0xff00ff00u) : (digits & 0x00ff00ffu) | ((other & 0x00ff00ffu) << 8);
    other = __shfl_xor_sync(0xffffffffu, digits, 1);
    digits = (lane & 1) ? ((other & 0xf0f0f0f0u) >> 4) | (digits & 0xf0f0f0f0u) : (digits & 0x0f0f0f0fu) | ((other & 0x0f0f0f0fu) << 4);
    if (active) {
        const uint32_t n = (lane & 7) * 8 + token, chunk = group >> 4, unit = (group & 15) >> 1, half = group & 1;
        uint8_t* codes = ph.split + static_cast<uint64_t>(chunk) * kChunkBytes + (n >> 3) * 1024 + (n & 7) * 128 + ((unit ^ (n & 7)) << 4);
        *reinterpret_cast<uint32_t*>(codes + half * 8 + ((lane >> 3) & 1) * 4) = digits;
        if ((lane & 8) == 0) {
            uint8_t* sf = ph.split + split_code_bytes(ph.cols) + static_cast<uint64_t>(group >> 2) * kSfAtomBytes + (group & 3);
            sf[(n & 31) * 16 + (n >> 5) * 4] = static_cast<uint8_t>(scale_code);
        }
    }
}

// Finished sums of 32 weight rows (lane = row) for the 8 tokens: scale, activation, rounding, store.
__device__ __forceinline__ void finish_rows(const TcPhase& ph, uint32_t tokens, uint32_t tile, uint32_t quadrant, uint32_t lane,
                                            const float (&y)[8], uint32_t* collected) {
    if (ph.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
        // 32 physical rows = 16 gate rows (lanes 0..15) and the matching 16 up rows (lanes 16..31)
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(ph.out);
        const uint32_t index = (tile * kTileM + quadrant * 32) / 2 + (lane & 15);
#pragma unroll
        for (uint32_t token = 0; token < 8; ++token) {
            const float up = __shfl_sync(0xffffffffu, y[token], (lane & 15) + 16) * ph.global_b;
            const float gate = y[token] * ph.global_a;
            uint32_t magnitude = 0;
            if (lane < 16 && token < tokens) {
                const __nv_bfloat16 h = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                out[static_cast<uint64_t>(token) * ph.out_rows + index] = h;
                magnitude = static_cast<uint32_t>(__bfloat16_as_ushort(h) & 0x7fffu) << 16;
            }
            if (ph.collect) {
                // the next phase splits these values: it needs every token row's largest magnitude
                magnitude = __reduce_max_sync(0xffffffffu, magnitude);
                if (lane == 0 && magnitude) atomicMax(&collected[token], magnitude);
            }
        }
        return;
    }
    const uint32_t row = tile * kTileM + quadrant * 32 + lane;
#pragma unroll
    for (uint32_t token = 0; token < 8; ++token) {
        if (token < tokens) {
            const float value = y[token] * ph.global_a;
            if (ph.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) {
                static_cast<float*>(ph.out)[static_cast<uint64_t>(token) * ph.out_rows + row] = value;
            } else {
                static_cast<__nv_bfloat16*>(ph.out)[static_cast<uint64_t>(token) * ph.out_rows + row] = __float2bfloat16_rn(value);
            }
        }
    }
}

// This CTA's share of 32 rows of `tile`: finished here if tiles are whole, else handed over; the last of the
// `parts` arrivals adds all shares in part order. Whole warps call this.
__device__ __forceinline__ void contribute_rows(const TcPhase& ph, uint32_t tokens, uint32_t tile, uint32_t quadrant, uint32_t part,
                                                uint32_t lane, const float (&y)[8], uint32_t* collected) {
    if (ph.parts == 1) {
        finish_rows(ph, tokens, tile, quadrant, lane, y, collected);
        return;
    }
    const uint32_t group = tile * 4 + quadrant;
    float* slots = ph.partials + static_cast<uint64_t>(group) * ph.parts * kSlotFloats;
    float4* mine = reinterpret_cast<float4*>(slots + static_cast<uint64_t>(part) * kSlotFloats) + lane * 2;
    mine[0] = make_float4(y[0], y[1], y[2], y[3]);
    mine[1] = make_float4(y[4], y[5], y[6], y[7]);
    __threadfence();
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(&ph.counters[group], 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived + 1 != ph.parts) return;
    __threadfence();
    float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t s0 = 0; s0 < ph.parts; s0 += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            a[j] = b[j] = make_float4(0, 0, 0, 0);
            if (s0 + j < ph.parts) {
                const float4* slot = reinterpret_cast<const float4*>(slots + static_cast<uint64_t>(s0 + j) * kSlotFloats) + lane * 2;
                a[j] = __ldcg(slot);
                b[j] = __ldcg(slot + 1);
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            if (s0 + j < ph.parts) {
                sum[0] += a[j].x; sum[1] += a[j].y; sum[2] += a[j].z; sum[3] += a[j].w;
                sum[4] += b[j].x; sum[5] += b[j].y; sum[6] += b[j].z; sum[7] += b[j].w;
            }
        }
    }
    finish_rows(ph, tokens, tile, quadrant, lane, sum, collected);
    if (lane == 0) ph.counters[group] = 0;   // clean for the next launch
}

// A CTA's ring stages in the order it streams them: over the phases, over its (tile, part) items blockIdx.x,
// blockIdx.x + gridDim.x, ... of a phase, over the k blocks of an item.
struct Cursor {
    uint32_t phase, index, tile, part, kb, kb0, kb1;
};
__device__ __forceinline__ bool cursor_load(const TcParams& p, Cursor& c) {
    while (c.phase < p.phases) {
        const TcPhase& ph = p.phase[c.phase];
        const uint32_t item = blockIdx.x + c.index * gridDim.x;
        if (item < ph.tiles * ph.parts) {
            c.tile = item / ph.parts;
            c.part = item - c.tile * ph.parts;
            c.kb0 = c.part * ph.k_blocks / ph.parts;
            c.kb1 = (c.part + 1) * ph.k_blocks / ph.parts;
            c.kb = c.kb0;
            return true;
        }
        ++c.phase;
        c.index = 0;
    }
    return false;
}
__device__ __forceinline__ bool cursor_begin(const TcParams& p, Cursor& c) {
    c = Cursor{0, 0, 0, 0, 0, 0, 0};
    return cursor_load(p, c);
}
__device__ __forceinline__ bool cursor_next(const TcParams& p, Cursor& c) {
    if (++c.kb < c.kb1) return true;
    ++c.index;
    return cursor_load(p, c);
}

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
tc_program_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    float* term_scale = reinterpret_cast<float*>(smem + kStages * kStageBytes);   // [token]: scale of term 0 in the current phase
    uint32_t* anchor = reinterpret_cast<uint32_t*>(term_scale + 8);               // [token]: exponent field the term scales are anchored on
    uint32_t* collected = anchor + 8;                                              // [token]: largest magnitudes of this CTA's SwiGLU outputs
    volatile uint32_t* acts_ready = collected + 8;                                 // [phase]: the phase's split activations are complete
    // full[S] (operand codes landed), empty[S], scales_landed[S], scales_ready[S] (copies to tensor memory issued),
    // acc_full[2], acc_empty[2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(const_cast<uint32_t*>(acts_ready) + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (smem_u32(smem) & 1023u) {
        // swizzled operand tiles want the window on a 1024-byte boundary, which is where the hardware puts it
        if (threadIdx.x == 0) atomicCAS(p.status_word, 0u, kErrTcWindow);
        return;
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
    const uint32_t bar_scales_landed = smem_u32(bars + 2 * kStages), bar_scales_ready = smem_u32(bars + 3 * kStages);
    const uint32_t bar_acc_full = smem_u32(bars + 4 * kStages), bar_acc_empty = smem_u32(bars + 4 * kStages + 2);

    auto issue_weights = [&](uint32_t stage, const Cursor& c) {
        const TcPhase& ph = p.phase[c.phase];
        const uint32_t k_valid = min(kStageK, ph.cols - c.kb * kStageK);
        const uint32_t sf_bytes = k_valid / 64 * kSfAtomBytes;
        const uint32_t dst = smem_u32(smem + stage * kStageBytes);
        // the scales first, on a barrier of their own: they are small, land early, and the copy thread moves
        // them on to tensor memory while the codes are still on their way
        mbar_expect_tx(bar_scales_landed + 8 * stage, sf_bytes);
        bulk_load(dst + kStageCodeBytes, ph.weight_sf + (static_cast<uint64_t>(c.tile) * (ph.cols / 64) + c.kb * 4) * kSfAtomBytes, sf_bytes,
                  bar_scales_landed + 8 * stage);
        mbar_expect_tx(bar_full + 8 * stage, kStageCodeBytes);
        tma_load_2d(dst, c.phase ? &map1 : &map0, c.kb * 128, c.tile * kTileM, bar_full + 8 * stage);
    };
    auto issue_activations = [&](uint32_t stage, const Cursor& c) {
        const TcPhase& ph = p.phase[c.phase];
        const uint32_t k_valid = min(kStageK, ph.cols - c.kb * kStageK);
        const uint32_t sf_bytes = k_valid / 64 * kSfAtomBytes;
        const uint32_t dst = smem_u32(smem + stage * kStageBytes);
        mbar_expect_tx(bar_scales_landed + 8 * stage, sf_bytes);
        bulk_load(dst + kStageActSf, ph.split + split_code_bytes(ph.cols) + static_cast<uint64_t>(c.kb) * kStageSfBytes, sf_bytes,
                  bar_scales_landed + 8 * stage);
        mbar_expect_tx(bar_full + 8 * stage, kChunkBytes);
        bulk_load(dst + kStageActCodes, ph.split + static_cast<uint64_t>(c.kb) * kChunkBytes, kChunkBytes, bar_full + 8 * stage);
    };

    Cursor weights_at;               // the producer's place in the weight stream (thread 0 only)
    bool weights_left = false;
    uint32_t weights_issued = 0;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 2);            // the weight half and the activation half of a stage are announced separately
            mbar_init(bar_scales_landed + 8 * s, 2);   // likewise for their block scales, which land first
            mbar_init(bar_scales_ready + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        acts_ready[0] = acts_ready[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The weight halves of the first ring fill go out at once, before anything else is set up: weights depend
        // on nothing, so HBM is busy while this CTA allocates tensor memory, while the launch before this one
        // finishes, and while the activations are split.
        weights_left = cursor_begin(p, weights_at);
        while (weights_left && weights_issued < kStages) {
            issue_weights(weights_issued, weights_at);
            ++weights_issued;
            weights_left = cursor_next(p, weights_at);
        }
    }
    if (threadIdx.x >= 64 && threadIdx.x < 64 + 16) anchor[threadIdx.x - 64] = 0;   // anchor and collected
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        // Weight halves run ahead as far as the ring allows; the activation half of a stage follows as soon as its
        // phase's split activations are complete. Neither waits for the other.
        Cursor acts_at;
        bool acts_left = cursor_begin(p, acts_at);
        uint32_t acts_issued = 0, idle = 0, fenced_phases = 0;
        while (acts_left) {
            bool progressed = false;
            if (weights_left) {
                // stage of step `weights_issued`: free once the MMAs of the step kStages before it are complete
                const uint32_t stage = weights_issued % kStages, round = weights_issued / kStages;
                if (mbar_test(bar_empty + 8 * stage, (round - 1) & 1)) {
                    issue_weights(stage, weights_at);
                    ++weights_issued;
                    weights_left = cursor_next(p, weights_at);
                    progressed = true;
                }
            }
            if (acts_issued < weights_issued && acts_ready[acts_at.phase]) {
                if (fenced_phases <= acts_at.phase) {
                    // the split activations were written with ordinary stores, by this and other CTAs
                    asm volatile("fence.proxy.async;" ::: "memory");
                    fenced_phases = acts_at.phase + 1;
                }
                issue_activations(acts_issued % kStages, acts_at);
                ++acts_issued;
                acts_left = cursor_next(p, acts_at);
                progressed = true;
            }
            if (progressed) {
                idle = 0;
            } else if (++idle > kWaitLimit || ((idle & 1023u) == 1023u && *abort_flag)) {
                *abort_flag = 1;
                atomicCAS(p.status_word, 0u, kErrTcProducer);
                break;
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = instr_desc(kCols);
        uint32_t step = 0, item_count = 0;
        uint32_t acc_phase[2] = {0, 0};
        Cursor c;
        bool more = cursor_begin(p, c);
        while (more) {
            const uint32_t buffer = item_count & 1;
            if (c.kb == c.kb0) {
                // the epilogue must have drained this buffer (two items ago)
                if (!mbar_wait(bar_acc_empty + 8 * buffer, acc_phase[buffer] ^ 1, abort_flag, p.status_word, kErrTcAccEmpty)) break;
                tc_fence_after();
            }
            const uint32_t acc = tmem_base + kTmemAcc + buffer * 64;
            const uint32_t stage = step % kStages, parity = (step / kStages) & 1;
            // operands in shared memory (TMA) and their block scales on the way to tensor memory (copy thread):
            // a copy and a later MMA execute in issue order, so the copies only have to be issued
            if (!mbar_wait(bar_full + 8 * stage, parity, abort_flag, p.status_word, kErrTcFull) ||
                !mbar_wait(bar_scales_ready + 8 * stage, parity, abort_flag, p.status_word, kErrTcScalesReady)) {
                break;
            }
            tc_fence_after();
            const uint32_t stage_smem = smem_u32(smem + stage * kStageBytes);
            const uint64_t weight_desc = operand_desc(stage_smem), act_desc = operand_desc(stage_smem + kStageActCodes);
            const uint32_t tmem_sf_weight = tmem_base + kTmemSfWeight + stage * 16, tmem_sf_act = tmem_base + kTmemSfAct + stage * 16;
            const uint32_t k_steps = min(kStageK, p.phase[c.phase].cols - c.kb * kStageK) / 64;
            // each MMA consumes 64 k = 32 bytes of every row: advance the start address by 32 >> 4
            if (k_steps == 4) {
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) {
                    tc_mma(acc, weight_desc + 2 * k, act_desc + 2 * k, idesc, tmem_sf_weight + 4 * k, tmem_sf_act + 4 * k,
                           (c.kb != c.kb0 || k != 0) ? 1u : 0u);
                }
            } else {
                for (uint32_t k = 0; k < k_steps; ++k) {
                    tc_mma(acc, weight_desc + 2 * k, act_desc + 2 * k, idesc, tmem_sf_weight + 4 * k, tmem_sf_act + 4 * k,
                           (c.kb != c.kb0 || k != 0) ? 1u : 0u);
                }
            }
            tc_commit(bar_empty + 8 * stage);   // frees the stage when these MMAs have read it
            if (c.kb + 1 == c.kb1) {
                tc_commit(bar_acc_full + 8 * buffer);
                acc_phase[buffer] ^= 1;
                ++item_count;
            }
            ++step;
            more = cursor_next(p, c);
        }
    } else if (warp == 6 && lane == 0) {
        // ---------------- scale copies: shared memory -> tensor memory, as soon as a stage's scales have landed ----------------
        // A stage's scale columns in tensor memory are free when its scales land again: the producer refilled the
        // stage only after the MMAs that read those columns were complete.
        uint32_t step = 0;
        Cursor c;
        bool more = cursor_begin(p, c);
        while (more) {
            const uint32_t stage = step % kStages, parity = (step / kStages) & 1;
            if (!mbar_wait(bar_scales_landed + 8 * stage, parity, abort_flag, p.status_word, kErrTcScalesLanded)) break;
            tc_fence_after();
            const uint32_t stage_smem = smem_u32(smem + stage * kStageBytes);
            const uint64_t weight_sf_desc = sf_desc(stage_smem + kStageCodeBytes), act_sf_desc = sf_desc(stage_smem + kStageActSf);
            const uint32_t tmem_sf_weight = tmem_base + kTmemSfWeight + stage * 16, tmem_sf_act = tmem_base + kTmemSfAct + stage * 16;
            const uint32_t k_steps = min(kStageK, p.phase[c.phase].cols - c.kb * kStageK) / 64;
            if (k_steps == 4) {
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) {
                    tc_copy_sf(tmem_sf_weight + 4 * k, weight_sf_desc + k * (kSfAtomBytes >> 4));
                    tc_copy_sf(tmem_sf_act + 4 * k, act_sf_desc + k * (kSfAtomBytes >> 4));
                }
            } else {
                for (uint32_t k = 0; k < k_steps; ++k) {
                    tc_copy_sf(tmem_sf_weight + 4 * k, weight_sf_desc + k * (kSfAtomBytes >> 4));
                    tc_copy_sf(tmem_sf_act + 4 * k, act_sf_desc + k * (kSfAtomBytes >> 4));
                }
            }
            tc_fence_before();
            mbar_arrive(bar_scales_ready + 8 * stage);
            ++step;
            more = cursor_next(p, c);
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------- workers: split the activations of a phase, then run its epilogues ----------------
        const uint32_t worker = threadIdx.x - 64, quadrant = warp & 3;   // tensor-memory lanes of this warp: 32 * quadrant .. + 31
        const bool leader = worker == 0;
        uint32_t item_count = 0;
        uint32_t acc_phase[2] = {0, 0};
        bool alive = true;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations may come from the launch before this one; all stores follow
        uint32_t meeting = 0;
        if (leader) meeting = *static_cast<volatile uint32_t*>(p.grid_barrier + 3);   // written by the launch before, at its last meeting
        const uint32_t first_pair = (blockIdx.x * 4 + (warp - 2)) * 2 + (lane >> 4), pair_stride = gridDim.x * 8;   // this half warp's groups
        for (uint32_t phase = 0; alive && phase < p.phases; ++phase) {
            const TcPhase& ph = p.phase[phase];
            const uint32_t groups = p.tokens * (ph.cols / 16);
            uint32_t held[kHeld];
            if (ph.scan) {
                // the row maxima of an input from outside: every lane looks at its own elements (and keeps them)
#pragma unroll
                for (uint32_t j = 0; j < kHeld; ++j) held[j] = load_element(ph, p.tokens, first_pair + j * pair_stride, lane);
                auto note = [&](uint32_t index, uint32_t bits) {   // whole warps: the two groups of a pair go together
                    uint32_t largest = bits & 0x7fffu;
                    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 8));
                    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 4));
                    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 2));
                    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 1));
                    if ((lane & 15) == 0 && largest) atomicMax(&collected[index / (ph.cols / 16)], largest << 16);   // zero past the end
                };
#pragma unroll
                for (uint32_t j = 0; j < kHeld; ++j) {
                    if (first_pair - (lane >> 4) + j * pair_stride < groups) note(first_pair + j * pair_stride, held[j]);
                }
                for (uint32_t index = first_pair + kHeld * pair_stride; index - (lane >> 4) < groups; index += pair_stride) {
                    note(index, load_element(ph, p.tokens, index, lane));
                }
                workers_sync();
                if (worker < 8) {
                    if (collected[worker]) atomicMax(ph.row_max + worker, collected[worker]);
                    collected[worker] = 0;
                }
            }
            // every CTA has found its maxima, or has finished the phase before: its output is this phase's input
            // and its maxima are collected
            if (!grid_meet(p, leader, meeting, abort_flag)) break;
            if (!ph.scan) {
#pragma unroll
                for (uint32_t j = 0; j < kHeld; ++j) held[j] = load_element(ph, p.tokens, first_pair + j * pair_stride, lane);
            }
            if (worker < 8) {
                // term 0 of the row has the global scale 2^(A - 135): all eight term scales are normal f32 numbers
                const uint32_t largest = *static_cast<volatile uint32_t*>(ph.row_max + worker) >> 16;
                const uint32_t a = min(max(largest >> 7, 40u), 250u);
                float scale = __uint_as_float((a - 8) << 23);
                if (largest >= 0x7f80u) scale = __uint_as_float(0x7fc00000u);   // a NaN or infinity in the row: the row's outputs are NaN
                term_scale[worker] = scale;
                anchor[worker] = a;
            }
            workers_sync();
#pragma unroll
            for (uint32_t j = 0; j < kHeld; ++j) {
                if (first_pair - (lane >> 4) + j * pair_stride < groups) split_group(ph, p.tokens, anchor, first_pair + j * pair_stride, held[j], lane);
            }
            for (uint32_t index = first_pair + kHeld * pair_stride; index - (lane >> 4) < groups; index += pair_stride) {
                split_group(ph, p.tokens, anchor, index, load_element(ph, p.tokens, index, lane), lane);
            }
            // every CTA's slice is in place (and readable by the TMA engine) before any CTA loads from the split
            asm volatile("fence.proxy.async;" ::: "memory");
            if (!grid_meet(p, leader, meeting, abort_flag)) break;
            if (blockIdx.x == 0 && worker < 8) ph.row_max[worker] = 0;   // every CTA has read them: clean for the next launch
            if (leader) acts_ready[phase] = 1;

            // ---- epilogues of this CTA's items of the phase ----
            const uint32_t items = ph.tiles * ph.parts;
            for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++item_count) {
                const uint32_t tile = item / ph.parts, part = item - tile * ph.parts;
                const uint32_t buffer = item_count & 1;
                if (!mbar_wait(bar_acc_full + 8 * buffer, acc_phase[buffer], abort_flag, p.status_word, kErrTcAccFull)) {
                    alive = false;
                    break;
                }
                acc_phase[buffer] ^= 1;
                tc_fence_after();
                uint32_t v[kCols / 16][16];
                const uint32_t taddr = tmem_base + kTmemAcc + buffer * 64 + ((quadrant * 32) << 16);
#pragma unroll
                for (uint32_t j = 0; j < kCols / 16; ++j) tc_load16(taddr + 16 * j, v[j]);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buffer);   // the buffer is free for the item after next
                float y[8];
#pragma unroll
                for (uint32_t token = 0; token < 8; ++token) {
                    // column = term * 8 + token; term t carries the factor 8^-t relative to term 0
                    float sum = 0.0f, factor = 1.0f;
#pragma unroll
                    for (uint32_t term = 0; term < kTerms; ++term) {
                        const uint32_t column = term * 8 + token;
                        sum = fmaf(__uint_as_float(v[column >> 4][column & 15]), factor, sum);
                        factor *= 0.125f;
                    }
                    y[token] = sum * term_scale[token];
                }
                contribute_rows(ph, p.tokens, tile, quadrant, part, lane, y, collected);
            }
            if (ph.collect) {
                workers_sync();
                if (worker < 8) {
                    if (collected[worker]) atomicMax(ph.collect + worker, collected[worker]);
                    collected[worker] = 0;
                }
            }
        }
        // the next launch goes on counting meetings where this one stopped (every CTA stores the same number)
        if (alive && leader) p.grid_barrier[3] = meeting;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------------
struct TcGeometry {
    uint32_t tiles, k_blocks, parts, ctas;
    uint64_t partial_bytes;
};

// Whole tiles dealt round-robin over the resident CTAs (two per SM) when there are enough of them; otherwise every
// tile is cut along k into as many equal parts as there are resident CTAs per tile (at least two ring stages per
// part, at most 16 parts).
TcGeometry tc_geometry(uint32_t physical_rows, uint32_t cols, uint32_t sm_count) {
    TcGeometry g{};
    g.tiles = physical_rows / kTileM;
    g.k_blocks = (cols + kStageK - 1) / kStageK;
    g.parts = 1;
    const uint32_t slots = sm_count * kCtasPerSm;   // CTAs resident at once
    if (g.tiles < slots) {
        uint32_t parts = slots / g.tiles;
        if (parts > g.k_blocks / 2) parts = g.k_blocks / 2;
        if (parts > 16) parts = 16;
        if (parts > 1) g.parts = parts;
    }
    const uint64_t items = static_cast<uint64_t>(g.tiles) * g.parts;
    g.ctas = items < slots ? static_cast<uint32_t>(items) : slots;
    g.partial_bytes = g.parts > 1 ? static_cast<uint64_t>(g.tiles) * 4 * g.parts * kSlotFloats * 4 : 0;
    return g;
}

bool check_tc_scalars(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t* physical_rows) {
    if (a->stored_rows || a->reserved1 || a->epilogue > AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) return false;
    const bool pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    if (!a->rows || !a->cols || a->rows > (1u << 30) || a->cols > INT_MAX) return false;
    *physical_rows = pair ? 2 * a->rows : a->rows;
    if (*physical_rows % kTileM != 0 || a->cols % 64 != 0) return false;
    if (static_cast<uint64_t>(*physical_rows) * a->cols > UINT32_MAX) return false;
    if (a->tokens < 1 || a->tokens > AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) return false;
    if (!scale_ok(a->global_scale)) return false;
    if (pair ? !scale_ok(a->global_scale_b) : a->global_scale_b != 0.0f) return false;
    if (a->weight_len_bytes != tcgen05_extent_bytes(*physical_rows, a->cols)) return false;
    if (a->input_len_bytes != static_cast<uint64_t>(a->tokens) * a->cols * 2) return false;
    const uint64_t out_elem = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32 ? 4 : 2;
    return a->output_len_bytes == static_cast<uint64_t>(a->tokens) * a->rows * out_elem;
}

uint32_t physical_rows_of(const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    return a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 ? 2 * a->rows : a->rows;
}

// What a phase needs of the plan scratch behind the counter regions: the split activations, then the partial sums.
uint64_t tc_scratch_need(const TcGeometry& g, uint32_t cols) { return (split_bytes(cols) + 255) / 256 * 256 + g.partial_bytes; }

// Scalars, extents, scratch room (`offset` .. `limit` of the plan scratch) and aliasing of one phase.
bool check_tc(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
              const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint64_t offset, uint64_t limit, bool full,
              augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    uint32_t physical_rows = 0;
    if (!plan_ok(plan, d, s) || !check_tc_scalars(a, &physical_rows)) return false;
    const TcGeometry g = tc_geometry(physical_rows, a->cols, plan->sm_count);
    if (g.tiles * 4 > kMaxGroups || offset < kCounterBytes || offset % 256 != 0 || limit < offset ||
        tc_scratch_need(g, a->cols) > limit - offset) {
        return false;
    }
    const Range r[4] = {{a->weight, a->weight_len_bytes, 256}, {a->input_bf16, a->input_len_bytes, 16},
                        {a->output, a->output_len_bytes, 4}, plan_scratch_range(plan)};
    if (!all_disjoint(r, 4)) return false;
    return !full || inspect_device_ranges(d, r, 3, failure);
}

// Packed codes as a 2-D byte tensor [rows][cols/2]; boxes of 128 rows x 128 bytes, 128-byte swizzle.
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
bool weight_map(CUtensorMap* map, uint64_t address, uint64_t rows, uint32_t cols) {
    static EncodeTiled encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            fn = nullptr;
        }
        return reinterpret_cast<EncodeTiled>(fn);
    }();
    if (!encode) return false;
    const cuuint64_t dims[2] = {cols / 2, rows};
    const cuuint64_t strides[1] = {cols / 2};
    const cuuint32_t box[2] = {128, 128};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void*>(address), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The grid barrier and the row maxima of both phases live in the plan's header (the 256 bytes in front of the
// scratch, behind the status word): no other kernel of the library writes there, plan creation zeroes them and
// every launch leaves them clean.
uint32_t* header_grid_barrier(const augur_cuda_nvfp4_sm100_plan_v1* plan) { return plan->status_word + 16; }
uint32_t* header_row_max(const augur_cuda_nvfp4_sm100_plan_v1* plan, uint32_t phase) { return plan->status_word + 32 + 8 * phase; }

// One launch for one or two phases (`b` null: one). Member m uses counter region m and the scratch at offsets[m].
augur_cuda_result_v1 launch_tc(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                               const augur_cuda_nvfp4_sm100_gemv_args_v1* a, const augur_cuda_nvfp4_sm100_gemv_args_v1* b,
                               const uint64_t (&offsets)[2]) {
    const augur_cuda_nvfp4_sm100_gemv_args_v1* members[2] = {a, b};
    CUtensorMap maps[2];
    TcParams p{};
    p.phases = b ? 2 : 1;
    p.tokens = a->tokens;
    p.grid_barrier = header_grid_barrier(plan);
    p.status_word = plan->status_word;
    uint32_t grid = 0;
    for (uint32_t m = 0; m < p.phases; ++m) {
        const augur_cuda_nvfp4_sm100_gemv_args_v1* args = members[m];
        const uint32_t physical_rows = physical_rows_of(args);
        const TcGeometry g = tc_geometry(physical_rows, args->cols, plan->sm_count);
        if (!weight_map(&maps[m], args->weight, physical_rows, args->cols)) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
        TcPhase& ph = p.phase[m];
        ph.weight_sf = reinterpret_cast<const uint8_t*>(args->weight) + tcgen05_codes_bytes(physical_rows, args->cols);
        ph.x = reinterpret_cast<const uint16_t*>(args->input_bf16);
        ph.split = plan->scratch + offsets[m];
        ph.out = reinterpret_cast<void*>(args->output);
        ph.counters = reinterpret_cast<uint32_t*>(plan->scratch + m * kCounterRegionBytes);
        ph.partials = reinterpret_cast<float*>(plan->scratch + offsets[m] + (split_bytes(args->cols) + 255) / 256 * 256);
        ph.row_max = header_row_max(plan, m);
        ph.collect = (m == 0 && b) ? header_row_max(plan, 1) : nullptr;
        ph.rows = physical_rows; ph.out_rows = args->rows; ph.cols = args->cols; ph.epilogue = args->epilogue;
        ph.tiles = g.tiles; ph.k_blocks = g.k_blocks; ph.parts = g.parts;
        ph.scan = m == 0 ? 1u : 0u;
        ph.global_a = args->global_scale; ph.global_b = args->global_scale_b;
        if (g.ctas > grid) grid = g.ctas;
    }
    if (!b) maps[1] = maps[0];
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config{};
    config.stream = s->stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    cudaLaunchKernelEx(&config, tc_program_kernel, maps[0], maps[1], p);
    count_launch();
    return submitted();
}

}  // namespace

cudaError_t gemv_tc_configure_device() {
    return cudaFuncSetAttribute(tc_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
}

}  // namespace augur_sm100

using namespace augur_sm100;

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_scratch_extent_host_v1(
    uint32_t rows, uint32_t cols, uint32_t epilogue, uint64_t* out_bytes) {
    if (!out_bytes || !rows || !cols || cols % 64 != 0 || epilogue > AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) return invalid();
    const uint64_t physical = epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 ? 2ull * rows : rows;
    if (physical % kTileM != 0 || physical * cols > UINT32_MAX) return invalid();
    uint64_t worst = 0;   // over any SM count up to 512
    for (uint32_t sms = 1; sms <= 512; ++sms) {
        const TcGeometry g = tc_geometry(static_cast<uint32_t>(physical), cols, sms);
        if (tc_scratch_need(g, cols) > worst) worst = tc_scratch_need(g, cols);
    }
    *out_bytes = kCounterBytes + (worst + 255) / 256 * 256;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_tc(d, s, plan, a, kCounterBytes, plan ? plan->scratch_bytes : 0, true, &failure)) return failure;
    CUtensorMap probe;
    return weight_map(&probe, a->weight, physical_rows_of(a), a->cols) ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_tc(d, s, plan, a, kCounterBytes, plan ? plan->scratch_bytes : 0, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    const uint64_t offsets[2] = {kCounterBytes, 0};
    return launch_tc(s, plan, a, nullptr, offsets);
}

// ---- the MLP block as one launch ----------------------------------------------------------------------
namespace {
// Both members plus every cross alias, before anything is enqueued; the members use separate counter regions and
// separate halves of the scratch behind them.
bool check_mlp_tc(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                  const augur_cuda_nvfp4_sm100_mlp_args_v1* a, bool full, uint64_t* down_offset, augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!plan_ok(plan, d, s) || plan->scratch_bytes < kCounterBytes) return false;
    const uint64_t middle = kCounterBytes + (plan->scratch_bytes - kCounterBytes) / 2 / 256 * 256;
    *down_offset = middle;
    if (!check_tc(d, s, plan, &a->gate_up, kCounterBytes, middle, false, failure)) return false;
    if (!check_tc(d, s, plan, &a->down, middle, plan->scratch_bytes, false, failure)) return false;
    *failure = invalid();
    if (a->gate_up.epilogue != AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 || a->down.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
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

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tc_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_mlp_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint64_t down_offset = 0;
    if (!check_mlp_tc(d, s, plan, a, true, &down_offset, &failure)) return failure;
    CUtensorMap probe;
    return weight_map(&probe, a->gate_up.weight, physical_rows_of(&a->gate_up), a->gate_up.cols) &&
                   weight_map(&probe, a->down.weight, physical_rows_of(&a->down), a->down.cols)
               ? ok()
               : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tc_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_mlp_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint64_t down_offset = 0;
    if (!check_mlp_tc(d, s, plan, a, false, &down_offset, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    const uint64_t offsets[2] = {kCounterBytes, down_offset};
    return launch_tc(s, plan, &a->gate_up, &a->down, offsets);
}
