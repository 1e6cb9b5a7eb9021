// Small-token (1..8) NVFP4 linear and MLP block for sm_100a on the tensor-memory path: the weights go from HBM to
// the tensor cores without a single per-element instruction on the SMs, and a whole MLP block is ONE launch in
// which the weight stream does not stop at the boundary between its two products.
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
// A launch is a list of steps, each a set of (row tile, k range) items dealt round-robin to the CTAs (two per
// SM, all resident: two short rings consumed in order lose less to a late stage than one long ring). A linear
// is one step: whole tiles when there are at least about as many as CTAs, else every tile cut along k into equal
// parts whose partial sums meet in plan scratch (arrival counter per 32 rows; the last arriver adds the parts in
// a fixed order and finishes the rows; bit-reproducible). The MLP block is two steps when the
// gate|up tiles fit the CTAs: gate|up in whole tiles, then down in k parts. The second product needs every CTA's
// outputs of the first and their largest magnitudes per token row before it can split them: the CTAs arrive at
// a counter when their outputs are stored, wait for all, split, arrive at a second counter, and the activation
// loads of the second product wait for that one; its weights are in the ring by then. With more gate|up tiles
// than CTAs the block is four steps in two waves - gate|up tiles 0..G-1 (G = CTAs), gate|up tiles G.., down over
// the k range that the first wave's outputs feed, down over the rest - so that the first wave's outputs are met
// over and split while the second wave streams: the down partial sums of the two k ranges carry separate
// power-of-two scales and are added in f32 like any other parts.
//
// Roles of a CTA: one thread streams the weight halves of the stages of all its items back to back and keeps
// doing so while activations are not ready yet (the ring buffers that time); one thread sends the activation
// halves after them; one copies block scales to tensor memory; one issues the MMAs; four warps split activations
// and run the epilogues. CTAs meet through counters in the
// plan's header: full meetings before the first product (row maxima of the input, then its split), and
// arrive-now / wait-later counters per wave.
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
constexpr uint32_t kCtasPerSm = 2;                     // two rings consumed in order stall less on a late stage than one of twice the depth
constexpr uint32_t kThreads = 416;                     // warp 0 TMA of weights, 1 MMA, 2..9 split and epilogue, 10 and 12 scale copies, 11 TMA of activations
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 512 /*small state*/;   // the stages start the (1024-byte aligned) window
constexpr uint32_t kTmemAcc = 0;                       // two accumulators of 64 columns
constexpr uint32_t kTmemSfWeight = 128;                // 16 columns per ring stage
constexpr uint32_t kTmemSfAct = kTmemSfWeight + kStages * 16;
constexpr uint32_t kTmemColumns = 256;
static_assert(kTmemSfAct + kStages * 16 <= kTmemColumns, "tensor memory columns");
static_assert(kCtasPerSm * kTmemColumns <= 512, "tensor memory of an SM");
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM, a kilobyte each reserved by the system");
static_assert(kTerms == 8, "the digit transposition is 8 lanes x 8 nibbles");
static_assert(kStageBytes % 1024 == 0 && kStageActCodes % 1024 == 0, "swizzled operand tiles are 1024-byte aligned");
constexpr uint32_t kSlotFloats = 256;                  // one partial: 32 rows x 8 tokens
constexpr uint32_t kWorkers = 256;                     // the eight split / epilogue warps: two per quarter of the accumulator's rows, four token rows each
constexpr uint32_t kMaxPhases = 2, kMaxJobs = 3, kMaxSteps = 4;
constexpr uint32_t kGridWaitLimit = 1u << 22;          // polls of a counter (a fraction of a microsecond each) before giving up
constexpr uint32_t kHeld = 4;                          // elements a lane keeps in registers between the scan and the split

constexpr uint32_t kErrTcProducer = 0x301, kErrTcFull = 0x302, kErrTcAccEmpty = 0x303, kErrTcAccFull = 0x304,
                   kErrTcScalesLanded = 0x305, kErrTcScalesReady = 0x306, kErrTcGridBarrier = 0x307, kErrTcWindow = 0x308,
                   kErrTcWave = 0x309;

// Words of the plan's header (the 256 bytes in front of the scratch; word 0 is the status word) that this kernel
// owns: no other kernel of the library writes there, plan creation zeroes them, every launch leaves them ready
// for the next one.
constexpr uint32_t kHeaderMeeting = 16;    // three arrival counters of the full meetings, used in turn
constexpr uint32_t kHeaderEpoch = 19;      // meetings held so far, modulo 3
constexpr uint32_t kHeaderWave = 20;       // [launch parity][wave]{outputs stored, split stored}
constexpr uint32_t kHeaderParity = 28;     // launches so far, modulo 2
// The plan's trailer: [launch parity][wave][CTA] one 64-bit word per CTA with the exponent fields of the largest
// magnitudes of its outputs, one byte per token row (0: not written yet).
constexpr uint32_t kMaxCtas = static_cast<uint32_t>(kPlanTrailerBytes / 32);
constexpr uint32_t kHeaderRowMax = 32;     // [job][token] bits of the row's largest magnitude

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
    float* partials;              // [tile * 4 + quadrant][contributor][32 rows][8 tokens]
    uint32_t* counters;           // [tile * 4 + quadrant][half of the token rows], zero between launches
    uint32_t rows;                // physical weight rows (SwiGLU: gate and up interleaved by 16)
    uint32_t out_rows;            // output width
    uint32_t cols, epilogue;
    uint32_t contributors;        // items per tile over all steps of the phase (1: whole tiles)
    float global_a, global_b;
};

// One split of activations: groups [group0, group0 + groups) of every token row of a phase's input.
struct TcJob {
    uint32_t phase, group0, groups;
};

// One set of items: tiles [tile0, tile0 + tiles) of a phase over the k blocks [kb0, kb1), every tile in `parts`
// equal k ranges; the activations come from `job`; a part is contributor slot0 + part of its tile.
struct TcStep {
    uint32_t phase, job, tile0, tiles, kb0, kb1, parts, slot0;
    uint32_t feeds;               // the job that splits this step's outputs (SwiGLU steps of the MLP block), or 0
    uint32_t keeps;               // every CTA has at most one item of the step and finishes it alone: it splits its own outputs
};

struct TcParams {
    TcPhase phase[kMaxPhases];
    TcJob job[kMaxJobs];
    TcStep step[kMaxSteps];
    uint32_t jobs, steps, tokens;
    uint32_t* header;             // the plan's header words; header[0] is the status word
    unsigned long long* slots;    // the plan's trailer
};

__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_load4(uint32_t taddr, uint32_t (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// ---- counters between CTAs (thread `leader` of the four worker warps speaks for its CTA) ----------------------
__device__ __forceinline__ uint32_t counter_arrive(uint32_t* counter) {
    uint32_t before;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(before) : "l"(counter) : "memory");
    return before;
}
__device__ __forceinline__ void counter_arrive_only(uint32_t* counter) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}
__device__ __forceinline__ uint32_t counter_read(const uint32_t* counter) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    return seen;
}
// Everything the CTAs wrote before arriving is visible after the wait. False if the wait ran out.
__device__ __forceinline__ bool counter_wait(const TcParams& p, const uint32_t* counter, uint32_t code, volatile uint32_t* abort_flag) {
    for (uint32_t spin = 0; counter_read(counter) < gridDim.x;) {
        if (++spin > kGridWaitLimit || ((spin & 255u) == 255u && *abort_flag)) {
            *abort_flag = 1;
            atomicCAS(p.header, 0u, code);
            return false;
        }
    }
    return true;
}

// All CTAs of the grid meet. Everything the workers wrote before is visible to every CTA's workers after.
// Meeting number m (counted over all launches of the plan, modulo 3, in `meeting`) uses counter m % 3. The last
// arriver clears counter (m - 1) % 3, which every CTA has stopped reading (all are at meeting m) and which is not
// used again before meeting m + 2; nobody gets to meeting m + 2 before the last arriver of m, its store behind it,
// has arrived at m + 1. A CTA may raise a flag as it arrives (the arrivals count in the low 16 bits, the flags
// above them): `*raised` says afterwards whether any CTA did.
__device__ __forceinline__ bool grid_meet(const TcParams& p, bool leader, uint32_t& meeting, bool raise, volatile uint32_t* raised,
                                          volatile uint32_t* abort_flag) {
    workers_sync();
    if (leader) {
        uint32_t* mine = p.header + kHeaderMeeting + meeting;
        uint32_t seen;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(seen) : "l"(mine), "r"(raise ? 0x10001u : 1u) : "memory");
        seen += raise ? 0x10001u : 1u;
        if ((seen & 0xffffu) == gridDim.x) {
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.header + kHeaderMeeting + (meeting + 2) % 3), "r"(0u) : "memory");
        } else {
            for (uint32_t spin = 0;;) {
                seen = counter_read(mine);
                if ((seen & 0xffffu) >= gridDim.x) break;
                if (++spin > kGridWaitLimit || ((spin & 255u) == 255u && *abort_flag)) {
                    *abort_flag = 1;
                    atomicCAS(p.header, 0u, kErrTcGridBarrier);
                    break;
                }
            }
        }
        *raised = seen >> 16;
    }
    meeting = (meeting + 1) % 3;
    workers_sync();
    return *abort_flag == 0;
}

// ---- activation split (the four worker warps of every CTA; the grid's worker warps share the groups out) ----
// One lane per element, sixteen neighbouring lanes per 16-element group; warp w of the grid's W worker warps
// takes the group pairs w, w + W, ... of a job. With A the exponent field of the largest magnitude of the token
// row (within the job) and G that of the group's, the group's block scale is 2^q, q = G + 8 - A (the row's
// largest group gets 2^8; E4M3 holds powers of two down to 2^-9, smaller groups keep 2^-9 and lose low bits),
// term t has the global scale 2^(A - 155) * 8^t (times the level, half the digit), and the element is the integer I = |x| / 2^(q + A - 156): at
// most 255 * 2^14 for the group's largest element, exact for every element within 2^-14 of it, rounded to
// nearest below. I is written in radix 8 with digits -4..3: I plus 4 in every octal place has the digits plus 4
// as its octal digits (eight of them: 3 * (8^8 - 1) / 7 > 255 * 2^14). Digit t is the code of term t: level
// |digit| / 2, sign of digit times sign of x; all eight are formed at once in the nibbles of one word. The eight
// lanes of a half group transpose their words so that lane t holds the eight codes of term t, and store one
// word each.
__device__ __forceinline__ uint32_t load_element(const TcPhase& ph, const TcJob& job, uint32_t tokens, uint32_t index, uint32_t lane) {
    if (index >= tokens * job.groups) return 0;
    const uint32_t token = index / job.groups, group = job.group0 + (index - token * job.groups);
    return __ldcg(ph.x + static_cast<uint64_t>(token) * ph.cols + group * 16 + (lane & 15));
}

// (Both halves are real functions, not inlined: the code that runs at the boundary between the two products is
// then the code the launch has already run for its input, and is still in the instruction cache.)
// First half of a group's split, before the row's anchor is known: the group's largest magnitude (returned), the
// digits relative to it (`drop` low bits fewer), the codes stored. Whole warps; `index` past the job is inactive.
struct SplitTarget {
    uint8_t* split;               // the phase's split activations
    uint32_t sf_offset;           // of its block-scale atoms
    uint32_t group0, groups;      // the job's groups of every token row
    uint32_t tokens;
};
__device__ __forceinline__ SplitTarget split_target(const TcParams& p, uint32_t job_index) {
    const TcJob& job = p.job[job_index];
    const TcPhase& ph = p.phase[job.phase];
    return SplitTarget{ph.split, static_cast<uint32_t>(split_code_bytes(ph.cols)), job.group0, job.groups, p.tokens};
}

// A group of a job by its index, as (token row, group of the row); the token row is ~0 past the job's end.
__device__ __forceinline__ uint2 group_of(const SplitTarget& to, uint32_t index) {
    if (index >= to.tokens * to.groups) return make_uint2(~0u, 0u);
    const uint32_t token = index / to.groups;
    return make_uint2(token, to.group0 + (index - token * to.groups));
}

__device__ __noinline__ uint32_t split_codes(const SplitTarget to, uint2 where, uint32_t bits, uint32_t drop, uint32_t lane) {
    const bool active = where.x != ~0u;
    const uint32_t token = active ? where.x : 0, group = where.y;
    const uint32_t magnitude = bits & 0x7fffu, negative = (bits >> 15) & 1u;
    uint32_t largest = max(magnitude, __shfl_xor_sync(0xffffffffu, magnitude, 8));
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 4));
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 2));
    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, 1));
    const int g = max(static_cast<int>(largest >> 7), 1);           // a subnormal has the exponent of field 1
    const uint32_t field = magnitude >> 7;
    const uint32_t significand = field ? 128u + (magnitude & 127u) : magnitude;
    // |x| = significand * 2^(max(field, 1) - 134); I = |x| * 2^(156 - q - A) = significand * 2^(field - G + 14) with q = G + 8 - A
    const int shift = max(static_cast<int>(max(field, 1u)) - g + 14 - static_cast<int>(drop), -16);
    const uint32_t value = shift >= 0 ? significand << shift : (significand + (1u << (-shift - 1))) >> -shift;
    // octal digits of I + 44444444 (octal), one per nibble: d = digit + 4 in 0..7
    uint32_t d = (value + 0x924924u) & 0xffffffu;
    d = (d & 0x00000fffu) | ((d & 0x00fff000u) << 4);
    d = (d & 0x003f003fu) | ((d & 0x0fc00fc0u) << 2);
    d = (d & 0x07070707u) | ((d & 0x38383838u) << 1);
    // level = |d - 4|: d & 3 where d >= 4, else 4 - d = (~d & 3) + 1; the digit is negative where d < 4
    const uint32_t upper = (d >> 2) & 0x11111111u, upper_mask = upper * 15u;
    const uint32_t level = ((d & 0x33333333u) & upper_mask) | (((~d & 0x33333333u) + 0x11111111u) & ~upper_mask);
    const uint32_t nonzero = (level | (level >> 1) | (level >> 2)) & 0x11111111u;
    const uint32_t minus = ((upper ^ 0x11111111u) ^ (negative * 0x11111111u)) & nonzero;
    uint32_t digits = level | (minus << 3);    // code of term t in bits 4t .. 4t + 3
    // 8 lanes x 8 nibbles, transposed: lane t of the eight ends up with nibble t of all eight, in lane order
    uint32_t other = __shfl_xor_sync(0xffffffffu, digits, 4);
    digits = (lane & 4) ? (other >> 16) | (digits & 0xffff0000u) : (digits & 0x0000ffffu) | (other << 16);
    other = __shfl_xor_sync(0xffffffffu, digits, 2);
    digits = (lane & 2) ? ((other & 0xff00ff00u) >> 8) | (digits & 0xff00ff00u) : (digits & 0x00ff00ffu) | ((other & 0x00ff00ffu) << 8);
    other = __shfl_xor_sync(0xffffffffu, digits, 1);
    digits = (lane & 1) ? ((other & 0xf0f0f0f0u) >> 4) | (digits & 0xf0f0f0f0u) : (digits & 0x0f0f0f0fu) | ((other & 0x0f0f0f0fu) << 4);
    // lanes t and t + 8 hold the two words of the group's eight bytes in row n = t * 8 + token
    other = __shfl_xor_sync(0xffffffffu, digits, 8);
    if (active && (lane & 8) == 0) {
        const uint32_t n = (lane & 7) * 8 + token, chunk = group >> 4, unit = (group & 15) >> 1, half = group & 1;
        uint8_t* codes = to.split + static_cast<uint64_t>(chunk) * kChunkBytes + (n >> 3) * 1024 + (n & 7) * 128 + ((unit ^ (n & 7)) << 4);
        *reinterpret_cast<uint2*>(codes + half * 8) = make_uint2(digits, other);
    }
    return largest;
}

// Second half, with the row's anchor: the group's block scale 2^q, q = G + 8 - A. A group more than 2^17 below its
// row's largest magnitude keeps 2^-9 and has its codes redone with that many low bits fewer (rare). True if the
// group is larger than the anchor provides for (an anchor that was guessed).
__device__ __noinline__ bool split_scales(const SplitTarget to, const uint32_t* anchor, uint2 where, uint32_t bits, uint32_t largest,
                                          uint32_t lane) {
    const bool active = where.x != ~0u;
    const uint32_t token = active ? where.x : 0, group = where.y;
    const int q = max(static_cast<int>(largest >> 7), 1) + 8 - static_cast<int>(anchor[token]);
    const uint32_t drop = active && q < -9 ? static_cast<uint32_t>(-9 - q) : 0u;
    if (__any_sync(0xffffffffu, drop != 0)) split_codes(to, where, bits, drop, lane);
    if (active && (lane & 8) == 0) {
        const int clamped = min(max(q, -9), 8);
        const uint32_t scale_code = clamped >= -6 ? static_cast<uint32_t>(clamped + 7) << 3 : 1u << (clamped + 9);
        const uint32_t n = (lane & 7) * 8 + token;
        uint8_t* sf = to.split + to.sf_offset + static_cast<uint64_t>(group >> 2) * kSfAtomBytes + (group & 3);
        sf[(n & 31) * 16 + (n >> 5) * 4] = static_cast<uint8_t>(scale_code);
    }
    return active && q > 8;   // the group is larger than the anchor allows for
}

// The term scales of a job from the row maxima every CTA has contributed to (workers 0..7, one token row each).
__device__ __forceinline__ void job_scales(const TcParams& p, uint32_t job, uint32_t worker, float* term_scale, uint32_t* anchor) {
    if (worker < 8) {
        const uint32_t largest = *static_cast<volatile uint32_t*>(p.header + kHeaderRowMax + 8 * job + worker) >> 16;
        // term 0 of the row has the global scale 2^(A - 155), term 7 2^(A - 134): all normal f32 numbers
        const uint32_t a = min(max(largest >> 7, 40u), 250u);
        float scale = __uint_as_float((a - 28) << 23);
        if (largest >= 0x7f80u) scale = __uint_as_float(0x7fc00000u);   // a NaN or infinity in the row: the row's outputs are NaN
        term_scale[8 * job + worker] = scale;
        anchor[8 * job + worker] = a;
    }
    workers_sync();
}

// This CTA's share of a job (group pairs first_pair, first_pair + pair_stride, ...): the first kHeld groups of each
// lane are in `held`; their codes are stored before the anchor is known (`largest` keeps what the second half
// needs), groups beyond them only add to the row maxima here and are split whole in the second half.
__device__ __forceinline__ void share_codes(const TcParams& p, uint32_t job_index, const uint32_t (&held)[kHeld], uint32_t (&largest)[kHeld],
                                            uint32_t* collected, uint32_t first_pair, uint32_t pair_stride, uint32_t lane) {
    const TcJob& job = p.job[job_index];
    const TcPhase& ph = p.phase[job.phase];
    const SplitTarget to = split_target(p, job_index);
    const uint32_t groups = p.tokens * job.groups, warp_first = first_pair - (lane >> 4);
#pragma unroll
    for (uint32_t j = 0; j < kHeld; ++j) {
        largest[j] = 0;
        if (warp_first + j * pair_stride < groups) {
            const uint32_t index = first_pair + j * pair_stride;
            largest[j] = split_codes(to, group_of(to, index), held[j], 0, lane);
            if (collected && (lane & 15) == 0 && largest[j]) atomicMax(&collected[index / job.groups], largest[j] << 16);   // zero past the end
        }
    }
    if (!collected) return;
    for (uint32_t index = first_pair + kHeld * pair_stride; index - (lane >> 4) < groups; index += pair_stride) {
        uint32_t most = load_element(ph, job, p.tokens, index, lane) & 0x7fffu;
        most = max(most, __shfl_xor_sync(0xffffffffu, most, 8));
        most = max(most, __shfl_xor_sync(0xffffffffu, most, 4));
        most = max(most, __shfl_xor_sync(0xffffffffu, most, 2));
        most = max(most, __shfl_xor_sync(0xffffffffu, most, 1));
        if ((lane & 15) == 0 && most) atomicMax(&collected[index / job.groups], most << 16);
    }
}
__device__ __forceinline__ bool share_scales(const TcParams& p, uint32_t job_index, const uint32_t* anchor, const uint32_t (&held)[kHeld],
                                             const uint32_t (&largest)[kHeld], uint32_t first_pair, uint32_t pair_stride, uint32_t lane) {
    bool beyond = false;
    const TcJob& job = p.job[job_index];
    const TcPhase& ph = p.phase[job.phase];
    const SplitTarget to = split_target(p, job_index);
    const uint32_t groups = p.tokens * job.groups, warp_first = first_pair - (lane >> 4);
#pragma unroll
    for (uint32_t j = 0; j < kHeld; ++j) {
        if (warp_first + j * pair_stride < groups) beyond |= split_scales(to, anchor + 8 * job_index, group_of(to, first_pair + j * pair_stride), held[j], largest[j], lane);
    }
    for (uint32_t index = first_pair + kHeld * pair_stride; index - (lane >> 4) < groups; index += pair_stride) {
        const uint32_t bits = load_element(ph, job, p.tokens, index, lane);
        beyond |= split_scales(to, anchor + 8 * job_index, group_of(to, index), bits, split_codes(to, group_of(to, index), bits, 0, lane), lane);
    }
    return beyond;
}

// Finished sums of 32 weight rows (lane = row) for the token rows token0 .. token0 + 3: scale, activation, rounding,
// store. `kept` (SwiGLU): the outputs stay with the caller, [0..3] as stored, [4] their exponent fields, a byte per row.
__device__ __forceinline__ void finish_rows(const TcPhase& ph, uint32_t tokens, uint32_t tile, uint32_t quadrant, uint32_t token0, uint32_t lane,
                                            const float (&y)[4], uint32_t* collected, uint32_t* kept) {
    if (ph.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
        // 32 physical rows = 16 gate rows (lanes 0..15) and the matching 16 up rows (lanes 16..31)
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(ph.out);
        const uint32_t index = (tile * kTileM + quadrant * 32) / 2 + (lane & 15);
        uint32_t fields = 0;   // exponent fields of this lane's outputs
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t token = token0 + j;
            const float up = __shfl_sync(0xffffffffu, y[j], (lane & 15) + 16) * ph.global_b;
            const float gate = y[j] * ph.global_a;
            uint32_t magnitude = 0;
            if (lane < 16 && token < tokens) {
                const __nv_bfloat16 h = __float2bfloat16_rn(__fdividef(gate, 1.0f + __expf(-gate)) * up);   // a few ulp of f32, far below the rounding
                magnitude = static_cast<uint32_t>(__bfloat16_as_ushort(h) & 0x7fffu) << 16;
                if (kept) {
                    kept[j] = __bfloat16_as_ushort(h);   // stored by the caller, behind its arrival with the maxima
                    fields |= (magnitude >> 23) << (8 * j);
                } else {
                    out[static_cast<uint64_t>(token) * ph.out_rows + index] = h;
                }
            }
            if (collected && !kept) {
                // a later step splits these values: it needs every token row's largest magnitude
                magnitude = __reduce_max_sync(0xffffffffu, magnitude);
                if (lane == 0 && magnitude) atomicMax(&collected[token], magnitude);
            }
        }
        if (kept) {
            // the caller only needs the exponent fields, the largest per token row over this warp
#pragma unroll
            for (uint32_t offset = 8; offset; offset >>= 1) fields = __vmaxu4(fields, __shfl_xor_sync(0xffffffffu, fields, offset));
            kept[4] = fields;
        }
        return;
    }
    const uint32_t row = tile * kTileM + quadrant * 32 + lane;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        const uint32_t token = token0 + j;
        if (token < tokens) {
            const float value = y[j] * ph.global_a;
            if (ph.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) {
                static_cast<float*>(ph.out)[static_cast<uint64_t>(token) * ph.out_rows + row] = value;
            } else {
                static_cast<__nv_bfloat16*>(ph.out)[static_cast<uint64_t>(token) * ph.out_rows + row] = __float2bfloat16_rn(value);
            }
        }
    }
}

// This warp's share (four token rows) of 32 rows of `tile`: finished here if tiles are whole, else handed over as
// contributor `slot`; the last of the arrivals adds all shares in slot order. Whole warps call this.
__device__ __forceinline__ void contribute_rows(const TcPhase& ph, uint32_t tokens, uint32_t tile, uint32_t quadrant, uint32_t token0, uint32_t slot,
                                                uint32_t lane, const float (&y)[4], uint32_t* collected, uint32_t* kept) {
    if (ph.contributors == 1) {
        finish_rows(ph, tokens, tile, quadrant, token0, lane, y, collected, kept);
        return;
    }
    const uint32_t group = tile * 4 + quadrant;
    float* slots = ph.partials + static_cast<uint64_t>(group) * ph.contributors * kSlotFloats;
    float4* mine = reinterpret_cast<float4*>(slots + static_cast<uint64_t>(slot) * kSlotFloats) + lane * 2 + (token0 >> 2);
    *mine = make_float4(y[0], y[1], y[2], y[3]);
    __syncwarp();
    // the arrival releases this warp's share and, for the last arriver, acquires the others'
    uint32_t arrived = 0;
    if (lane == 0) arrived = counter_arrive(&ph.counters[group * 2 + (token0 >> 2)]);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    __syncwarp();
    if (arrived + 1 != ph.contributors) return;
    float sum[4] = {0, 0, 0, 0};
    for (uint32_t s0 = 0; s0 < ph.contributors; s0 += 8) {
        float4 a[8];
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            a[j] = make_float4(0, 0, 0, 0);
            if (s0 + j < ph.contributors) {
                a[j] = __ldcg(reinterpret_cast<const float4*>(slots + static_cast<uint64_t>(s0 + j) * kSlotFloats) + lane * 2 + (token0 >> 2));
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            if (s0 + j < ph.contributors) {
                sum[0] += a[j].x; sum[1] += a[j].y; sum[2] += a[j].z; sum[3] += a[j].w;
            }
        }
    }
    finish_rows(ph, tokens, tile, quadrant, token0, lane, sum, collected, nullptr);
    if (lane == 0) ph.counters[group * 2 + (token0 >> 2)] = 0;   // clean for the next launch
}

// A CTA's ring stages in the order it streams them: over the steps, over its items blockIdx.x,
// blockIdx.x + gridDim.x, ... of a step, over the k blocks of an item.
struct Cursor {
    uint32_t step, index, tile, part, kb, kb0, kb1;
};
__device__ __forceinline__ bool cursor_load(const TcParams& p, Cursor& c) {
    while (c.step < p.steps) {
        const TcStep& st = p.step[c.step];
        const uint32_t item = blockIdx.x + c.index * gridDim.x;
        if (item < st.tiles * st.parts) {
            const uint32_t tile = item / st.parts, span = st.kb1 - st.kb0;
            c.tile = st.tile0 + tile;
            c.part = item - tile * st.parts;
            c.kb0 = st.kb0 + c.part * span / st.parts;
            c.kb1 = st.kb0 + (c.part + 1) * span / st.parts;
            c.kb = c.kb0;
            return true;
        }
        ++c.step;
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
    float* term_scale = reinterpret_cast<float*>(smem + kStages * kStageBytes);   // [job][token]: scale of term 0
    uint32_t* anchor = reinterpret_cast<uint32_t*>(term_scale + 8 * kMaxJobs);    // [job][token]: exponent field the term scales are anchored on
    uint32_t* collected = anchor + 8 * kMaxJobs;                                  // [token]: largest magnitudes this CTA has seen (scan, SwiGLU outputs)
    volatile uint32_t* input_ready = collected + 8;                               // the split of job 0 is complete
    volatile uint32_t* wave_set = input_ready + 1;                                // which half of the wave counters this launch uses
    volatile uint32_t* raised = wave_set + 1;                                     // flags of the last full meeting
    uint32_t* beyond = const_cast<uint32_t*>(raised) + 1;                         // a group of this CTA's share was beyond its row's guessed anchor
    uint32_t* gathered = beyond + 1;                                              // [worker warp][2]: bytewise maxima of what a warp has seen
    // full[S] (operand codes landed), empty[S], scales_landed[S], scales_ready[S] (copies to tensor memory issued),
    // acc_full[2], acc_empty[2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(gathered + 16);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (smem_u32(smem) & 1023u) {
        // swizzled operand tiles want the window on a 1024-byte boundary, which is where the hardware puts it
        if (threadIdx.x == 0) atomicCAS(p.header, 0u, kErrTcWindow);
        return;
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
    const uint32_t bar_scales_landed = smem_u32(bars + 2 * kStages), bar_scales_ready = smem_u32(bars + 3 * kStages);
    const uint32_t bar_acc_full = smem_u32(bars + 4 * kStages), bar_acc_empty = smem_u32(bars + 4 * kStages + 2);

    auto issue_weights = [&](uint32_t stage, const Cursor& c) {
        const uint32_t phase = p.step[c.step].phase;
        const TcPhase& ph = p.phase[phase];
        const uint32_t k_valid = min(kStageK, ph.cols - c.kb * kStageK);
        const uint32_t sf_bytes = k_valid / 64 * kSfAtomBytes;
        const uint32_t dst = smem_u32(smem + stage * kStageBytes);
        // the scales first, on a barrier of their own: they are small, land early, and the copy thread moves
        // them on to tensor memory while the codes are still on their way
        mbar_expect_tx(bar_scales_landed + 8 * stage, sf_bytes);
        bulk_load(dst + kStageCodeBytes, ph.weight_sf + (static_cast<uint64_t>(c.tile) * (ph.cols / 64) + c.kb * 4) * kSfAtomBytes, sf_bytes,
                  bar_scales_landed + 8 * stage);
        mbar_expect_tx(bar_full + 8 * stage, kStageCodeBytes);
        tma_load_2d(dst, phase ? &map1 : &map0, c.kb * 128, c.tile * kTileM, bar_full + 8 * stage);
    };
    auto issue_activations = [&](uint32_t stage, const Cursor& c) {
        const TcPhase& ph = p.phase[p.step[c.step].phase];
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
            mbar_init(bar_scales_ready + 8 * s, 2);    // one arrival per copy thread
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 8);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        *input_ready = 0;
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
    if (threadIdx.x >= 64 && threadIdx.x < 64 + 8) collected[threadIdx.x - 64] = 0;
    if (threadIdx.x == 64) *beyond = 0;
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
        // ---------------- TMA producer, weights: runs ahead as far as the ring allows ----------------
        while (weights_left) {
            // stage of step `weights_issued`: free once the MMAs of the step kStages before it are complete
            const uint32_t stage = weights_issued % kStages, round = weights_issued / kStages;
            if (!mbar_wait(bar_empty + 8 * stage, (round - 1) & 1, abort_flag, p.header, kErrTcProducer)) break;
            issue_weights(stage, weights_at);
            ++weights_issued;
            weights_left = cursor_next(p, weights_at);
        }
    } else if (warp == 11 && lane == 0) {
        // ---------------- TMA producer, activations: a stage's half follows as soon as the stage is free and the
        // split it comes from is complete in every CTA ----------------
        Cursor acts_at;
        bool acts_left = cursor_begin(p, acts_at);
        uint32_t acts_issued = 0, idle = 0, polls = 0, open_jobs = 0;   // jobs 0 .. open_jobs - 1 are known to be complete
        while (acts_left) {
            const uint32_t stage = acts_issued % kStages, round = acts_issued / kStages;
            const uint32_t job = p.step[acts_at.step].job;
            bool progressed = false;
            if (round != 0 && !mbar_wait(bar_empty + 8 * stage, (round - 1) & 1, abort_flag, p.header, kErrTcProducer)) break;
            {
                if (open_jobs <= job) {
                    // job 0: this CTA's workers have been through the meeting behind it; later jobs: every CTA has
                    // arrived at the wave's second counter
                    bool open = *input_ready != 0;
                    __threadfence_block();
                    if (open && job != 0) {
                        open = counter_read(p.header + kHeaderWave + *wave_set * 4 + (job - 1) * 2 + 1) >= gridDim.x;
                        if (!open && ++polls > kGridWaitLimit) idle = kWaitLimit;   // a poll of global memory takes about a microsecond
                    }
                    if (open) {
                        // the split activations were written with ordinary stores, by this and other CTAs
                        asm volatile("fence.proxy.async;" ::: "memory");
                        open_jobs = job + 1;
                    }
                }
                if (open_jobs > job) {
                    issue_activations(stage, acts_at);
                    ++acts_issued;
                    acts_left = cursor_next(p, acts_at);
                    progressed = true;
                }
            }
            if (progressed) {
                idle = 0;
            } else {
                if (job == 0) __nanosleep(100);   // polling shared memory: leave the issue slots to the warps that are splitting
                if (++idle > kWaitLimit / 8 || ((idle & 255u) == 255u && *abort_flag)) {
                    *abort_flag = 1;
                    atomicCAS(p.header, 0u, kErrTcProducer);
                    break;
                }
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
                if (!mbar_wait(bar_acc_empty + 8 * buffer, acc_phase[buffer] ^ 1, abort_flag, p.header, kErrTcAccEmpty)) break;
                tc_fence_after();
            }
            const uint32_t acc = tmem_base + kTmemAcc + buffer * 64;
            const uint32_t stage = step % kStages, parity = (step / kStages) & 1;
            // operands in shared memory (TMA) and their block scales on the way to tensor memory (copy thread):
            // a copy and a later MMA execute in issue order, so the copies only have to be issued
            if (!mbar_wait(bar_full + 8 * stage, parity, abort_flag, p.header, kErrTcFull) ||
                !mbar_wait(bar_scales_ready + 8 * stage, parity, abort_flag, p.header, kErrTcScalesReady)) {
                break;
            }
            tc_fence_after();
            const uint32_t stage_smem = smem_u32(smem + stage * kStageBytes);
            const uint64_t weight_desc = operand_desc(stage_smem), act_desc = operand_desc(stage_smem + kStageActCodes);
            const uint32_t tmem_sf_weight = tmem_base + kTmemSfWeight + stage * 16, tmem_sf_act = tmem_base + kTmemSfAct + stage * 16;
            const uint32_t k_steps = min(kStageK, p.phase[p.step[c.step].phase].cols - c.kb * kStageK) / 64;
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
    } else if ((warp == 10 || warp == 12) && lane == 0) {
        // ---------------- scale copies: shared memory -> tensor memory, as soon as a stage's scales have landed ----------------
        // Two threads, one for the weights' scales and one for the activations': a thread gets one copy accepted
        // about every hundred cycles. A stage's scale columns in tensor memory are free when its scales land again:
        // the producer refilled the stage only after the MMAs that read those columns were complete.
        const bool weights = warp == 10;
        uint32_t step = 0;
        Cursor c;
        bool more = cursor_begin(p, c);
        while (more) {
            const uint32_t stage = step % kStages, parity = (step / kStages) & 1;
            if (!mbar_wait(bar_scales_landed + 8 * stage, parity, abort_flag, p.header, kErrTcScalesLanded)) break;
            tc_fence_after();
            const uint32_t stage_smem = smem_u32(smem + stage * kStageBytes);
            const uint64_t desc = sf_desc(stage_smem + (weights ? kStageCodeBytes : kStageActSf));
            const uint32_t columns = tmem_base + (weights ? kTmemSfWeight : kTmemSfAct) + stage * 16;
            const uint32_t k_steps = min(kStageK, p.phase[p.step[c.step].phase].cols - c.kb * kStageK) / 64;
            if (k_steps == 4) {
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k) tc_copy_sf(columns + 4 * k, desc + k * (kSfAtomBytes >> 4));
            } else {
                for (uint32_t k = 0; k < k_steps; ++k) tc_copy_sf(columns + 4 * k, desc + k * (kSfAtomBytes >> 4));
            }
            tc_fence_before();
            mbar_arrive(bar_scales_ready + 8 * stage);
            ++step;
            more = cursor_next(p, c);
        }
    } else if (warp >= 2 && warp < 10) {
        // ---------------- workers: split activations, run the epilogues ----------------
        const uint32_t worker = threadIdx.x - 64, quadrant = warp & 3;   // tensor-memory lanes of this warp: 32 * quadrant .. + 31
        const uint32_t token0 = ((warp - 2) >> 2) * 4;                   // and its four token rows
        const bool leader = worker == 0;
        const uint32_t first_pair = (blockIdx.x * 8 + (warp - 2)) * 2 + (lane >> 4), pair_stride = gridDim.x * 16;   // this half warp's groups of a job
        uint32_t item_count = 0;
        uint32_t acc_phase[2] = {0, 0};
        uint32_t held[kHeld], largest[kHeld];
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations may come from the launch before this one; all stores follow
        uint32_t meeting = 0, parity = 0;
        uint32_t* wave = nullptr;                              // this launch's wave counters: [wave]{outputs stored, split stored}
        if (leader) {
            meeting = *static_cast<volatile uint32_t*>(p.header + kHeaderEpoch);   // left by the launch before
            parity = *static_cast<volatile uint32_t*>(p.header + kHeaderParity);
            wave = p.header + kHeaderWave + parity * 4;
            *wave_set = parity;
            if (blockIdx.x == 0) {
                // the other half of the wave counters belongs to the launch before (complete) and to the launch after;
                // the maxima of the later jobs were last read by the launch before and are added to only by CTAs
                // that have been through a full meeting, i.e. after this CTA has arrived there
                for (uint32_t i = 0; i < 4; ++i) p.header[kHeaderWave + (parity ^ 1) * 4 + i] = 0;
                for (uint32_t i = 8; i < 8 * p.jobs; ++i) p.header[kHeaderRowMax + i] = 0;
            }
        }
        bool alive = true;
        {
            // ---- job 0: the input of the first step comes from outside ----
            // Its row maxima would take a meeting of their own. Instead every CTA looks at the same sample, the first
            // 256 elements of every row, takes the anchors three binades above the sample's maxima, and splits its
            // share with them; a CTA that finds a group beyond its row's anchor says so as it arrives at the meeting
            // that follows the split, and then all CTAs do the split again with the true maxima, which they have
            // collected on the way. Which of the two happens depends on the input alone.
            const TcJob& job = p.job[0];
            const TcPhase& ph = p.phase[job.phase];
#pragma unroll
            for (uint32_t j = 0; j < kHeld; ++j) held[j] = load_element(ph, job, p.tokens, first_pair + j * pair_stride, lane);
            {
                const uint32_t token = worker >> 5;   // a warp per token row
                uint32_t packed = 0;
                if (token < p.tokens) {
                    const uint4* row = reinterpret_cast<const uint4*>(ph.x + static_cast<uint64_t>(token) * ph.cols);
                    for (uint32_t i = lane; i < min(ph.cols, 256u) / 8; i += 32) {
                        const uint4 v = __ldcg(row + i);
                        packed = __vmaxu2(packed, __vmaxu2(__vmaxu2(v.x & 0x7fff7fffu, v.y & 0x7fff7fffu), __vmaxu2(v.z & 0x7fff7fffu, v.w & 0x7fff7fffu)));
                    }
                }
                uint32_t most = max(packed & 0xffffu, packed >> 16);
                most = max(most, __shfl_xor_sync(0xffffffffu, most, 16));
                most = max(most, __shfl_xor_sync(0xffffffffu, most, 8));
                most = max(most, __shfl_xor_sync(0xffffffffu, most, 4));
                most = max(most, __shfl_xor_sync(0xffffffffu, most, 2));
                most = max(most, __shfl_xor_sync(0xffffffffu, most, 1));
                if (lane == 0) {
                    // term 0 of the row has the global scale 2^(A - 155), term 7 2^(A - 134): all normal f32 numbers
                    const uint32_t a = min(max((most >> 7) + 3, 40u), 250u);
                    anchor[token] = a;
                    term_scale[token] = __uint_as_float((a - 28) << 23);
                }
            }
            workers_sync();
            // the other half of the trailer belongs to the launch before (complete) and to the launch after
            for (uint32_t i = blockIdx.x * kWorkers + worker; i < 2 * kMaxCtas; i += gridDim.x * kWorkers) p.slots[(*wave_set ^ 1) * 2 * kMaxCtas + i] = 0;
            share_codes(p, 0, held, largest, collected, first_pair, pair_stride, lane);
            if (share_scales(p, 0, anchor, held, largest, first_pair, pair_stride, lane)) *beyond = 1;   // any lane; a non-finite element is beyond too
            workers_sync();
            if (worker < 8) {
                if (collected[worker]) atomicMax(p.header + kHeaderRowMax + worker, collected[worker]);
                collected[worker] = 0;
            }
            // every CTA's slice is in place before any CTA loads from the split (the thread that issues the loads puts
            // a proxy fence between the meeting and them)
            alive = grid_meet(p, leader, meeting, *beyond != 0, raised, abort_flag);
            if (alive && *raised) {
                job_scales(p, 0, worker, term_scale, anchor);
                share_codes(p, 0, held, largest, nullptr, first_pair, pair_stride, lane);
                share_scales(p, 0, anchor, held, largest, first_pair, pair_stride, lane);
                alive = grid_meet(p, leader, meeting, false, raised, abort_flag);
            }
            if (alive) {
                if (blockIdx.x == 0 && worker < 8) p.header[kHeaderRowMax + worker] = 0;   // clean for the next launch
                if (leader) {
                    __threadfence_block();
                    *input_ready = 1;
                }
            }
        }
        for (uint32_t s = 0; alive && s < p.steps; ++s) {
            const TcStep& st = p.step[s];
            const TcPhase& ph = p.phase[st.phase];
            uint32_t* gather = st.feeds ? collected : nullptr;
            uint32_t kept[5] = {0, 0, 0, 0, 0};             // lanes 0..15: the outputs of this warp's 16 columns and 4 token rows, as stored; their exponent fields
            uint32_t kept_group = ~0u;                      // their 16-element group in the rows of the next product's input
            // ---- epilogues of this CTA's items of the step ----
            const uint32_t items = st.tiles * st.parts;
            for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++item_count) {
                const uint32_t tile = item / st.parts, part = item - tile * st.parts;
                const uint32_t buffer = item_count & 1;
                if (!mbar_wait_suspended(bar_acc_full + 8 * buffer, acc_phase[buffer], abort_flag, p.header, kErrTcAccFull)) {
                    alive = false;
                    break;
                }
                acc_phase[buffer] ^= 1;
                tc_fence_after();
                // column = term * 8 + token: this warp's four token rows are four neighbouring columns of every term
                uint32_t v[kTerms][4];
                const uint32_t taddr = tmem_base + kTmemAcc + buffer * 64 + token0 + ((quadrant * 32) << 16);
#pragma unroll
                for (uint32_t term = 0; term < kTerms; ++term) tc_load4(taddr + 8 * term, v[term]);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buffer);   // the buffer is free for the item after next
                float y[4];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    // term t carries the factor 8^t relative to term 0
                    float sum = 0.0f, factor = 1.0f;
#pragma unroll
                    for (uint32_t term = 0; term < kTerms; ++term) {
                        sum = fmaf(__uint_as_float(v[term][j]), factor, sum);
                        factor *= 8.0f;
                    }
                    y[j] = sum * term_scale[8 * st.job + token0 + j];
                }
                contribute_rows(ph, p.tokens, st.tile0 + tile, quadrant, token0, st.slot0 + part, lane, y, gather, st.keeps ? kept : nullptr);
                kept_group = (st.tile0 + tile) * 4 + quadrant;
            }
            if (!alive || !st.feeds) continue;
            // ---- this step's outputs are the activations of job `feeds`: maxima, arrive, wait, split, arrive ----
            const uint32_t w = st.feeds - 1;
            const TcJob& job = p.job[st.feeds];
            const TcPhase& next = p.phase[job.phase];
            const SplitTarget to = split_target(p, st.feeds);
            if (st.keeps && lane == 0) gathered[warp - 2] = kept[4];   // warps 2..5: token rows 0..3, warps 6..9: rows 4..7
            workers_sync();
            if (st.keeps) {
                // this CTA's maxima as one word of its own: exponent fields, one byte per token row (40 at least, so the
                // word is never 0; 251 for a non-finite value). Nothing has to be visible with it, so no release.
                if (worker < 32) {   // the first worker warp: lanes 0..7 a token row each, then the eight bytes gathered in lane 0
                    uint32_t low = 0, high = 0;
                    if (lane < 8) {
                        uint32_t field = 0;
                        for (uint32_t k = 0; k < 4; ++k) field = max(field, (gathered[(lane >> 2) * 4 + k] >> (8 * (lane & 3))) & 0xffu);
                        const uint32_t byte = (field >= 255 ? 251u : min(max(field, 40u), 250u)) << (8 * (lane & 3));
                        low = lane < 4 ? byte : 0;
                        high = lane < 4 ? 0 : byte;
                    }
#pragma unroll
                    for (uint32_t offset = 4; offset; offset >>= 1) {
                        low |= __shfl_xor_sync(0xffffffffu, low, offset);
                        high |= __shfl_xor_sync(0xffffffffu, high, offset);
                    }
                    if (lane == 0) {
                        const unsigned long long word = (static_cast<unsigned long long>(high) << 32) | low;
                        asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p.slots + (*wave_set * 2 + w) * kMaxCtas + blockIdx.x), "l"(word) : "memory");
                    }
                }
                workers_sync();   // `gathered` is used again below
            } else {
                if (worker < 8) {
                    if (collected[worker]) atomicMax(p.header + kHeaderRowMax + 8 * st.feeds + worker, collected[worker]);
                    collected[worker] = 0;
                }
                workers_sync();
                if (leader) counter_arrive_only(wave + 2 * w);
            }
            // While the other CTAs arrive: every warp writes the codes of the 16 columns and 4 token rows it has just
            // computed, from registers: lanes 0..15 take its first two token rows, lanes 16..31 the other two, a group each.
            uint2 where[2];
            uint32_t bits[2] = {0, 0};
            if (st.keeps && kept_group != ~0u) {
#pragma unroll
                for (uint32_t j = 0; j < 2; ++j) {
                    const uint32_t token = token0 + j + ((lane >> 4) << 1);
                    const uint32_t theirs = __shfl_sync(0xffffffffu, kept[2 + j], lane & 15);
                    where[j] = make_uint2(token < p.tokens ? token : ~0u, kept_group);
                    bits[j] = lane < 16 ? kept[j] : theirs;
                    largest[j] = split_codes(to, where[j], bits[j], 0, lane);
                }
            }
            if (st.keeps) {
                // every CTA's word: a worker reads a few until they are written, the warps and then the CTA combine them
                uint32_t low = 0, high = 0;
                for (uint32_t first = worker; first < gridDim.x; first += 4 * kWorkers) {
                    unsigned long long word[4];
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {   // all at once; one that is not written yet is read again below
                        word[k] = 0x2828282828282828ull;
                        if (first + k * kWorkers < gridDim.x) {
                            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word[k]) : "l"(p.slots + (*wave_set * 2 + w) * kMaxCtas + first + k * kWorkers) : "memory");
                        }
                    }
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {
                        for (uint32_t spin = 0; word[k] == 0;) {
                            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word[k]) : "l"(p.slots + (*wave_set * 2 + w) * kMaxCtas + first + k * kWorkers) : "memory");
                            if (word[k] == 0 && (++spin > kGridWaitLimit || ((spin & 255u) == 255u && *abort_flag))) {
                                *abort_flag = 1;
                                atomicCAS(p.header, 0u, kErrTcWave);
                                break;
                            }
                        }
                        low = __vmaxu4(low, static_cast<uint32_t>(word[k]));
                        high = __vmaxu4(high, static_cast<uint32_t>(word[k] >> 32));
                    }
                }
#pragma unroll
                for (uint32_t offset = 16; offset; offset >>= 1) {
                    low = __vmaxu4(low, __shfl_xor_sync(0xffffffffu, low, offset));
                    high = __vmaxu4(high, __shfl_xor_sync(0xffffffffu, high, offset));
                }
                if (lane == 0) {
                    gathered[(warp - 2) * 2] = low;
                    gathered[(warp - 2) * 2 + 1] = high;
                }
                workers_sync();
                if (worker < 8) {
                    uint32_t field = 0;
                    for (uint32_t k = 0; k < 8; ++k) field = max(field, (gathered[k * 2 + (worker >> 2)] >> (8 * (worker & 3))) & 0xffu);
                    // term 0 of the row has the global scale 2^(A - 155), term 7 2^(A - 134): all normal f32 numbers
                    const uint32_t a = min(field, 250u);
                    term_scale[8 * st.feeds + worker] = field > 250 ? __uint_as_float(0x7fc00000u) : __uint_as_float((a - 28) << 23);
                    anchor[8 * st.feeds + worker] = a;
                }
                workers_sync();
            } else {
                if (leader) counter_wait(p, wave + 2 * w, kErrTcWave, abort_flag);
                workers_sync();
            }
            if (*abort_flag) {
                alive = false;
                break;
            }
            if (!st.keeps) job_scales(p, st.feeds, worker, term_scale, anchor);
            if (st.keeps) {
                if (kept_group != ~0u) {
#pragma unroll
                    for (uint32_t j = 0; j < 2; ++j) split_scales(to, anchor + 8 * st.feeds, where[j], bits[j], largest[j], lane);
                }
            } else {
                // items of several CTAs per tile, or several items per CTA: the outputs are read back, every CTA a share
#pragma unroll
                for (uint32_t j = 0; j < kHeld; ++j) held[j] = load_element(next, job, p.tokens, first_pair + j * pair_stride, lane);
                share_codes(p, st.feeds, held, largest, nullptr, first_pair, pair_stride, lane);
                share_scales(p, st.feeds, anchor, held, largest, first_pair, pair_stride, lane);
            }
            workers_sync();
            if (leader) counter_arrive_only(wave + 2 * w + 1);
            if (st.keeps && kept_group != ~0u) {
                // the outputs themselves, last: nobody in this launch reads them back, and neither arrival above had to
                // wait for them
                if (lane < 16) {
                    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(ph.out);
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        if (token0 + j < p.tokens) out[static_cast<uint64_t>(token0 + j) * ph.out_rows + kept_group * 16 + lane] = __ushort_as_bfloat16(static_cast<unsigned short>(kept[j]));
                    }
                }
            }
        }
        // the next launch goes on counting meetings where this one stopped, with the other half of the wave counters
        if (alive && leader && blockIdx.x == 0) {
            p.header[kHeaderEpoch] = meeting;
            p.header[kHeaderParity] = parity ^ 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------------
// Equal k ranges per tile of a step with `tiles` tiles over `k_blocks` stages on `ctas` CTAs: whole tiles when
// there are more tiles than half the CTAs, otherwise as many parts as CTAs per tile (at least two stages per
// part, at most 16 parts).
uint32_t parts_for(uint32_t tiles, uint32_t k_blocks, uint32_t ctas) {
    if (tiles * 2 > ctas) return 1;
    uint32_t parts = ctas / tiles;
    if (parts > k_blocks / 2) parts = k_blocks / 2;
    if (parts > 16) parts = 16;
    return parts > 1 ? parts : 1;
}

struct TcProgram {
    TcJob job[kMaxJobs];
    TcStep step[kMaxSteps];
    uint32_t jobs, steps, ctas;
    uint32_t contributors[kMaxPhases];
};

// The steps of a linear (`b` null) or of the MLP block on a device with `sm_count` SMs.
TcProgram tc_program(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, const augur_cuda_nvfp4_sm100_gemv_args_v1* b, uint32_t sm_count) {
    TcProgram g{};
    const uint32_t slots = sm_count * kCtasPerSm;   // CTAs resident at once
    const uint32_t rows_a = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 ? 2 * a->rows : a->rows;
    const uint32_t tiles_a = rows_a / kTileM, kb_a = (a->cols + kStageK - 1) / kStageK;
    g.job[0] = TcJob{0, 0, a->cols / 16};
    g.jobs = 1;
    if (!b) {
        const uint32_t parts = parts_for(tiles_a, kb_a, slots);
        g.step[0] = TcStep{0, 0, 0, tiles_a, 0, kb_a, parts, 0, 0, 0};
        g.steps = 1;
        g.contributors[0] = parts;
        g.ctas = tiles_a * parts < slots ? tiles_a * parts : slots;
        return g;
    }
    // gate|up in whole tiles, in two waves when there are more tiles than CTAs: a wave's outputs are 64 columns of
    // the intermediate per tile, and the first wave must end on a k block of the second product
    const uint32_t tiles_b = b->rows / kTileM, kb_b = (b->cols + kStageK - 1) / kStageK;
    uint32_t first = tiles_a;
    if (tiles_a > slots && (slots & ~3u) != 0) first = slots & ~3u;
    g.ctas = slots;
    g.contributors[0] = 1;
    uint32_t s = 0;
    g.step[s++] = TcStep{0, 0, 0, first, 0, kb_a, 1, 0, 1, first <= slots && slots <= kMaxCtas ? 1u : 0u};
    g.job[1] = TcJob{1, 0, first * 4};
    g.jobs = 2;
    if (first < tiles_a) {
        g.step[s++] = TcStep{0, 0, first, tiles_a - first, 0, kb_a, 1, 0, 2, tiles_a - first <= slots && slots <= kMaxCtas ? 1u : 0u};
        g.job[2] = TcJob{1, first * 4, b->cols / 16 - first * 4};
        g.jobs = 3;
    }
    const uint32_t kb_first = first < tiles_a ? first / 4 : kb_b;
    const uint32_t parts_first = parts_for(tiles_b, kb_first, slots);
    g.step[s++] = TcStep{1, 1, 0, tiles_b, 0, kb_first, parts_first, 0, 0, 0};
    g.contributors[1] = parts_first;
    if (first < tiles_a) {
        const uint32_t parts_rest = parts_for(tiles_b, kb_b - kb_first, slots);
        g.step[s++] = TcStep{1, 2, 0, tiles_b, kb_first, kb_b, parts_rest, parts_first, 0, 0};
        g.contributors[1] += parts_rest;
    }
    g.steps = s;
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

// What a phase needs of the plan scratch behind the counter regions: the split activations, then the partial
// sums of `contributors` items per tile.
uint64_t tc_scratch_need(uint32_t physical_rows, uint32_t cols, uint32_t contributors) {
    const uint64_t partial_bytes = contributors > 1 ? static_cast<uint64_t>(physical_rows / kTileM) * 4 * contributors * kSlotFloats * 4 : 0;
    return (split_bytes(cols) + 255) / 256 * 256 + partial_bytes;
}

// Scalars, extents, scratch room (`offset` .. `limit` of the plan scratch) and aliasing of one phase.
bool check_tc(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
              const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t contributors, uint64_t offset, uint64_t limit, bool full,
              augur_cuda_result_v1* failure) {
    *failure = invalid();
    uint32_t physical_rows = 0;
    if (!check_tc_scalars(a, &physical_rows)) return false;
    if (physical_rows / kTileM * 8 > kMaxGroups || offset < kCounterBytes || offset % 256 != 0 || limit < offset ||
        tc_scratch_need(physical_rows, a->cols, contributors) > limit - offset) {
        return false;
    }
    const Range r[4] = {{a->weight, a->weight_len_bytes, 256}, {a->input_bf16, a->input_len_bytes, 16},
                        {a->output, a->output_len_bytes, 4}, plan_scratch_range(plan)};
    if (!all_disjoint(r, 4)) return false;
    return !full || inspect_device_ranges(d, r, 3, failure);
}

bool check_tc_header(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan, const void* a, uint32_t abi_version,
                     bool header, augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header) {
        if (a && s && d >= 0 && s->ordinal == d && abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    return plan_ok(plan, d, s);
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

// One launch for a linear (`b` null) or the MLP block. Member m uses counter region m and the scratch at offsets[m].
augur_cuda_result_v1 launch_tc(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                               const augur_cuda_nvfp4_sm100_gemv_args_v1* a, const augur_cuda_nvfp4_sm100_gemv_args_v1* b,
                               const uint64_t (&offsets)[2]) {
    const augur_cuda_nvfp4_sm100_gemv_args_v1* members[2] = {a, b};
    const TcProgram g = tc_program(a, b, plan->sm_count);
    CUtensorMap maps[2];
    TcParams p{};
    p.tokens = a->tokens;
    p.header = plan->status_word;
    p.slots = reinterpret_cast<unsigned long long*>(plan->scratch + plan->scratch_bytes);
    p.jobs = g.jobs;
    p.steps = g.steps;
    for (uint32_t j = 0; j < g.jobs; ++j) p.job[j] = g.job[j];
    for (uint32_t i = 0; i < g.steps; ++i) p.step[i] = g.step[i];
    for (uint32_t m = 0; m < (b ? 2u : 1u); ++m) {
        const augur_cuda_nvfp4_sm100_gemv_args_v1* args = members[m];
        const uint32_t physical_rows = physical_rows_of(args);
        if (!weight_map(&maps[m], args->weight, physical_rows, args->cols)) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
        TcPhase& ph = p.phase[m];
        ph.weight_sf = reinterpret_cast<const uint8_t*>(args->weight) + tcgen05_codes_bytes(physical_rows, args->cols);
        ph.x = reinterpret_cast<const uint16_t*>(args->input_bf16);
        ph.split = plan->scratch + offsets[m];
        ph.out = reinterpret_cast<void*>(args->output);
        ph.counters = reinterpret_cast<uint32_t*>(plan->scratch + m * kCounterRegionBytes);
        ph.partials = reinterpret_cast<float*>(plan->scratch + offsets[m] + (split_bytes(args->cols) + 255) / 256 * 256);
        ph.rows = physical_rows; ph.out_rows = args->rows; ph.cols = args->cols; ph.epilogue = args->epilogue;
        ph.contributors = g.contributors[m];
        ph.global_a = args->global_scale; ph.global_b = args->global_scale_b;
    }
    if (!b) maps[1] = maps[0];
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config{};
    config.stream = s->stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    config.gridDim = dim3(g.ctas);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    cudaLaunchKernelEx(&config, tc_program_kernel, maps[0], maps[1], p);
    count_launch();
    return submitted();
}

// Contributors per tile of a single linear on a device with `sm_count` SMs.
uint32_t linear_contributors(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t sm_count) { return tc_program(a, nullptr, sm_count).contributors[0]; }

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
    // on any device with up to 512 SMs; the second product of the MLP block has two k ranges, each cut like a linear,
    // and the first has its tiles in two halves
    uint32_t contributors = 2;
    for (uint32_t sms = 1; sms <= 512; ++sms) {
        const uint32_t parts = 2 * parts_for(static_cast<uint32_t>(physical / kTileM), (cols + kStageK - 1) / kStageK, sms * kCtasPerSm);
        if (parts > contributors) contributors = parts;
    }
    *out_bytes = kCounterBytes + (tc_scratch_need(static_cast<uint32_t>(physical), cols, contributors) + 255) / 256 * 256;
    return ok();
}

static_assert(kMaxSteps == 4 && kMaxJobs == 3 && kMaxPhases == 2, "the described program has the kernel's bounds");

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_tc_program_describe_host_v1(
    uint32_t rows_a, uint32_t cols_a, uint32_t epilogue_a, uint32_t rows_b, uint32_t cols_b, uint32_t sm_count,
    augur_cuda_nvfp4_sm100_tc_program_v1* out) {
    if (!out || !sm_count || sm_count > 512) return invalid();
    // the scalar rules of the entries, on the fields that shape the program
    augur_cuda_nvfp4_sm100_gemv_args_v1 a{}, b{};
    a.rows = rows_a;
    a.cols = cols_a;
    a.epilogue = rows_b ? static_cast<uint32_t>(AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) : epilogue_a;
    b.rows = rows_b;
    b.cols = cols_b;
    b.epilogue = AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16;
    for (const augur_cuda_nvfp4_sm100_gemv_args_v1* m : {&a, &b}) {
        if (m == &b && !rows_b) break;
        const uint64_t physical = physical_rows_of(m);
        if (m->epilogue > AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32 || !m->rows || !m->cols || m->rows > (1u << 30) ||
            physical % kTileM != 0 || m->cols % 64 != 0 || physical * m->cols > UINT32_MAX || physical / kTileM * 8 > kMaxGroups) {
            return invalid();
        }
    }
    if (rows_b && (cols_b != rows_a || rows_b != cols_a)) return invalid();   // the second product consumes the first's outputs
    const TcProgram g = tc_program(&a, rows_b ? &b : nullptr, sm_count);
    *out = augur_cuda_nvfp4_sm100_tc_program_v1{};
    out->steps = g.steps;
    out->jobs = g.jobs;
    out->ctas = g.ctas;
    for (uint32_t i = 0; i < kMaxPhases; ++i) out->contributors[i] = g.contributors[i];
    for (uint32_t i = 0; i < g.steps; ++i) {
        const TcStep& st = g.step[i];
        out->step[i] = {st.phase, st.job, st.tile0, st.tiles, st.kb0, st.kb1, st.parts, st.slot0, st.feeds, st.keeps};
    }
    for (uint32_t i = 0; i < g.jobs; ++i) out->job[i] = {g.job[i].phase, g.job[i].group0, g.job[i].groups};
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_tc_header(d, s, plan, a, a ? a->abi_version : 0, header_ok(d, s, a), &failure)) return failure;
    uint32_t physical = 0;
    if (!check_tc_scalars(a, &physical)) return invalid();
    if (!check_tc(d, s, plan, a, linear_contributors(a, plan->sm_count), kCounterBytes, plan->scratch_bytes, true, &failure)) return failure;
    CUtensorMap probe;
    return weight_map(&probe, a->weight, physical_rows_of(a), a->cols) ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_tc_header(d, s, plan, a, a ? a->abi_version : 0, header_ok(d, s, a), &failure)) return failure;
    uint32_t physical = 0;
    if (!check_tc_scalars(a, &physical)) return invalid();
    if (!check_tc(d, s, plan, a, linear_contributors(a, plan->sm_count), kCounterBytes, plan->scratch_bytes, false, &failure)) return failure;
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
    if (!check_tc_header(d, s, plan, a, a ? a->abi_version : 0, header_ok(d, s, a), failure)) return false;
    if (plan->scratch_bytes < kCounterBytes) return false;
    uint32_t physical = 0;
    if (!check_tc_scalars(&a->gate_up, &physical) || !check_tc_scalars(&a->down, &physical)) return false;
    if (a->gate_up.epilogue != AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 || a->down.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
        return false;
    }
    // The intermediate is the one shared range: gate_up writes what down reads.
    if (a->down.input_bf16 != a->gate_up.output || a->down.input_len_bytes != a->gate_up.output_len_bytes ||
        a->down.cols != a->gate_up.rows || a->down.tokens != a->gate_up.tokens || a->down.rows != a->gate_up.cols) {
        return false;
    }
    const TcProgram g = tc_program(&a->gate_up, &a->down, plan->sm_count);
    const uint64_t middle = kCounterBytes + (plan->scratch_bytes - kCounterBytes) / 2 / 256 * 256;
    *down_offset = middle;
    if (!check_tc(d, s, plan, &a->gate_up, g.contributors[0], kCounterBytes, middle, false, failure)) return false;
    if (!check_tc(d, s, plan, &a->down, g.contributors[1], middle, plan->scratch_bytes, false, failure)) return false;
    *failure = invalid();
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
