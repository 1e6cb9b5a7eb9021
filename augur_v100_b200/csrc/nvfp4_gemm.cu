// Prefill NVFP4 linear for sm_100a: BF16 -> NVFP4 activation quantiser and a
// warp-specialised tcgen05 block-scaled GEMM (kind::mxf4nvf4, scale_vec::4X) with
// TMA-fed shared-memory stages and the accumulator in tensor memory.
//
// D[token][feature] = g_w * g_a * sum_terms sum_k A_term[token][k] * W[feature][k]
//   A operand: quantised activations, 128 token rows per tile (UMMA M = 128)
//   B operand: weights, up to 256 feature rows per tile (UMMA N = 128 or 256)
//   both K-major, packed two E2M1 codes per byte, 128-byte swizzled rows of 256 k
//   block scales: 512-byte atoms (128 rows x 4 scales) copied smem -> TMEM by tcgen05.cp
//
// One persistent CTA per SM, 192 threads: warp 0 issues TMA, warp 1 owns tensor memory
// and issues the MMAs, warps 2..5 drain the accumulator (tcgen05.ld), scale, round to
// BF16 and store. Every mbarrier wait is bounded: a wait that runs out records a code in
// the plan's status word, raises a CTA-wide abort flag, and all roles fall through to the
// common exit where tensor memory is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>


#include "nvfp4_internal.h"
#include "nvfp4_layout.cuh"
#include "nvfp4_tc.cuh"

namespace augur_sm100 {
namespace {
using namespace tc;

static_assert(sizeof(augur_cuda_nvfp4_sm100_act_quant_args_v1) == 56, "act_quant ABI");
static_assert(sizeof(augur_cuda_nvfp4_sm100_gemm_args_v1) == 80, "gemm ABI");

constexpr uint32_t kTileN = 256;          // features per tile (128 for a ragged last tile)
constexpr uint32_t kBlockK = 256;         // k per shared-memory stage = one 128-byte swizzled row
constexpr uint32_t kStages = 4;
constexpr uint32_t kBytesA = kTileM * 128;            // 16 KB
constexpr uint32_t kBytesB = kTileN * 128;            // 32 KB
constexpr uint32_t kBytesSfA = 4 * kSfAtomBytes;      // 2 KB: 4 atoms (k) of one 128-row block
constexpr uint32_t kBytesSfB = 8 * kSfAtomBytes;      // 4 KB: 2 row blocks x 4 atoms
constexpr uint32_t kStageBytes = kBytesA + kBytesB + kBytesSfA + kBytesSfB;  // 55296
constexpr uint32_t kGemmSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kGemmThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemAcc = 0;          // 256 accumulator columns
constexpr uint32_t kTmemSfA = 256;        // 2 x 16 columns (k-block parity)
constexpr uint32_t kTmemSfB = 320;        // 2 x 32 columns

constexpr uint32_t kErrProducerWait = 0x101, kErrMmaWaitFull = 0x102, kErrMmaWaitTmem = 0x103,
                   kErrEpilogueWait = 0x104, kErrCopyWait = 0x105, kErrMmaWaitScales = 0x106,
                   kErrSplitWait = 0x107;

struct GemmParams {
    const uint8_t* weight_sf;      // scale region of the weight tensor
    const uint8_t* act_sf;         // scale region of term 0; terms are `act_term_stride` bytes apart
    uint64_t act_term_stride;
    __nv_bfloat16* out;
    uint32_t* status_word;
    uint32_t rows, cols, tokens, terms;
    uint32_t padded_tokens;        // tokens rounded up to whole 128-row tiles: row stride of the staged activation planes
    float scale;                   // g_w * g_a
    float scale_b;                 // SwiGLU: g_w of the up rows * g_a
    uint32_t swiglu;               // weight rows alternate 16 gate / 16 up; output is bf16(silu(gate) * up), rows / 2 wide
    // SwiGLU on pair tiles only: the intermediate is also (or only, if `out` is null) quantised for the next GEMM
    uint8_t* quant_out;            // staged activations: [terms] code planes of whole tiles, then the scale regions
    uint32_t quant_terms;
    float quant_global_scale;
    // Pair tiles whose count is not a multiple of the pairs: the tiles left over are cut along k between all pairs
    // (null: whole tiles only). Partial accumulators pass through `split_slots`, announced by `split_flags`.
    float* split_slots;            // [pair][CTA of the pair][epilogue warp][128 columns / 4][lane] x float4
    uint32_t* split_flags;         // [pair][CTA of the pair][epilogue warp], zero between launches
    uint32_t split_sharers;        // pairs that share the leftover tiles (0: whole tiles only)
};

// ---- activation quantiser ------------------------------------------------------------------
__host__ __device__ constexpr uint32_t padded_tokens(uint32_t tokens) { return (tokens + kTileM - 1) / kTileM * kTileM; }
// Bytes of the staged activations of one term: code plane of whole tiles, then the scale atoms.
__host__ __device__ constexpr uint64_t staged_term_bytes(uint32_t tokens, uint32_t cols) {
    return tcgen05_extent_bytes(padded_tokens(tokens), cols);
}


// 32 accumulator columns of one token row -> packed BF16. Plain: 32 outputs. SwiGLU: the weight rows
// alternate 16 gate / 16 up, so columns 0..15 are gate sums and 16..31 the matching up sums of 16
// intermediate columns; the 16 outputs bf16(silu(gate) * up) fill packed[0..8).
__device__ __forceinline__ void convert_chunk(const uint32_t (&v)[32], float scale, float scale_b, bool swiglu, uint32_t (&packed)[16]) {
    if (!swiglu) {
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i) {
            const __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(v[2 * i]) * scale, __uint_as_float(v[2 * i + 1]) * scale);
            packed[i] = *reinterpret_cast<const uint32_t*>(&two);
        }
        return;
    }
    float h[16];
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) {
        const float gate = __uint_as_float(v[i]) * scale, up = __uint_as_float(v[16 + i]) * scale_b;
        // fast exponential and reciprocal (a few 1e-7 relative): this runs between the accumulator read and
        // its release, in front of the next tile's MMAs. A gate below -87 gives exp = inf and h = -0.
        h[i] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
    }
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const __nv_bfloat162 two = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
        packed[i] = *reinterpret_cast<const uint32_t*>(&two);
    }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_weight,
            const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte alignment.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    // bars[0..S) full, [S..2S) empty, [2S] tmem_full, [2S+1] tmem_empty; then tmem base + abort flag
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
    const uint32_t bar_tmem_full = smem_u32(bars + 2 * kStages), bar_tmem_empty = smem_u32(bars + 2 * kStages + 1);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_tmem_full, 1);
        mbar_init(bar_tmem_empty, 4);   // one arrival per epilogue warp
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t m_tiles = p.padded_tokens / kTileM;
    const uint32_t n_tiles = (p.rows + kTileN - 1) / kTileN;
    const uint32_t total_tiles = m_tiles * n_tiles;
    const uint32_t k_blocks = (p.cols + kBlockK - 1) / kBlockK;
    const uint32_t steps = k_blocks * p.terms;              // pipeline steps per tile
    const uint64_t sf_atoms_per_row_block = p.cols / 64;    // atoms along k

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        uint32_t stage = 0, phase = 0;
        bool alive = true;
        for (uint32_t tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x) {
            const uint32_t m_tile = tile % m_tiles, n_tile = tile / m_tiles;
            const uint32_t n_rows = min(kTileN, p.rows - n_tile * kTileN);
            for (uint32_t step = 0; step < steps; ++step) {
                const uint32_t kb = step / p.terms, term = step % p.terms;
                const uint32_t k_valid = min(kBlockK, p.cols - kb * kBlockK);   // multiple of 64
                const uint32_t sf_bytes = k_valid / 64 * kSfAtomBytes;
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status_word, kErrProducerWait)) {
                    alive = false;
                    break;
                }
                uint8_t* base = smem + stage * kStageBytes;
                const uint32_t full = bar_full + 8 * stage;
                const uint32_t row_blocks_b = n_rows / 128;
                mbar_expect_tx(full, kBytesA + n_rows * 128 + sf_bytes * (1 + row_blocks_b));
                tma_load_2d(smem_u32(base), &map_act, kb * 128, term * p.padded_tokens + m_tile * kTileM, full);
                tma_load_2d(smem_u32(base + kBytesA), &map_weight, kb * 128, n_tile * kTileN, full);
                if (n_rows > 128) {
                    tma_load_2d(smem_u32(base + kBytesA + 128 * 128), &map_weight, kb * 128, n_tile * kTileN + 128, full);
                }
                const uint8_t* sfa = p.act_sf + term * p.act_term_stride +
                                     (static_cast<uint64_t>(m_tile) * sf_atoms_per_row_block + kb * 4) * kSfAtomBytes;
                bulk_load(smem_u32(base + kBytesA + kBytesB), sfa, sf_bytes, full);
                for (uint32_t rb = 0; rb < row_blocks_b; ++rb) {
                    const uint8_t* sfb = p.weight_sf +
                        ((static_cast<uint64_t>(n_tile) * 2 + rb) * sf_atoms_per_row_block + kb * 4) * kSfAtomBytes;
                    bulk_load(smem_u32(base + kBytesA + kBytesB + kBytesSfA + rb * kBytesSfA), sfb, sf_bytes, full);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        uint32_t stage = 0, phase = 0, tmem_phase = 0, sf_buffer = 0;
        bool alive = true;
        for (uint32_t tile = blockIdx.x; alive && tile < total_tiles; tile += gridDim.x) {
            const uint32_t n_tile = tile / m_tiles;
            const uint32_t n_rows = min(kTileN, p.rows - n_tile * kTileN);
            const uint32_t idesc = instr_desc(n_rows);
            // the epilogue must have drained the previous tile's accumulator
            if (!mbar_wait(bar_tmem_empty, tmem_phase ^ 1, abort_flag, p.status_word, kErrMmaWaitTmem)) break;
            tc_fence_after();
            for (uint32_t step = 0; step < steps; ++step) {
                const uint32_t kb = step / p.terms;
                const uint32_t k_valid = min(kBlockK, p.cols - kb * kBlockK);
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status_word, kErrMmaWaitFull)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint32_t base = smem_u32(smem + stage * kStageBytes);
                const uint32_t sfa_smem = base + kBytesA + kBytesB, sfb_smem = sfa_smem + kBytesSfA;
                const uint32_t tmem_sfa = tmem_base + kTmemSfA + sf_buffer * 16;
                const uint32_t tmem_sfb = tmem_base + kTmemSfB + sf_buffer * 32;
                const uint64_t a_desc = operand_desc(base), b_desc = operand_desc(base + kBytesA);
                for (uint32_t k = 0; k < k_valid / 64; ++k) {
                    tc_copy_sf(tmem_sfa + 4 * k, sf_desc(sfa_smem + k * kSfAtomBytes));
                    tc_copy_sf(tmem_sfb + 8 * k, sf_desc(sfb_smem + k * kSfAtomBytes));
                    if (n_rows > 128) tc_copy_sf(tmem_sfb + 8 * k + 4, sf_desc(sfb_smem + kBytesSfA + k * kSfAtomBytes));
                    // each MMA consumes 64 k = 32 bytes of every row: advance the start address by 32 >> 4
                    tc_mma(tmem_base + kTmemAcc, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_sfa + 4 * k,
                           tmem_sfb + 8 * k, (step | k) ? 1u : 0u);
                }
                tc_commit(bar_empty + 8 * stage);   // frees the stage when these MMAs have read it
                sf_buffer ^= 1;
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
            if (alive) tc_commit(bar_tmem_full);      // accumulator complete
            tmem_phase ^= 1;
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: TMEM -> registers -> BF16 -> global ----------------
        const uint32_t quadrant = warp & 3;          // TMEM lanes this warp may read: 32*quadrant..+31
        uint32_t tmem_phase = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const uint32_t m_tile = tile % m_tiles, n_tile = tile / m_tiles;
            const uint32_t n_rows = min(kTileN, p.rows - n_tile * kTileN);
            if (!mbar_wait(bar_tmem_full, tmem_phase, abort_flag, p.status_word, kErrEpilogueWait)) break;
            tc_fence_after();
            const uint32_t token = m_tile * kTileM + quadrant * 32 + lane;
            // SwiGLU halves the output width: 32 accumulator columns give 16 outputs
            const uint32_t out_width = p.swiglu ? p.rows / 2 : p.rows, out_first = p.swiglu ? n_tile * kTileN / 2 : n_tile * kTileN;
            __nv_bfloat16* out_row = p.out + static_cast<uint64_t>(token) * out_width + out_first;
            for (uint32_t c = 0; c < n_rows; c += 32) {
                uint32_t v[32];
                tc_load32(tmem_base + kTmemAcc + ((quadrant * 32) << 16) + c, v);
                tc_wait_ld();
                if (token >= p.tokens) continue;   // padding rows of the last tile are computed, never stored
                uint32_t packed[16];
                convert_chunk(v, p.scale, p.scale_b, p.swiglu != 0, packed);
                if (p.swiglu) {
                    uint4* dst = reinterpret_cast<uint4*>(out_row + c / 2);
                    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(out_row + c);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tmem_empty);
            tmem_phase ^= 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- two-CTA tiles ------------------------------------------------------------------------------
// The 128 x 256 tile above pulls 54 KB through L2 -> shared memory per 256-deep k block, and that
// path, not the tensor pipe, bounds it. Here two CTAs of a cluster (a pair of SMs) share one
// 256 x 256 tile with tcgen05 cta_group::2: each CTA loads its own 128 token rows (A), its own
// half of the 256 weight rows (B) and the scales of both, 38 KB per k block for the same
// 128 x 256 x 256 of arithmetic per SM. The even CTA of the pair (the leader) issues the MMAs for
// both; each CTA's accumulator half sits in its own tensor memory and is drained by its own
// epilogue warps.
//
// Barriers (same offsets in both CTAs):
//   full[s]   leader's only: one arrival (leader's producer, expecting the bytes of both CTAs);
//             both producers' TMA loads complete on it (cta_group::2 loads, leader's address);
//   empty[s]  one per CTA, arrived by the leader's tcgen05.commit multicast to both CTAs;
//   tmem_full one per CTA, same multicast;   tmem_empty leader's only, one arrival per epilogue
//             warp of either CTA (the peer's through a cluster-scope arrive);
//   scales_landed[s] leader's only: the stage's block-scale atoms of both CTAs have landed (loaded before
//             the operand tiles);   scales_ready[s] leader's only: the copy thread has issued the stage's
//             shared -> tensor memory scale copies.
constexpr uint32_t kPairStages = 5;
// Tensor memory of the pair kernel: 256 accumulator columns, then one set of token-row scale columns per stage
// (16 each) and one set of weight-row scale columns per k-block slot (32 each).
constexpr uint32_t kTmemPairSfA = 256;
constexpr uint32_t kTmemPairSfB = kTmemPairSfA + kPairStages * 16;
static_assert(kTmemPairSfB + kPairStages * 32 <= kTmemCols, "scale columns of all stages fit beside the accumulator");
constexpr uint32_t kPairBytesB = 128 * 128;                                            // this CTA's 128 weight rows
constexpr uint32_t kPairStageBytes = kBytesA + kPairBytesB + kBytesSfA + kBytesSfB;   // 38912
// Epilogue transposition rows: an epilogue warp holds one accumulator row per lane; to store row pieces that are
// contiguous in global memory it parks one 32-column chunk (64 bytes of BF16 per row, rows padded by 16 bytes so
// that the row-per-lane writes spread over all banks) and reads it back with 4 lanes per row.
constexpr uint32_t kPairEpilogueWarps = 8;      // two per tensor-memory lane quadrant
constexpr uint32_t kPairOutRowBytes = 64 + 16;
constexpr uint32_t kPairOutBytes = kPairEpilogueWarps * 32 * kPairOutRowBytes;         // 20480
constexpr uint32_t kPairSmemBytes = kPairStages * kPairStageBytes + kPairOutBytes + 1024 + 256;
constexpr uint32_t kPairCopyWarp = 2 + kPairEpilogueWarps;
constexpr uint32_t kPairThreads = 32 * (kPairCopyWarp + 1);   // TMA warp, MMA warp, epilogue warps, scale-copy warp
constexpr uint32_t kSplitWorthSteps = 16;       // pipeline steps a pair issues in the time a hand-over costs
constexpr uint32_t kSplitWays = 8;              // a leftover tile is cut into this many parts at most
constexpr uint32_t kSplitWaitLimit = 1u << 20;  // polls of a handed-over part's flag (each a round trip to L2) before giving up
constexpr uint64_t kSplitSlotBytes = 2ull * kPairEpilogueWarps * 32 * 128 * 4;   // one pair's accumulator: 256 x 256 f32
constexpr uint32_t kLeaderMask = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address within a pair

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile load whose bytes are counted on the barrier at `bar`'s offset in the pair's leader CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar & kLeaderMask)
        : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3))
                 : "memory");
}
__device__ __forceinline__ void tc_copy_sf_pair(uint32_t tmem, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kLeaderMask) : "memory");
}

// The work of one CTA pair, in the order it is done: the head or middle part of a leftover tile (its partial
// accumulator is handed to the pair that finishes the tile), the part that finishes a leftover tile, then the
// pair's whole tiles. Tiles are numbered m-pair fastest; whole tiles of pair p are p, p + pairs, ...; with `split` the
// tiles past the last full round are cut along k into equal contiguous ranges, one per pair, so that every pair
// issues the same number of k blocks. A range is at most one tile long: it holds the tail of one tile, the head
// of the next, or both. A part handed over is its pair's first item and nothing waits in front of it; a
// finishing part follows, and only its epilogue warps wait (for first items of other pairs, about as long as
// its own), with the accumulator already released; the reads of the handed-over sums then run under the
// MMAs of the whole tiles that follow.
struct PairItem {
    uint32_t tile, kb0, kb1;
    uint32_t kind;           // 0: whole tile, 1: part handed over, 2: part that finishes the tile
    uint32_t first_giver;    // kind 2: the pairs first_giver .. this pair - 1 hand their parts over
};
struct PairWork {
    uint32_t items, whole;
    PairItem given, finishing;
    bool gives, finishes;
    __device__ PairItem item(uint32_t index, uint32_t pair, uint32_t pairs, uint32_t k_blocks) const {
        const uint32_t parts = (gives ? 1u : 0u) + (finishes ? 1u : 0u);
        if (gives && index == 0) return given;
        if (finishes && index + 1 == parts) return finishing;
        return PairItem{pair + (index - parts) * pairs, 0, k_blocks, 0, 0};
    }
};
// `sharers` (0: whole tiles only): the first `sharers` pairs share the leftover tiles (at most kSplitWays per tile).
__device__ __forceinline__ PairWork pair_work(uint32_t pair, uint32_t pairs, uint32_t tiles, uint32_t k_blocks, uint32_t sharers) {
    PairWork w{};
    if (!sharers) {
        w.whole = tiles > pair ? (tiles - pair + pairs - 1) / pairs : 0;
        w.items = w.whole;
        return w;
    }
    w.whole = tiles / pairs;
    w.items = w.whole;
    if (pair >= sharers) return w;
    const uint32_t first_left = w.whole * pairs;
    const uint64_t units = static_cast<uint64_t>(tiles - first_left) * k_blocks;   // k blocks of the leftover tiles
    const uint64_t x0 = pair * units / sharers, x1 = (pair + 1) * units / sharers;  // this pair's range (not empty: units >= sharers)
    const uint32_t a = static_cast<uint32_t>(x0 / k_blocks), b = static_cast<uint32_t>((x1 - 1) / k_blocks);
    const uint64_t a_begin = static_cast<uint64_t>(a) * k_blocks, a_end = a_begin + k_blocks;
    if (x1 >= a_end) {
        // the range holds the tail of tile a: every pair from the one that owns the tile's first k block hands over
        w.finishes = true;
        w.finishing = PairItem{first_left + a, static_cast<uint32_t>(x0 - a_begin), k_blocks, 2,
                               static_cast<uint32_t>(((a_begin + 1) * sharers - 1) / units)};
        if (w.finishing.first_giver == pair) w.finishing.kind = 0;   // the whole tile
    } else {
        w.gives = true;
        w.given = PairItem{first_left + a, static_cast<uint32_t>(x0 - a_begin), static_cast<uint32_t>(x1 - a_begin), 1, 0};
    }
    if (b > a) {
        // and the head of tile b (never all of it: the range is at most one tile long)
        w.gives = true;
        w.given = PairItem{first_left + b, 0, static_cast<uint32_t>(x1 - static_cast<uint64_t>(b) * k_blocks), 1, 0};
    }
    w.items = w.whole + (w.gives ? 1u : 0u) + (w.finishes ? 1u : 0u);
    return w;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_weight,
                 const __grid_constant__ CUtensorMap map_act_sf, const __grid_constant__ CUtensorMap map_weight_sf,
                 const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* out_stage = smem + kPairStages * kPairStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + kPairOutBytes);
    // full[S], empty[S], tmem_full, tmem_empty, scales_ready[S], scales_landed[S]; then the TMEM base and the abort flag
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kPairStages + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();            // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kPairStages);
    const uint32_t bar_tmem_full = smem_u32(bars + 2 * kPairStages), bar_tmem_empty = smem_u32(bars + 2 * kPairStages + 1);
    const uint32_t bar_scales_ready = smem_u32(bars + 2 * kPairStages + 2), bar_scales_landed = smem_u32(bars + 3 * kPairStages + 2);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kPairStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
            mbar_init(bar_scales_ready + 8 * s, 1);
            mbar_init(bar_scales_landed + 8 * s, 1);
        }
        mbar_init(bar_tmem_full, 1);
        mbar_init(bar_tmem_empty, 2 * kPairEpilogueWarps);   // one arrival per epilogue warp of either CTA
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();   // the peer's barriers exist before anything can signal them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // An odd number of 128-row token tiles leaves the second CTA of the last pair without rows of its own: it
    // loads whatever follows (the next term's rows, or the fill value past the tensor) and stores nothing.
    const uint32_t m_pairs = (p.padded_tokens + 2 * kTileM - 1) / (2 * kTileM);
    const uint32_t n_tiles = p.rows / kTileN;
    const uint32_t total_tiles = m_pairs * n_tiles;
    // A last k block that is only partly inside the tensor is loaded like the others (the TMA fills what lies past
    // the edge); the MMA issuer only consumes the k steps inside.
    const uint32_t k_blocks = (p.cols + kBlockK - 1) / kBlockK;
    const uint32_t atoms_per_row_block = p.cols / 64;
    const uint32_t act_term_atoms = p.padded_tokens / 128 * atoms_per_row_block;   // scale atoms of one activation term
    const PairWork work = pair_work(pair, pairs, total_tiles, k_blocks, p.split_sharers);

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        uint32_t stage = 0, phase = 0;
        bool alive = true;
        for (uint32_t index = 0; alive && index < work.items; ++index) {
            const PairItem item = work.item(index, pair, pairs, k_blocks);
            const uint32_t m_pair = item.tile % m_pairs, n_tile = item.tile / m_pairs;
            const uint32_t item_steps = (item.kb1 - item.kb0) * p.terms;
            for (uint32_t step = 0; step < item_steps; ++step) {
                const uint32_t kb = item.kb0 + step / p.terms, term = step % p.terms;
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status_word, kErrProducerWait)) {
                    alive = false;
                    break;
                }
                const uint32_t base = smem_u32(smem + stage * kPairStageBytes);
                const uint32_t full = bar_full + 8 * stage;
                // The block scales go first, on a barrier of their own: they are small and land early, so the copy
                // thread has them in tensor memory by the time the operand tiles arrive.
                const uint32_t landed = bar_scales_landed + 8 * stage;
                const uint32_t token_row = m_pair * 2 * kTileM + rank * kTileM;
                if (rank == 0) mbar_expect_tx(landed, 2 * (kBytesSfA + kBytesSfB));
                tma_load_2d_pair(base + kBytesA + kPairBytesB, &map_act_sf, 0,
                                 term * act_term_atoms + (token_row / 128) * atoms_per_row_block + kb * 4, landed);
                tma_load_2d_pair(base + kBytesA + kPairBytesB + kBytesSfA, &map_weight_sf, 0,
                                 (n_tile * 2) * atoms_per_row_block + kb * 4, landed);
                tma_load_2d_pair(base + kBytesA + kPairBytesB + 2 * kBytesSfA, &map_weight_sf, 0,
                                 (n_tile * 2 + 1) * atoms_per_row_block + kb * 4, landed);
                if (rank == 0) mbar_expect_tx(full, 2 * (kBytesA + kPairBytesB));
                tma_load_2d_pair(base, &map_act, kb * 128, term * p.padded_tokens + token_row, full);
                tma_load_2d_pair(base + kBytesA, &map_weight, kb * 128, n_tile * kTileN + rank * 128, full);
                if (++stage == kPairStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------- MMA issuer (leader only) ----------------
        // Issuing a tcgen05 operation keeps a thread busy for tens of cycles, and one thread issuing the
        // 12 scale copies and the 4 MMAs of every stage could not keep the tensor pipe fed; the copies are
        // issued by a thread of their own (below) into the stage's scale columns, this thread issues
        // only the MMAs. Descriptors advance by additions (their low bits hold address >> 4).
        uint32_t stage = 0, phase = 0, tmem_phase = 0;
        uint32_t kb_slot = 0;   // k blocks counted across tiles, modulo kPairStages: the weight-row scale buffer
        bool alive = true;
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((kTileN >> 3) << 17) | (((2 * kTileM) >> 4) << 24);
        const uint32_t smem_base = smem_u32(smem);
        const uint64_t a_desc0 = operand_desc(smem_base), b_desc0 = operand_desc(smem_base + kBytesA);
        constexpr uint64_t kStageStep = kPairStageBytes >> 4;
        const uint32_t last_k_steps = (p.cols - (k_blocks - 1) * kBlockK) / 64;   // 1..4 k steps of 64 in the last k block
        for (uint32_t index = 0; alive && index < work.items; ++index) {
            const PairItem item = work.item(index, pair, pairs, k_blocks);
            const uint32_t item_steps = (item.kb1 - item.kb0) * p.terms;
            // the epilogues of both CTAs must have drained the previous tile's accumulator
            if (!mbar_wait(bar_tmem_empty, tmem_phase ^ 1, abort_flag, p.status_word, kErrMmaWaitTmem)) break;
            tc_fence_after();
            uint32_t accumulate = 0, term = 0, kb = item.kb0;
            for (uint32_t step = 0; step < item_steps; ++step) {
                // operands in shared memory (TMA) and block scales in tensor memory (copy thread)
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status_word, kErrMmaWaitFull) ||
                    !mbar_wait(bar_scales_ready + 8 * stage, phase, abort_flag, p.status_word, kErrMmaWaitScales)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint64_t a_desc = a_desc0 + stage * kStageStep, b_desc = b_desc0 + stage * kStageStep;
                // the token rows' scales change with every step (term), the weight rows' scales only with the k block
                const uint32_t tmem_sfa = tmem_base + kTmemPairSfA + stage * 16;
                const uint32_t tmem_sfb = tmem_base + kTmemPairSfB + kb_slot * 32;
                // each MMA consumes 64 k = 32 bytes of every row: start address + 2; only k steps inside the tensor
                const uint32_t k_steps = (kb + 1 < k_blocks) ? 4u : last_k_steps;
                if (k_steps == 4) {
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {
                        tc_mma_pair(tmem_base + kTmemAcc, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_sfa + 4 * k, tmem_sfb + 8 * k,
                                    accumulate | k);
                    }
                } else {
                    for (uint32_t k = 0; k < k_steps; ++k) {
                        tc_mma_pair(tmem_base + kTmemAcc, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_sfa + 4 * k, tmem_sfb + 8 * k,
                                    accumulate | k);
                    }
                }
                accumulate = 1;
                tc_commit_pair(bar_empty + 8 * stage);   // frees the stage, and with it the stage's scale columns, in both CTAs
                if (++term == p.terms) {
                    term = 0;
                    ++kb;
                    if (++kb_slot == kPairStages) kb_slot = 0;
                }
                if (++stage == kPairStages) { stage = 0; phase ^= 1; }
            }
            if (alive) tc_commit_pair(bar_tmem_full);     // both accumulator halves complete
            tmem_phase ^= 1;
        }
    } else if (warp == kPairCopyWarp && lane == 0 && rank == 0) {
        // ---------------- scale-copy issuer (leader only): shared memory -> tensor memory, both CTAs ----------------
        uint32_t stage = 0, phase = 0, kb_slot = 0;
        const uint32_t smem_base = smem_u32(smem);
        const uint64_t sfa_desc0 = sf_desc(smem_base + kBytesA + kPairBytesB), sfb_desc0 = sf_desc(smem_base + kBytesA + kPairBytesB + kBytesSfA);
        constexpr uint64_t kStageStep = kPairStageBytes >> 4, kAtomStep = kSfAtomBytes >> 4, kRowBlockStep = kBytesSfA >> 4;
        const uint32_t last_k_steps = (p.cols - (k_blocks - 1) * kBlockK) / 64;
        bool alive = true;
        for (uint32_t index = 0; alive && index < work.items; ++index) {
            const PairItem item = work.item(index, pair, pairs, k_blocks);
            const uint32_t item_steps = (item.kb1 - item.kb0) * p.terms;
            uint32_t term = 0, kb = item.kb0;
            for (uint32_t step = 0; step < item_steps; ++step) {
                // The stage's scale atoms have landed. The producer refilled the stage only after the MMAs of the
                // step that used it last (kPairStages steps ago) were complete, and operations complete in
                // order, so every older MMA is complete too: the stage's token-row scale columns are free, and
                // so are the weight-row scale columns of this k block's slot, last read by the k block
                // kPairStages before it (at least kPairStages steps ago for any number of terms).
                if (!mbar_wait(bar_scales_landed + 8 * stage, phase, abort_flag, p.status_word, kErrCopyWait)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint64_t sfa_desc = sfa_desc0 + stage * kStageStep, sfb_desc = sfb_desc0 + stage * kStageStep;
                // Token-row scales change with every step; weight-row scales are the same for all activation
                // terms of a k block and are copied with term 0 only.
                const uint32_t tmem_sfa = tmem_base + kTmemPairSfA + stage * 16;
                const uint32_t tmem_sfb = tmem_base + kTmemPairSfB + kb_slot * 32;
                const uint32_t k_steps = (kb + 1 < k_blocks) ? 4u : last_k_steps;
                if (k_steps == 4) {
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {
                        tc_copy_sf_pair(tmem_sfa + 4 * k, sfa_desc + k * kAtomStep);
                    }
                    if (term == 0) {
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k) {
                            tc_copy_sf_pair(tmem_sfb + 8 * k, sfb_desc + k * kAtomStep);
                            tc_copy_sf_pair(tmem_sfb + 8 * k + 4, sfb_desc + kRowBlockStep + k * kAtomStep);
                        }
                    }
                } else {
                    for (uint32_t k = 0; k < k_steps; ++k) {
                        tc_copy_sf_pair(tmem_sfa + 4 * k, sfa_desc + k * kAtomStep);
                        if (term == 0) {
                            tc_copy_sf_pair(tmem_sfb + 8 * k, sfb_desc + k * kAtomStep);
                            tc_copy_sf_pair(tmem_sfb + 8 * k + 4, sfb_desc + kRowBlockStep + k * kAtomStep);
                        }
                    }
                }
                // The copies only have to be issued before the MMAs that read them: a copy and a later MMA
                // execute in issue order, and the fences on either side of this arrival order the two threads' issues.
                tc_fence_before();
                mbar_arrive(bar_scales_ready + 8 * stage);
                if (++term == p.terms) {
                    term = 0;
                    ++kb;
                    if (++kb_slot == kPairStages) kb_slot = 0;
                }
                if (++stage == kPairStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp >= 2 && warp < 2 + kPairEpilogueWarps) {
        // ---------------- epilogue (both CTAs): own TMEM half -> BF16 -> global ----------------
        // Two warps per lane quadrant, 128 accumulator columns each. A warp reads its columns into registers
        // in one go and releases the accumulator at once; conversion, staging and the stores to global memory
        // run while the next tile's MMAs are already under way.
        const uint32_t quadrant = warp & 3, half = (warp - 2) >> 2;
        uint32_t tmem_phase = 0;
        // this warp's transposition rows (lane = row): one 32-column chunk at a time
        uint8_t* my_rows = out_stage + (warp - 2) * 32 * kPairOutRowBytes;
        for (uint32_t index = 0; index < work.items; ++index) {
            const PairItem item = work.item(index, pair, pairs, k_blocks);
            const uint32_t m_pair = item.tile % m_pairs, n_tile = item.tile / m_pairs;
            if (!mbar_wait(bar_tmem_full, tmem_phase, abort_flag, p.status_word, kErrEpilogueWait)) break;
            tc_fence_after();
            uint32_t v[4][32];
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) tc_load32(tmem_base + kTmemAcc + ((quadrant * 32) << 16) + half * 128 + c * 32, v[c]);
            tc_wait_ld();
            // the accumulator is free for the next tile's MMAs from here on
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(bar_tmem_empty);
            tmem_phase ^= 1;

            if (item.kind == 1) {
                // a part of a leftover tile: the sums go, as they are, to the pair that finishes the tile
                const uint32_t slot = (pair * 2 + rank) * kPairEpilogueWarps + (warp - 2);
                float4* dst = reinterpret_cast<float4*>(p.split_slots) + static_cast<uint64_t>(slot) * (32 * 32) + lane;
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) {
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        dst[(c * 8 + i) * 32] = make_float4(__uint_as_float(v[c][4 * i]), __uint_as_float(v[c][4 * i + 1]),
                                                            __uint_as_float(v[c][4 * i + 2]), __uint_as_float(v[c][4 * i + 3]));
                    }
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicExch(p.split_flags + slot, 1u);
                continue;
            }
            if (item.kind == 2) {
                // the part that finishes a leftover tile: add the parts handed over, in pair order
                bool arrived = true;
                for (uint32_t giver = item.first_giver; giver < pair; ++giver) {
                    const uint32_t slot = (giver * 2 + rank) * kPairEpilogueWarps + (warp - 2);
                    if (lane == 0) {
                        uint32_t spin = 0;
                        while (atomicAdd(p.split_flags + slot, 0u) == 0u) {
                            if (++spin > kSplitWaitLimit || ((spin & 255u) == 255u && *abort_flag)) { arrived = false; break; }
                        }
                    }
                    arrived = __shfl_sync(0xffffffffu, arrived, 0);
                    if (!arrived) break;
                    __threadfence();
                    const float4* src = reinterpret_cast<const float4*>(p.split_slots) + static_cast<uint64_t>(slot) * (32 * 32) + lane;
#pragma unroll
                    for (uint32_t c = 0; c < 4; ++c) {
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) {
                            const float4 part = __ldcg(src + (c * 8 + i) * 32);
                            v[c][4 * i] = __float_as_uint(__uint_as_float(v[c][4 * i]) + part.x);
                            v[c][4 * i + 1] = __float_as_uint(__uint_as_float(v[c][4 * i + 1]) + part.y);
                            v[c][4 * i + 2] = __float_as_uint(__uint_as_float(v[c][4 * i + 2]) + part.z);
                            v[c][4 * i + 3] = __float_as_uint(__uint_as_float(v[c][4 * i + 3]) + part.w);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) p.split_flags[slot] = 0;   // the flags read zero again when the launch is over
                }
                if (!arrived) {
                    if (lane == 0) {
                        *abort_flag = 1;
                        atomicCAS(p.status_word, 0u, kErrSplitWait);
                        // The launch has failed and says so; the flags of the parts it gave up on go back to zero all
                        // the same, so that a late giver cannot leave one set for the next launch on this plan.
                        for (uint32_t giver = item.first_giver; giver < pair; ++giver) {
                            p.split_flags[(giver * 2 + rank) * kPairEpilogueWarps + (warp - 2)] = 0;
                        }
                    }
                    break;
                }
            }

            const uint32_t first_token = m_pair * 2 * kTileM + rank * kTileM + quadrant * 32;
            if (p.swiglu) {
                // 32 accumulator columns = gate and up sums of 16 intermediate columns = one quantisation group per row
                const uint32_t out_width = p.rows / 2;
                const uint64_t code_bytes = tcgen05_codes_bytes(p.padded_tokens, out_width);
                const uint64_t scale_bytes = tcgen05_scale_bytes(p.padded_tokens, out_width);
                const uint32_t token = first_token + lane;
                uint32_t scale_words[3] = {0, 0, 0};   // the scale bytes of this row's 4 groups, per term: one word of an atom
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) {
                    uint32_t packed[16];
                    convert_chunk(v[c], p.scale, p.scale_b, true, packed);
                    if (p.quant_out) {
                        // The BF16 values this lane holds, quantised for the next GEMM while the next tile's MMAs run.
                        const uint32_t group = n_tile * (kTileN / 32) + half * 4 + c;
                        float2 residual[8];
#pragma unroll
                        for (uint32_t i = 0; i < 8; ++i) {
                            residual[i] = make_float2(__uint_as_float(packed[i] << 16), __uint_as_float(packed[i] & 0xffff0000u));
                        }
#pragma unroll
                        for (uint32_t term = 0; term < 3; ++term) {
                            if (term >= p.quant_terms) break;
                            uint32_t codes[2], scale_code;
                            quantise_term(residual, p.quant_global_scale, term + 1 < p.quant_terms, codes, &scale_code);
                            scale_words[term] |= scale_code << (8 * c);
                            if (token < p.tokens) {
                                *reinterpret_cast<uint2*>(p.quant_out + term * code_bytes + static_cast<uint64_t>(token) * (out_width / 2) + group * 8) =
                                    make_uint2(codes[0], codes[1]);
                            }
                        }
                    }
                    if (p.out) {
                        // transpose through shared memory: 32 bytes of every row, written out as 2 lanes per row
                        uint4* dst = reinterpret_cast<uint4*>(my_rows + lane * kPairOutRowBytes);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        __syncwarp();
                        uint8_t* out_base = reinterpret_cast<uint8_t*>(p.out + static_cast<uint64_t>(first_token) * out_width +
                                                                       n_tile * (kTileN / 2) + half * 64 + c * 16);
#pragma unroll
                        for (uint32_t r16 = 0; r16 < 32; r16 += 16) {
                            const uint32_t r = r16 + (lane >> 1), piece = lane & 1;
                            if (first_token + r >= p.tokens) continue;   // padding rows of the last tile are computed, never stored
                            const uint4 value = *reinterpret_cast<const uint4*>(my_rows + r * kPairOutRowBytes + piece * 16);
                            *reinterpret_cast<uint4*>(out_base + static_cast<uint64_t>(r) * out_width * 2 + piece * 16) = value;
                        }
                        __syncwarp();   // the rows are rewritten for the next chunk
                    }
                }
                if (p.quant_out && token < p.tokens) {
#pragma unroll
                    for (uint32_t term = 0; term < 3; ++term) {
                        if (term >= p.quant_terms) break;
                        *reinterpret_cast<uint32_t*>(p.quant_out + p.quant_terms * code_bytes + term * scale_bytes +
                                                     tcgen05_scale_offset(token, n_tile * (kTileN / 32) + half * 4, out_width)) = scale_words[term];
                    }
                }
            } else {
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) {
                    uint32_t packed[16];
                    convert_chunk(v[c], p.scale, p.scale_b, false, packed);
                    // transpose through shared memory: 64 bytes of every row, written out as 4 lanes per row
                    uint4* dst = reinterpret_cast<uint4*>(my_rows + lane * kPairOutRowBytes);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                    }
                    __syncwarp();
                    uint8_t* out_base = reinterpret_cast<uint8_t*>(p.out + static_cast<uint64_t>(first_token) * p.rows + n_tile * kTileN +
                                                                   half * 128 + c * 32);
#pragma unroll
                    for (uint32_t r8 = 0; r8 < 32; r8 += 8) {
                        const uint32_t r = r8 + (lane >> 2), piece = lane & 3;
                        if (first_token + r >= p.tokens) continue;   // padding rows of the last tile are computed, never stored
                        const uint4 value = *reinterpret_cast<const uint4*>(my_rows + r * kPairOutRowBytes + piece * 16);
                        *reinterpret_cast<uint4*>(out_base + static_cast<uint64_t>(r) * p.rows * 2 + piece * 16) = value;
                    }
                    __syncwarp();   // the rows are rewritten for the next chunk
                }
            }
        }
    }

    // Neither CTA may release tensor memory while the other can still be written by an MMA or read
    // by an epilogue: every thread of the pair meets here (all waits above are bounded).
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- activation quantiser kernel ---------------------------------------------------------------
// One thread per (token, 16-element group). Destination: the code planes of all terms
// stacked ([terms][tokens][cols/2], one TMA tensor of terms*tokens rows), then the scale
// regions of all terms.
__global__ void act_quant_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ destination, uint32_t tokens,
                                 uint32_t cols, uint32_t terms, float global_scale) {
    const uint32_t groups = cols / 16;
    // tokens * cols fits 32 bits, so the group index does too
    const uint32_t index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= tokens * groups) return;
    const uint32_t token = index / groups, group = index - token * groups;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<uint64_t>(token) * cols + group * 16);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    float2 residual[8];   // pairs of neighbouring elements, as the two-wide F32 instructions take them
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        residual[i] = make_float2(__uint_as_float(words[i] << 16), __uint_as_float(words[i] & 0xffff0000u));
    }
    // every term's code plane has whole 128-row tiles (the rows past `tokens` are never written and
    // only ever feed output rows that are not stored)
    const uint64_t code_bytes = tcgen05_codes_bytes(padded_tokens(tokens), cols), scale_bytes = tcgen05_scale_bytes(tokens, cols);
    for (uint32_t term = 0; term < terms; ++term) {
        uint32_t packed[2], scale_code;
        quantise_term(residual, global_scale, term + 1 < terms, packed, &scale_code);
        *reinterpret_cast<uint2*>(destination + term * code_bytes + static_cast<uint64_t>(token) * (cols / 2) + group * 8) =
            make_uint2(packed[0], packed[1]);
        // The scales of four consecutive groups of a token are four consecutive bytes of an atom: lanes are
        // consecutive groups (cols / 16 is a multiple of 4, so a quad of lanes never straddles a token or the
        // end of the grid), and the first lane of every quad stores the four as one word.
        const uint32_t active = __activemask();
        uint32_t quad = scale_code;
        quad |= __shfl_down_sync(active, scale_code, 1) << 8;
        quad |= __shfl_down_sync(active, scale_code, 2) << 16;
        quad |= __shfl_down_sync(active, scale_code, 3) << 24;
        if ((group & 3u) == 0) {
            *reinterpret_cast<uint32_t*>(destination + terms * code_bytes + term * scale_bytes + tcgen05_scale_offset(token, group, cols)) = quad;
        }
    }
}

// ---- tensor maps --------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_entry() {
    static EncodeTiled cached = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            fn = nullptr;
        }
        return reinterpret_cast<EncodeTiled>(fn);
    }();
    return cached;
}

// Packed codes as a 2-D byte tensor [rows][cols/2]; boxes of 128 rows x 128 bytes, 128-byte swizzle.
// A host-side computation: no allocation and no device access.
bool make_code_map(CUtensorMap* map, uint64_t address, uint64_t rows, uint32_t cols) {
    const EncodeTiled encode = encode_entry();
    if (!encode) return false;
    const cuuint64_t dims[2] = {cols / 2, rows};
    const cuuint64_t strides[1] = {cols / 2};
    const cuuint32_t box[2] = {128, 128};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void*>(address), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Block-scale atoms as a 2-D tensor [atoms][256 x u16] (512 bytes each); a box is the 4 atoms of
// one 128-row block and one 256-deep k block.
bool make_scale_map(CUtensorMap* map, uint64_t address, uint64_t atoms) {
    const EncodeTiled encode = encode_entry();
    if (!encode) return false;
    const cuuint64_t dims[2] = {256, atoms};
    const cuuint64_t strides[1] = {kSfAtomBytes};
    const cuuint32_t box[2] = {256, 4};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, reinterpret_cast<void*>(address), dims, strides, box,
                  element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---- validation ------------------------------------------------------------------------------------
bool act_shape_ok(uint32_t tokens, uint32_t cols, uint32_t terms) {
    return tokens && cols && tokens <= (1u << 24) && cols % 64 == 0 && terms >= 1 && terms <= 3 &&
           static_cast<uint64_t>(padded_tokens(tokens)) * cols <= UINT32_MAX;
}

bool check_act_quant(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_act_quant_args_v1* a, bool full,
                     augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!act_shape_ok(a->tokens, a->cols, a->terms) || !std::isfinite(a->global_scale) || a->global_scale <= 0.0f) {
        return false;
    }
    if (a->input_len_bytes != static_cast<uint64_t>(a->tokens) * a->cols * 2 ||
        a->destination_len_bytes != a->terms * staged_term_bytes(a->tokens, a->cols)) {
        return false;
    }
    const Range r[2] = {{a->input_bf16, a->input_len_bytes, 16}, {a->destination, a->destination_len_bytes, 256}};
    if (!all_disjoint(r, 2)) return false;
    return !full || inspect_device_ranges(d, r, 2, failure);
}

// What `output_bf16` of a GEMM descriptor is: [tokens][rows], [tokens][rows / 2] (fused SwiGLU), or absent.
enum class GemmOutput { kFull, kHalfWidth, kNone };

bool check_gemm(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                const augur_cuda_nvfp4_sm100_gemm_args_v1* a, bool full, augur_cuda_result_v1* failure,
                GemmOutput output = GemmOutput::kFull) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!plan_ok(plan, d, s) || !act_shape_ok(a->tokens, a->cols, a->activation_terms)) return false;
    if (!a->rows || a->rows % 128 != 0 || static_cast<uint64_t>(a->rows) * a->cols > UINT32_MAX) return false;
    if (!scale_ok(a->weight_global_scale) || !std::isfinite(a->activation_global_scale) ||
        a->activation_global_scale <= 0.0f) {
        return false;
    }
    if (a->weight_len_bytes != tcgen05_extent_bytes(a->rows, a->cols) ||
        a->activation_len_bytes != a->activation_terms * staged_term_bytes(a->tokens, a->cols)) {
        return false;
    }
    Range r[4] = {{a->weight, a->weight_len_bytes, 256}, {a->activation, a->activation_len_bytes, 256}, plan_scratch_range(plan), {}};
    size_t count = 3;
    if (output != GemmOutput::kNone) {
        const uint64_t width = output == GemmOutput::kHalfWidth ? a->rows / 2 : a->rows;
        if (a->output_len_bytes != static_cast<uint64_t>(a->tokens) * width * 2) return false;
        r[count++] = {a->output_bf16, a->output_len_bytes, 16};
    } else if (a->output_bf16 || a->output_len_bytes) {
        return false;
    }
    if (!all_disjoint(r, count)) return false;
    if (!full) return true;
    // the plan's scratch was inspected when the plan was made
    if (!inspect_device_ranges(d, r, 2, failure)) return false;
    return output == GemmOutput::kNone || inspect_device_ranges(d, r + 3, 1, failure);
}

}  // namespace

// How many two-CTA clusters of the pair kernel fit the current device at once. The leftover-tile split lets
// a pair wait for parts that lower-numbered pairs produce, so every pair of the grid has to be resident:
// the grid is capped with this number (it can be below SMs / 2 when cluster placement leaves SMs unused).
uint32_t gemm_pair_resident_clusters() {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(2);
    config.blockDim = dim3(kPairThreads);
    config.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel, &config) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        return 0;
    }
    return static_cast<uint32_t>(clusters);
}

cudaError_t gemm_configure_device() {
    const cudaError_t e = cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
}

}  // namespace augur_sm100

using namespace augur_sm100;

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_plan_scratch_extent_host_v1(
    uint32_t sm_count, uint64_t* out_bytes) {
    if (!out_bytes || !sm_count || sm_count > 4096) return invalid();
    *out_bytes = kCounterBytes + static_cast<uint64_t>(sm_count / 2) * kSplitSlotBytes;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_scratch_extent_host_v1(
    uint32_t rows, uint32_t cols, uint32_t tokens, uint32_t activation_terms, uint64_t* out_bytes) {
    if (!out_bytes || !rows || rows % 128 != 0 || !act_shape_ok(tokens, cols, activation_terms)) return invalid();
    // The GEMM itself needs no scratch; a caller that lets the plan stage the quantised
    // activations needs this much.
    *out_bytes = activation_terms * staged_term_bytes(tokens, cols);
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_act_quant_preflight_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_act_quant_args_v1* a) {
    augur_cuda_result_v1 failure;
    return check_act_quant(d, s, a, true, &failure) ? ok() : failure;
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_act_quant_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_act_quant(d, s, a, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    const uint64_t groups = static_cast<uint64_t>(a->tokens) * (a->cols / 16);
    // Rows past `tokens` in the last 128-row tile (codes and scale bytes) are left as they are: they only
    // feed output rows that the GEMM never stores.
    act_quant_kernel<<<static_cast<uint32_t>((groups + 255) / 256), 256, 0, s->stream>>>(
        reinterpret_cast<const uint16_t*>(a->input_bf16), reinterpret_cast<uint8_t*>(a->destination), a->tokens,
        a->cols, a->terms, a->global_scale);
    count_launch();
    return submitted();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_gemm(d, s, plan, a, true, &failure)) return failure;
    CUtensorMap probe;
    return make_code_map(&probe, a->weight, a->rows, a->cols) ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

namespace {
// Enqueues the GEMM of a validated descriptor. `swiglu`: a->rows counts the physical weight rows
// (gate and up interleaved), the output is a->rows / 2 wide.
struct QuantTarget {
    uint64_t destination = 0;
    uint32_t terms = 0;
    float global_scale = 0.0f;
};

augur_cuda_result_v1 launch_gemm(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                                 const augur_cuda_nvfp4_sm100_gemm_args_v1* a, bool swiglu, float up_global_scale,
                                 QuantTarget quant = QuantTarget()) {
    // Tensor maps are encoded on the host into kernel parameter space: no allocation, no driver query.
    // The activation map spans the stacked code planes of all terms (terms * padded tokens rows).
    CUtensorMap map_act, map_weight;
    if (!make_code_map(&map_weight, a->weight, a->rows, a->cols) ||
        !make_code_map(&map_act, a->activation, static_cast<uint64_t>(a->activation_terms) * padded_tokens(a->tokens), a->cols)) {
        return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
    }
    GemmParams p{};
    p.weight_sf = reinterpret_cast<const uint8_t*>(a->weight) + tcgen05_codes_bytes(a->rows, a->cols);
    const uint32_t padded = padded_tokens(a->tokens);
    p.act_sf = reinterpret_cast<const uint8_t*>(a->activation) + a->activation_terms * tcgen05_codes_bytes(padded, a->cols);
    p.act_term_stride = tcgen05_scale_bytes(a->tokens, a->cols);
    p.out = reinterpret_cast<__nv_bfloat16*>(a->output_bf16);
    p.status_word = plan->status_word;
    p.rows = a->rows; p.cols = a->cols; p.tokens = a->tokens; p.terms = a->activation_terms;
    p.padded_tokens = padded;
    p.scale = a->weight_global_scale * a->activation_global_scale;
    p.scale_b = up_global_scale * a->activation_global_scale;
    p.swiglu = swiglu ? 1u : 0u;
    p.quant_out = reinterpret_cast<uint8_t*>(quant.destination);
    p.quant_terms = quant.terms;
    p.quant_global_scale = quant.global_scale;
    if (a->rows % kTileN == 0 && plan->sm_count >= 2) {
        // 256 x 256 tiles on pairs of CTAs (clusters of two); the grid is a whole number of pairs.
        CUtensorMap map_act_sf, map_weight_sf;
        const uint64_t atoms_per_row_block = a->cols / 64;
        if (!make_scale_map(&map_weight_sf, reinterpret_cast<uint64_t>(p.weight_sf), (a->rows / 128) * atoms_per_row_block) ||
            !make_scale_map(&map_act_sf, reinterpret_cast<uint64_t>(p.act_sf),
                            static_cast<uint64_t>(a->activation_terms) * (padded / 128) * atoms_per_row_block)) {
            return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
        }
        const uint32_t tiles = ((padded + 2 * kTileM - 1) / (2 * kTileM)) * (a->rows / kTileN);
        const uint32_t all_pairs = plan->pair_clusters;   // pairs that are resident together (at most SMs / 2)
        uint32_t pairs = tiles < all_pairs ? tiles : all_pairs;
        // Tiles past the last full round of the pairs (all tiles, when there are fewer tiles than pairs) are cut
        // along k between all pairs when the plan's scratch has room for the partial accumulators handed over
        // (one slot per pair behind the counter regions, whose first words serve as the flags) and those tiles
        // hold at least one k block per pair.
        const uint32_t k_blocks = (a->cols + kBlockK - 1) / kBlockK;
        const uint32_t left = tiles % all_pairs;
        uint32_t sharers = left * kSplitWays < all_pairs ? left * kSplitWays : all_pairs;   // a tile is cut in kSplitWays parts at most
        if (sharers > static_cast<uint64_t>(left) * k_blocks) sharers = left * k_blocks;      // and every part holds a k block
        // Handing parts over costs about as much as 16 pipeline steps (k block x term) of a pair: the cut is made
        // when the pairs would otherwise idle for longer than that, on average, in the last round.
        const uint64_t idle_steps = static_cast<uint64_t>(all_pairs - left) * k_blocks * a->activation_terms;
        if (left != 0 && sharers > left && idle_steps >= static_cast<uint64_t>(kSplitWorthSteps) * all_pairs &&
            plan->scratch_bytes >= kCounterBytes + sharers * kSplitSlotBytes) {
            if (pairs < sharers) pairs = sharers;
            p.split_sharers = sharers;
            p.split_flags = reinterpret_cast<uint32_t*>(plan->scratch);
            p.split_slots = reinterpret_cast<float*>(plan->scratch + kCounterBytes);
        }
        gemm_pair_kernel<<<2 * pairs, kPairThreads, kPairSmemBytes, s->stream>>>(map_act, map_weight, map_act_sf, map_weight_sf, p);
        count_launch();
        return submitted();
    }
    const uint32_t m_tiles = padded / kTileM, n_tiles = (a->rows + kTileN - 1) / kTileN;
    uint32_t grid = m_tiles * n_tiles;
    if (grid > plan->sm_count) grid = plan->sm_count;
    gemm_kernel<<<grid, kGemmThreads, kGemmSmemBytes, s->stream>>>(map_act, map_weight, p);
    count_launch();
    return submitted();
}

static_assert(sizeof(augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1) == 88, "gemm_swiglu ABI");

// The fused form as a plain GEMM descriptor over the physical (interleaved) weight rows; false if the
// descriptor's own fields are bad. Output extent is checked here (it is half as wide).
bool swiglu_as_gemm(const augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1* a, augur_cuda_nvfp4_sm100_gemm_args_v1* g) {
    if (a->reserved || !a->rows || a->rows % 64 != 0 || a->rows > (1u << 30) || !scale_ok(a->up_global_scale)) return false;
    if (a->output_len_bytes != static_cast<uint64_t>(a->tokens) * a->rows * 2) return false;
    *g = augur_cuda_nvfp4_sm100_gemm_args_v1{};
    g->abi_version = a->abi_version;
    g->struct_size = sizeof(*g);
    g->weight = a->weight; g->weight_len_bytes = a->weight_len_bytes;
    g->activation = a->activation; g->activation_len_bytes = a->activation_len_bytes;
    g->output_bf16 = a->output_bf16;
    g->rows = 2 * a->rows; g->cols = a->cols; g->tokens = a->tokens; g->activation_terms = a->activation_terms;
    g->output_len_bytes = static_cast<uint64_t>(a->tokens) * g->rows * 2;   // what check_gemm expects for 2*rows columns
    g->weight_global_scale = a->gate_global_scale; g->activation_global_scale = a->activation_global_scale;
    return true;
}
}  // namespace

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_gemm(d, s, plan, a, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    return launch_gemm(s, plan, a, false, 0.0f);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1* a) {
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            return make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return invalid();
    }
    augur_cuda_nvfp4_sm100_gemm_args_v1 g;
    if (!swiglu_as_gemm(a, &g)) return invalid();
    augur_cuda_result_v1 failure;
    // the output range handed to the range checks is the real (half-width) one
    g.output_len_bytes = a->output_len_bytes;
    if (!check_gemm(d, s, plan, &g, true, &failure, GemmOutput::kHalfWidth)) return failure;
    CUtensorMap probe;
    return make_code_map(&probe, g.weight, g.rows, g.cols) ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1* a) {
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            return make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return invalid();
    }
    augur_cuda_nvfp4_sm100_gemm_args_v1 g;
    if (!swiglu_as_gemm(a, &g)) return invalid();
    augur_cuda_result_v1 failure;
    g.output_len_bytes = a->output_len_bytes;
    if (!check_gemm(d, s, plan, &g, false, &failure, GemmOutput::kHalfWidth)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    return launch_gemm(s, plan, &g, true, a->up_global_scale);
}

namespace {
static_assert(sizeof(augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1) == 112, "gemm_swiglu_quant ABI");

// Pair tiles only: padded tokens a multiple of 256 and an intermediate size that is a multiple of 128.
bool check_swiglu_quant(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                        const augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1* a, bool full,
                        augur_cuda_nvfp4_sm100_gemm_args_v1* g, augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (a->reserved || !a->rows || a->rows % 128 != 0 || a->rows > (1u << 30) || !scale_ok(a->up_global_scale) ||
        a->destination_terms < 1 || a->destination_terms > 3 || !std::isfinite(a->destination_global_scale) ||
        a->destination_global_scale <= 0.0f || !a->tokens || !plan ||
        plan->sm_count < 2) {
        return false;
    }
    const bool writes_bf16 = a->output_bf16 != 0;
    if (!act_shape_ok(a->tokens, a->rows, a->destination_terms) ||
        a->destination_len_bytes != a->destination_terms * staged_term_bytes(a->tokens, a->rows)) {
        return false;
    }
    // the members it shares with the plain GEMM, over the physical (interleaved) weight rows
    *g = augur_cuda_nvfp4_sm100_gemm_args_v1{};
    g->abi_version = a->abi_version;
    g->struct_size = sizeof(*g);
    g->weight = a->weight; g->weight_len_bytes = a->weight_len_bytes;
    g->activation = a->activation; g->activation_len_bytes = a->activation_len_bytes;
    g->output_bf16 = a->output_bf16; g->output_len_bytes = a->output_len_bytes;
    g->rows = 2 * a->rows; g->cols = a->cols; g->tokens = a->tokens; g->activation_terms = a->activation_terms;
    g->weight_global_scale = a->gate_global_scale; g->activation_global_scale = a->activation_global_scale;
    if (!check_gemm(d, s, plan, g, full, failure, writes_bf16 ? GemmOutput::kHalfWidth : GemmOutput::kNone)) return false;
    *failure = invalid();
    // the staged destination against every other range
    const Range destination = {a->destination, a->destination_len_bytes, 256};
    const Range others[4] = {{a->weight, a->weight_len_bytes, 256}, {a->activation, a->activation_len_bytes, 256},
                             plan_scratch_range(plan), {a->output_bf16, a->output_len_bytes, 16}};
    for (size_t i = 0; i < (writes_bf16 ? 4u : 3u); ++i) {
        if (!disjoint(destination, others[i])) return false;
    }
    return !full || inspect_device_ranges(d, &destination, 1, failure);
}
}  // namespace

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_quant_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1* a) {
    augur_cuda_nvfp4_sm100_gemm_args_v1 g;
    augur_cuda_result_v1 failure;
    if (!check_swiglu_quant(d, s, plan, a, true, &g, &failure)) return failure;
    CUtensorMap probe;
    return make_code_map(&probe, g.weight, g.rows, g.cols) ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_quant_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1* a) {
    augur_cuda_nvfp4_sm100_gemm_args_v1 g;
    augur_cuda_result_v1 failure;
    if (!check_swiglu_quant(d, s, plan, a, false, &g, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    QuantTarget quant;
    quant.destination = a->destination;
    quant.terms = a->destination_terms;
    quant.global_scale = a->destination_global_scale;
    return launch_gemm(s, plan, &g, true, a->up_global_scale, quant);
}
