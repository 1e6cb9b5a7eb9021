// Small-token (1..8) NVFP4 linear for sm_100a on the tensor-memory path: the weights go from HBM to the
// tensor cores without a single per-element instruction on the SMs.
//
//   weights      TCGEN05 layout (codes K-major as in the checkpoint, block scales in 512-byte atoms), the
//                128-row operand of tcgen05.mma kind::mxf4nvf4: TMA brings 128 rows x 256 k (16 KB of codes
//                plus 2 KB of scales) per stage into a ring in shared memory, tcgen05.cp moves the scales on
//                to tensor memory, the MMA reads the codes where the TMA put them;
//   activations  BF16 in global memory. A block-scaled FP4 MMA wants FP4 on both sides, so every CTA splits
//                the activations of its own k-slab, once, into kTerms NVFP4 residual terms (term t holds
//                the part of x that terms 0..t-1 left over) with power-of-two per-token global scales; the
//                terms sit side by side on the MMA n dimension (column = term * 8 + token), resident in
//                shared memory and their block scales resident in tensor memory for the whole launch. Six
//                terms reproduce a BF16 value to about 3e-7 of its group's largest magnitude, below the f32
//                accumulation noise; one MMA per 64 k covers all tokens and all terms;
//   accumulator  128 weight rows x 48 columns of f32 in tensor memory, two buffers; the epilogue warps add
//                the terms of a token with their scales and either finish the rows or, when the k dimension
//                is cut into slabs, hand a partial sum over through plan scratch.
//
// Work split: the k dimension is cut into `slabs` (a slab's activations must fit shared memory), every CTA
// belongs to one slab and owns a contiguous range of 128-row tiles. A row tile is complete when all slabs
// have delivered: partial sums go to plan scratch with an arrival counter per 32 rows, the last arriver adds
// them in slab order and finishes the rows. Nothing spins on another CTA; results are bit-reproducible.
// The kernel is bandwidth-bound: a CTA with fewer tiles ends early and the others take up its share of HBM.
//
// Every mbarrier wait is bounded; a wait that runs out records a code in the plan's status word, raises a
// CTA-wide abort flag, and all roles fall through to the common exit where tensor memory is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "nvfp4_internal.h"
#include "nvfp4_layout.cuh"
#include "nvfp4_tc.cuh"

namespace augur_sm100 {
namespace {
using namespace tc;

constexpr uint32_t kTerms = 6;                         // residual terms of the activation split
constexpr uint32_t kCols = 8 * kTerms;                 // MMA n: column = term * 8 + token
constexpr uint32_t kStageK = 256;                      // k per ring stage = one 128-byte swizzled row of codes
constexpr uint32_t kStageCodeBytes = kTileM * 128;     // 16 KB
constexpr uint32_t kStageSfBytes = 4 * kSfAtomBytes;   // 2 KB: the 4 scale atoms of the stage
constexpr uint32_t kStageBytes = kStageCodeBytes + kStageSfBytes;
constexpr uint32_t kStages = 8;
constexpr uint32_t kMaxSlabStages = 8;                 // k-slab of a CTA: at most 2048 k
constexpr uint32_t kChunkBytes = kCols * 128;          // activation codes of one 256-k chunk: 48 rows x 128 bytes
constexpr uint32_t kActCodeBytes = kMaxSlabStages * kChunkBytes;
constexpr uint32_t kActSfBytes = kMaxSlabStages * 4 * kSfAtomBytes;
constexpr uint32_t kThreads = 320;                     // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue, all ten quantise
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kActCodeBytes + kActSfBytes + 1024 /*alignment*/ + 1024 /*small state*/;
constexpr uint32_t kTmemAcc = 0;                       // two accumulators of 64 columns (48 used)
constexpr uint32_t kTmemSfAct = 128;                   // 4 columns per 64 k of the slab: 128 columns
constexpr uint32_t kTmemSfWeight = 256;                // 16 columns per ring stage
constexpr uint32_t kTmemColumns = 512;
static_assert(kTmemSfWeight + kStages * 16 <= kTmemColumns, "tensor memory columns");
constexpr uint32_t kSlotFloats = 256;                  // one partial: 32 rows x 8 tokens

constexpr uint32_t kErrTcProducer = 0x301, kErrTcFull = 0x302, kErrTcAccEmpty = 0x303, kErrTcAccFull = 0x304;

struct TcParams {
    const uint8_t* weight_sf;     // scale region of the weight
    const uint16_t* x;            // [tokens][cols] BF16
    void* out;
    float* partials;              // [tile * 4 + quadrant][slab][32 rows][8 tokens]
    uint32_t* counters;           // [tile * 4 + quadrant], zero between launches
    uint32_t* status_word;
    uint32_t rows;                // physical weight rows (SwiGLU: gate and up interleaved by 16)
    uint32_t out_rows;            // output width
    uint32_t cols, tokens, epilogue;
    uint32_t tiles, k_blocks, slabs;
    float global_a, global_b;
};

__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// Finished sums of 32 weight rows (lane = row) for the 8 tokens: scale, activation, rounding, store.
__device__ __forceinline__ void finish_rows(const TcParams& p, uint32_t tile, uint32_t quadrant, uint32_t lane, const float (&y)[8]) {
    if (p.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
        // 32 physical rows = 16 gate rows (lanes 0..15) and the matching 16 up rows (lanes 16..31)
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
        const uint32_t index = (tile * kTileM + quadrant * 32) / 2 + (lane & 15);
#pragma unroll
        for (uint32_t token = 0; token < 8; ++token) {
            const float up = __shfl_sync(0xffffffffu, y[token], (lane & 15) + 16) * p.global_b;
            const float gate = y[token] * p.global_a;
            if (lane < 16 && token < p.tokens) {
                out[static_cast<uint64_t>(token) * p.out_rows + index] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
            }
        }
        return;
    }
    const uint32_t row = tile * kTileM + quadrant * 32 + lane;
#pragma unroll
    for (uint32_t token = 0; token < 8; ++token) {
        if (token < p.tokens) {
            const float value = y[token] * p.global_a;
            if (p.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) {
                static_cast<float*>(p.out)[static_cast<uint64_t>(token) * p.out_rows + row] = value;
            } else {
                static_cast<__nv_bfloat16*>(p.out)[static_cast<uint64_t>(token) * p.out_rows + row] = __float2bfloat16_rn(value);
            }
        }
    }
}

// This CTA's share of 32 rows of `tile`: finished here if there is one slab, else handed over; the last of
// the `slabs` arrivals adds all shares in slab order. Whole warps call this.
__device__ __forceinline__ void contribute_rows(const TcParams& p, uint32_t tile, uint32_t quadrant, uint32_t slab, uint32_t lane,
                                                const float (&y)[8]) {
    if (p.slabs == 1) {
        finish_rows(p, tile, quadrant, lane, y);
        return;
    }
    const uint32_t group = tile * 4 + quadrant;
    float* slots = p.partials + static_cast<uint64_t>(group) * p.slabs * kSlotFloats;
    float4* mine = reinterpret_cast<float4*>(slots + static_cast<uint64_t>(slab) * kSlotFloats) + lane * 2;
    mine[0] = make_float4(y[0], y[1], y[2], y[3]);
    mine[1] = make_float4(y[4], y[5], y[6], y[7]);
    __threadfence();
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(&p.counters[group], 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived + 1 != p.slabs) return;
    __threadfence();
    float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t s0 = 0; s0 < p.slabs; s0 += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            a[j] = b[j] = make_float4(0, 0, 0, 0);
            if (s0 + j < p.slabs) {
                const float4* slot = reinterpret_cast<const float4*>(slots + static_cast<uint64_t>(s0 + j) * kSlotFloats) + lane * 2;
                a[j] = __ldcg(slot);
                b[j] = __ldcg(slot + 1);
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            if (s0 + j < p.slabs) {
                sum[0] += a[j].x; sum[1] += a[j].y; sum[2] += a[j].z; sum[3] += a[j].w;
                sum[4] += b[j].x; sum[5] += b[j].y; sum[6] += b[j].z; sum[7] += b[j].w;
            }
        }
    }
    finish_rows(p, tile, quadrant, lane, sum);
    if (lane == 0) p.counters[group] = 0;   // clean for the next launch
}

__global__ void __launch_bounds__(kThreads, 1)
gemv_tc_kernel(const __grid_constant__ CUtensorMap map_weight, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* act_codes = smem + kStages * kStageBytes;            // [chunk][48 rows][128 bytes], 128-byte swizzle
    uint8_t* act_sf = act_codes + kActCodeBytes;                   // [64-k step] x 512-byte atoms
    float* term_scale = reinterpret_cast<float*>(act_sf + kActSfBytes);   // [token]: scale of term 0 (a power of two)
    uint32_t* row_max = reinterpret_cast<uint32_t*>(term_scale + 8);      // [token]: bits of the largest magnitude; [8..16): a NaN or infinity seen
    uint64_t* bars = reinterpret_cast<uint64_t*>(row_max + 16);           // full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * kStages), bar_acc_empty = smem_u32(bars + 2 * kStages + 2);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 16) row_max[threadIdx.x] = 0;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // ---- this CTA's slab and tiles ----
    const uint32_t base = gridDim.x / p.slabs, extra = gridDim.x % p.slabs;   // the first `extra` slabs have one CTA more
    uint32_t slab, place, sharers;
    if (blockIdx.x < extra * (base + 1)) {
        slab = blockIdx.x / (base + 1); place = blockIdx.x % (base + 1); sharers = base + 1;
    } else {
        const uint32_t rest = blockIdx.x - extra * (base + 1);
        slab = extra + rest / base; place = rest % base; sharers = base;
    }
    const uint32_t tile0 = place * p.tiles / sharers, tile1 = (place + 1) * p.tiles / sharers;
    const uint32_t kb0 = slab * p.k_blocks / p.slabs, kb1 = (slab + 1) * p.k_blocks / p.slabs;
    const uint32_t slab_stages = kb1 - kb0;
    const uint32_t k0 = kb0 * kStageK;
    const uint32_t slab_k = (kb1 * kStageK < p.cols ? kb1 * kStageK : p.cols) - k0;    // a multiple of 64
    const uint32_t total_steps = (tile1 - tile0) * slab_stages;                       // ring stages this CTA streams
    const uint32_t atoms_per_row_block = p.cols / 64;

    auto issue_stage = [&](uint32_t step) {
        const uint32_t tile = tile0 + step / slab_stages, kb = kb0 + step % slab_stages, stage = step % kStages;
        const uint32_t k_valid = min(kStageK, p.cols - kb * kStageK);
        const uint32_t sf_bytes = k_valid / 64 * kSfAtomBytes;
        const uint32_t dst = smem_u32(smem + stage * kStageBytes), full = bar_full + 8 * stage;
        mbar_expect_tx(full, kStageCodeBytes + sf_bytes);
        tma_load_2d(dst, &map_weight, kb * 128, tile * kTileM, full);
        bulk_load(dst + kStageCodeBytes, p.weight_sf + (static_cast<uint64_t>(tile) * atoms_per_row_block + kb * 4) * kSfAtomBytes,
                  sf_bytes, full);
    };
    // The first ring fill goes out before anything else: weights do not depend on the launch before this one,
    // so HBM is busy while that launch drains and while the activations are split below.
    if (threadIdx.x == 0) {
        const uint32_t first = total_steps < kStages ? total_steps : kStages;
        for (uint32_t step = 0; step < first; ++step) issue_stage(step);
    }

    // ---- split the slab's activations into residual NVFP4 terms (all warps) ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t groups = slab_k / 16, items = p.tokens * groups;
    for (uint32_t i = threadIdx.x; i < items; i += kThreads) {
        const uint32_t token = i / groups, group = i - token * groups;
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<uint64_t>(token) * p.cols + k0 + group * 16);
        const uint4 lo = __ldcg(src), hi = __ldcg(src + 1);
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint32_t largest = 0;
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            largest = max(largest, max((w[j] << 16) & 0x7fff0000u, w[j] & 0x7fff0000u));   // magnitudes order like their bit patterns
        }
        if (largest >= 0x7f800000u) row_max[8 + token] = 1;
        atomicMax(&row_max[token], largest);
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        // term 0 divides by 2^(e - 7), e the exponent of the row's largest magnitude: its block scales come out
        // below 43 (E4M3 reaches 448) and groups down to 2^-13 of the row's largest still get a normal scale.
        // Every further term divides by 8 times less. Clamped so that all six stay normal f32 numbers.
        int field = static_cast<int>(row_max[threadIdx.x] >> 23);
        field = field < 30 ? 30 : (field > 250 ? 250 : field);
        float scale = __uint_as_float(static_cast<uint32_t>(field - 7) << 23);
        if (row_max[8 + threadIdx.x]) scale = __uint_as_float(0x7fc00000u);   // a NaN or infinity in the row: the row's outputs are NaN
        term_scale[threadIdx.x] = scale;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < items; i += kThreads) {
        const uint32_t token = i / groups, group = i - token * groups;
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<uint64_t>(token) * p.cols + k0 + group * 16);
        const uint4 lo = __ldcg(src), hi = __ldcg(src + 1);
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float residual[16];
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            residual[2 * j] = __uint_as_float(w[j] << 16);
            residual[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
        float scale = term_scale[token];
        if (!(scale == scale)) scale = 1.0f;     // the codes of a non-finite row do not matter
        const uint32_t chunk = group >> 4, unit = (group & 15) >> 1, half = group & 1;
#pragma unroll
        for (uint32_t term = 0; term < kTerms; ++term) {
            uint32_t packed[2], scale_code;
            quantise_term(residual, scale, term + 1 < kTerms, packed, &scale_code);
            scale *= 0.125f;
            const uint32_t n = term * 8 + token;
            uint8_t* row = act_codes + chunk * kChunkBytes + (n >> 3) * 1024 + (n & 7) * 128;
            *reinterpret_cast<uint2*>(row + ((unit ^ (n & 7)) << 4) + half * 8) = make_uint2(packed[0], packed[1]);
            act_sf[(group >> 2) * kSfAtomBytes + (n & 31) * 16 + (n >> 5) * 4 + (group & 3)] = static_cast<uint8_t>(scale_code);
        }
    }
    // the tensor core reads shared memory through the asynchronous proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer: the rest of the stream ----------------
        uint32_t phase = 0;
        for (uint32_t step = kStages; step < total_steps; ++step) {
            const uint32_t stage = step % kStages;
            if (!mbar_wait(bar_empty + 8 * stage, phase, abort_flag, p.status_word, kErrTcProducer)) break;
            issue_stage(step);
            if (stage == kStages - 1) phase ^= 1;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = instr_desc(kCols);
        const uint32_t tmem_sf_act = tmem_base + kTmemSfAct;
        // the activations' block scales: tensor-memory resident for the whole launch
        for (uint32_t a = 0; a < slab_k / 64; ++a) tc_copy_sf(tmem_sf_act + 4 * a, sf_desc(smem_u32(act_sf) + a * kSfAtomBytes));
        const uint64_t act_desc0 = operand_desc(smem_u32(act_codes));
        uint32_t step = 0, phase = 0;
        uint32_t acc_phase[2] = {0, 0};
        bool alive = true;
        for (uint32_t tile = tile0; alive && tile < tile1; ++tile) {
            const uint32_t buffer = (tile - tile0) & 1;
            // the epilogue must have drained this buffer (two tiles ago)
            if (!mbar_wait(bar_acc_empty + 8 * buffer, acc_phase[buffer] ^ 1, abort_flag, p.status_word, kErrTcAccEmpty)) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + kTmemAcc + buffer * 64;
            for (uint32_t s = 0; s < slab_stages; ++s, ++step) {
                const uint32_t stage = step % kStages;
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status_word, kErrTcFull)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint32_t stage_smem = smem_u32(smem + stage * kStageBytes);
                const uint64_t weight_desc = operand_desc(stage_smem), act_desc = act_desc0 + s * (kChunkBytes >> 4);
                const uint32_t tmem_sf_weight = tmem_base + kTmemSfWeight + stage * 16;
                const uint32_t k_steps = min(kStageK, slab_k - s * kStageK) / 64;
                for (uint32_t k = 0; k < k_steps; ++k) {
                    tc_copy_sf(tmem_sf_weight + 4 * k, sf_desc(stage_smem + kStageCodeBytes + k * kSfAtomBytes));
                    // each MMA consumes 64 k = 32 bytes of every row: advance the start address by 32 >> 4
                    tc_mma(acc, weight_desc + 2 * k, act_desc + 2 * k, idesc, tmem_sf_weight + 4 * k, tmem_sf_act + 4 * (s * 4 + k),
                           (s | k) ? 1u : 0u);
                }
                tc_commit(bar_empty + 8 * stage);   // frees the stage when these MMAs have read it
                if (stage == kStages - 1) phase ^= 1;
            }
            if (alive) tc_commit(bar_acc_full + 8 * buffer);
            acc_phase[buffer] ^= 1;
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------- epilogue: accumulator -> sums per token -> finished rows or a partial ----------------
        const uint32_t quadrant = warp & 3;          // tensor-memory lanes this warp may read: 32 * quadrant .. + 31
        uint32_t acc_phase[2] = {0, 0};
        for (uint32_t tile = tile0; tile < tile1; ++tile) {
            const uint32_t buffer = (tile - tile0) & 1;
            if (!mbar_wait(bar_acc_full + 8 * buffer, acc_phase[buffer], abort_flag, p.status_word, kErrTcAccFull)) break;
            acc_phase[buffer] ^= 1;
            tc_fence_after();
            uint32_t v[3][16];
            const uint32_t taddr = tmem_base + kTmemAcc + buffer * 64 + ((quadrant * 32) << 16);
            tc_load16(taddr, v[0]);
            tc_load16(taddr + 16, v[1]);
            tc_load16(taddr + 32, v[2]);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buffer);   // the buffer is free for the tile after next
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
            contribute_rows(p, tile, quadrant, slab, lane, y);
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
struct TcGeometry {
    uint32_t tiles, k_blocks, slabs, ctas;
    uint64_t partial_bytes;
};

// Slabs: at least enough for a slab's activations to fit shared memory; more when there are fewer row tiles than
// SMs (so that every SM streams) or when that evens out the load. The cost of a candidate is the number of ring
// stages of its busiest CTA.
TcGeometry tc_geometry(uint32_t physical_rows, uint32_t cols, uint32_t sm_count) {
    TcGeometry g{};
    g.tiles = physical_rows / kTileM;
    g.k_blocks = (cols + kStageK - 1) / kStageK;
    const uint32_t least = (g.k_blocks + kMaxSlabStages - 1) / kMaxSlabStages;
    uint64_t best_cost = UINT64_MAX;
    for (uint32_t slabs = least; slabs <= g.k_blocks && slabs <= sm_count; ++slabs) {
        const uint64_t items = static_cast<uint64_t>(g.tiles) * slabs;
        const uint32_t ctas = items < sm_count ? static_cast<uint32_t>(items) : sm_count;
        if (ctas < slabs) continue;
        const uint32_t fewest_sharers = ctas / slabs;                                      // CTAs of the slabs that have one less
        const uint32_t most_tiles = (g.tiles + fewest_sharers - 1) / fewest_sharers;
        const uint32_t most_stages = (g.k_blocks + slabs - 1) / slabs;
        // every slab costs each row group one hand-over (about a stage's time per eight of them at the end of the launch)
        const uint64_t cost = static_cast<uint64_t>(most_tiles) * most_stages * 8 + slabs * 4;
        if (cost < best_cost) {
            best_cost = cost;
            g.slabs = slabs;
            g.ctas = ctas;
        }
        if (slabs >= least + 24) break;
    }
    g.partial_bytes = g.slabs > 1 ? static_cast<uint64_t>(g.tiles) * 4 * g.slabs * kSlotFloats * 4 : 0;
    return g;
}

bool check_tc_scalars(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t* physical_rows) {
    if (a->reserved0 || a->reserved1 || a->epilogue > AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) return false;
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

// `partial_offset` .. `partial_limit`: the part of the plan scratch this launch may use for its partial sums.
bool check_tc(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
              const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint64_t partial_offset, uint64_t partial_limit, bool full,
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
    if (!g.slabs || g.tiles * 4 > kMaxGroups || partial_offset < kCounterBytes || partial_limit < partial_offset ||
        g.partial_bytes > partial_limit - partial_offset) {
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

augur_cuda_result_v1 launch_tc(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                               const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t member, uint64_t partial_offset) {
    const bool pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    const uint32_t physical_rows = pair ? 2 * a->rows : a->rows;
    const TcGeometry g = tc_geometry(physical_rows, a->cols, plan->sm_count);
    CUtensorMap map;
    if (!weight_map(&map, a->weight, physical_rows, a->cols)) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
    TcParams p{};
    p.weight_sf = reinterpret_cast<const uint8_t*>(a->weight) + tcgen05_codes_bytes(physical_rows, a->cols);
    p.x = reinterpret_cast<const uint16_t*>(a->input_bf16);
    p.out = reinterpret_cast<void*>(a->output);
    p.counters = reinterpret_cast<uint32_t*>(plan->scratch + member * kCounterRegionBytes);
    p.partials = reinterpret_cast<float*>(plan->scratch + partial_offset);
    p.status_word = plan->status_word;
    p.rows = physical_rows; p.out_rows = a->rows; p.cols = a->cols; p.tokens = a->tokens; p.epilogue = a->epilogue;
    p.tiles = g.tiles; p.k_blocks = g.k_blocks; p.slabs = g.slabs;
    p.global_a = a->global_scale; p.global_b = a->global_scale_b;
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
    cudaLaunchKernelEx(&config, gemv_tc_kernel, map, p);
    count_launch();
    return submitted();
}

}  // namespace

cudaError_t gemv_tc_configure_device() {
    return cudaFuncSetAttribute(gemv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
        if (g.partial_bytes > worst) worst = g.partial_bytes;
    }
    *out_bytes = kCounterBytes + worst;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_preflight_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_tc(d, s, plan, a, kCounterBytes, plan ? plan->scratch_bytes : 0, true, &failure)) return failure;
    CUtensorMap probe;
    const uint32_t physical = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 ? 2 * a->rows : a->rows;
    return weight_map(&probe, a->weight, physical, a->cols) ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, augur_cuda_nvfp4_sm100_plan_v1* plan, const augur_cuda_nvfp4_sm100_gemv_args_v1* a) {
    augur_cuda_result_v1 failure;
    if (!check_tc(d, s, plan, a, kCounterBytes, plan ? plan->scratch_bytes : 0, false, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    const cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    return launch_tc(s, plan, a, 0, kCounterBytes);
}
