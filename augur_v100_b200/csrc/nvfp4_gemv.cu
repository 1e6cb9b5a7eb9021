// Small-token (1..8) NVFP4 linear for sm_100a: a bandwidth-bound dequantising GEMV.
//
// Data path per weight block (32 rows x 128 k, 2304 bytes, already in mma fragment
// order): six 128-bit coalesced loads per lane -> cvt.rn.f16x2.e2m1x2 (codes) and
// cvt.rn.f16x2.e4m3x2 (block scales) -> one packed f16 multiply per fragment register
// (e2m1 x e4m3 is exact in f16) -> mma.sync.m16n8k16 with the 8 token rows on the
// MMA n dimension and f32 accumulators. An FP32 SIMT inner product cannot keep up
// with HBM at 8 tokens (8 FMA per weight element), so the inner product is on the
// tensor cores and the ALU work is the dequantisation only.
//
// Activations: each CTA stages the BF16 activations of its k-slab into shared memory
// as f16 B fragments, multiplied per token by an exact power of two chosen so that the
// largest magnitude lands in [2^14, 2^15); partial sums are scaled back before they
// leave the warp, so CTAs need not agree on the exponent.
//
// Work split (balanced over any grid): the block space of a k-slab is cut into equal
// contiguous spans, one per CTA, and each CTA's span into equal contiguous spans, one
// per warp. Row groups that straddle a warp boundary are combined in shared memory in
// warp order; row groups that straddle a CTA or slab boundary are combined through
// plan scratch with an arrival counter, the last arriver summing the slots in a fixed
// order. Nothing spins, and the result does not depend on scheduling.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nvfp4_internal.h"
#include "nvfp4_layout.cuh"

namespace augur_sm100 {
namespace {

static_assert(sizeof(augur_cuda_nvfp4_sm100_gemv_args_v1) == 88, "gemv ABI");
static_assert(sizeof(augur_cuda_nvfp4_sm100_mlp_args_v1) == 184, "mlp ABI");

constexpr uint32_t kWarps = 16;
constexpr uint32_t kDepth = 2;             // weight blocks in flight per warp
constexpr uint32_t kMaxSlabBlocks = 40;    // 40 * 128 k = 5120 activations columns per slab (80 KB)
constexpr uint32_t kSlotFloats = 256;      // one partial tile: 32 lanes x 8 f32
// Plan scratch layout: two arrival-counter regions (one per member of a two-launch program)
// at fixed offsets, then partial-sum slots. Counters must read zero when a launch starts and
// every launch leaves them at zero; keeping them apart from the slots means no launch of any
// shape can ever leave slot data where another launch expects counters.
constexpr uint32_t kMaxGroups = 16384;
constexpr uint64_t kCounterRegionBytes = static_cast<uint64_t>(kMaxGroups) * 4;
constexpr uint64_t kCounterBytes = 2 * kCounterRegionBytes;

struct GemvParams {
    const uint8_t* weight;
    const uint16_t* x;
    void* out;
    float* partials;
    uint32_t* counters;
    uint32_t groups, kb_count, slabs, ctas_per_slab, max_contrib;
    uint32_t rows, cols, tokens, epilogue;
    float global_a, global_b;
};

struct GemvGeometry {
    uint32_t groups, kb_count, slabs, ctas_per_slab, max_contrib;
    uint64_t partial_bytes;   // partial-sum slots
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
    const uint64_t least_blocks = static_cast<uint64_t>(g.groups) * min_kbs;
    if (per_slab > least_blocks) per_slab = least_blocks;  // every CTA owns at least one block
    g.ctas_per_slab = static_cast<uint32_t>(per_slab);
    g.max_contrib = g.slabs * ((g.ctas_per_slab + g.groups - 1) / g.groups + 1);
    g.partial_bytes = static_cast<uint64_t>(g.groups) * g.max_contrib * kSlotFloats * 4;
    return g;
}

__device__ __forceinline__ uint4 ld_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Four bytes of two E2M1 codes each -> four f16x2 registers.
__device__ __forceinline__ void cvt_e2m1x8(uint32_t word, uint32_t (&a)[4]) {
    asm("{\n"
        ".reg .b8 c0, c1, c2, c3;\n"
        "mov.b32 {c0, c1, c2, c3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, c0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, c1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, c2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, c3;\n"
        "}"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
        : "r"(word));
}

// Four E4M3 bytes -> two f16x2 registers (bytes 0,1 and bytes 2,3).
__device__ __forceinline__ void cvt_e4m3x4(uint32_t word, uint32_t& lo, uint32_t& hi) {
    asm("{\n"
        ".reg .b16 h0, h1;\n"
        "mov.b32 {h0, h1}, %2;\n"
        "cvt.rn.f16x2.e4m3x2 %0, h0;\n"
        "cvt.rn.f16x2.e4m3x2 %1, h1;\n"
        "}"
        : "=r"(lo), "=r"(hi)
        : "r"(word));
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, __half2 b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), b);
    return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct WeightRegs {
    uint4 code[4];   // [tile*2 + quad]
    uint4 scale[2];  // [tile]
};

__device__ __forceinline__ void load_block(WeightRegs& r, const uint8_t* block, uint32_t lane) {
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) r.code[i] = ld_stream(block + (i * 32 + lane) * 16);
#pragma unroll
    for (uint32_t t = 0; t < 2; ++t) r.scale[t] = ld_stream(block + kStreamCodeBytes + (t * 8 + (lane >> 2)) * 16);
}

// acc[t*4 + i] += block(32 rows x 128 k) * activations, `act` points at this block's B fragments.
__device__ __forceinline__ void compute_block(float (&acc)[8], const WeightRegs& r, const uint4* act, uint32_t lane) {
    uint4 bfrag[4];
#pragma unroll
    for (uint32_t kp = 0; kp < 4; ++kp) bfrag[kp] = act[kp * 32 + lane];
#pragma unroll
    for (uint32_t t = 0; t < 2; ++t) {
        // scale bytes: x,y = row g (k-steps 0..3, 4..7); z,w = row g+8
        uint32_t sg[4], sh[4];  // f16x2 pairs: k-steps (0,1) (2,3) (4,5) (6,7)
        cvt_e4m3x4(r.scale[t].x, sg[0], sg[1]);
        cvt_e4m3x4(r.scale[t].y, sg[2], sg[3]);
        cvt_e4m3x4(r.scale[t].z, sh[0], sh[1]);
        cvt_e4m3x4(r.scale[t].w, sh[2], sh[3]);
        float(&d)[4] = *reinterpret_cast<float(*)[4]>(&acc[t * 4]);
#pragma unroll
        for (uint32_t q = 0; q < 2; ++q) {
            const uint4 cw = r.code[t * 2 + q];
            const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                const uint32_t ks = q * 4 + j;
                const __half2 pg = *reinterpret_cast<const __half2*>(&sg[ks >> 1]);
                const __half2 ph = *reinterpret_cast<const __half2*>(&sh[ks >> 1]);
                const __half2 scale_g = (ks & 1) ? __high2half2(pg) : __low2half2(pg);
                const __half2 scale_h = (ks & 1) ? __high2half2(ph) : __low2half2(ph);
                uint32_t a[4];
                cvt_e2m1x8(words[j], a);
                a[0] = hmul2_u32(a[0], scale_g);
                a[1] = hmul2_u32(a[1], scale_h);
                a[2] = hmul2_u32(a[2], scale_g);
                a[3] = hmul2_u32(a[3], scale_h);
                const uint4 b = bfrag[ks >> 1];
                mma_f16(d, a, (ks & 1) ? b.z : b.x, (ks & 1) ? b.w : b.y);
            }
        }
    }
}

// Which of `parts` equal contiguous spans of [0, total) holds index `at`.
__device__ __forceinline__ uint32_t span_of(uint64_t at, uint64_t total, uint32_t parts) {
    return static_cast<uint32_t>(((at + 1) * parts - 1) / total);
}

__device__ __forceinline__ void epilogue(const GemvParams& p, uint32_t group, const float (&v)[8], uint32_t lane) {
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
                out[static_cast<uint64_t>(token) * p.rows + row] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
            }
        }
        return;
    }
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t token = 2 * t4 + (i & 1);
        const uint32_t row = group * 32 + (i >> 2) * 16 + g + ((i >> 1) & 1) * 8;
        if (token < p.tokens) {
            const float value = v[i] * p.global_a;
            if (p.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) {
                static_cast<float*>(p.out)[static_cast<uint64_t>(token) * p.rows + row] = value;
            } else {
                static_cast<__nv_bfloat16*>(p.out)[static_cast<uint64_t>(token) * p.rows + row] = __float2bfloat16_rn(value);
            }
        }
    }
}

// One CTA's finished share of row group `group` in k-slab `slab` (whole warp calls this).
__device__ __forceinline__ void contribute(const GemvParams& p, uint32_t group, uint32_t slab, uint32_t cta_in_slab,
                                           const float (&v)[8], uint32_t lane) {
    uint32_t total = 0, mine = 0;
    for (uint32_t s = 0; s < p.slabs; ++s) {
        const uint32_t kbs = (s + 1) * p.kb_count / p.slabs - s * p.kb_count / p.slabs;
        const uint64_t blocks = static_cast<uint64_t>(p.groups) * kbs;
        const uint32_t first = span_of(static_cast<uint64_t>(group) * kbs, blocks, p.ctas_per_slab);
        const uint32_t last = span_of(static_cast<uint64_t>(group + 1) * kbs - 1, blocks, p.ctas_per_slab);
        if (s == slab) mine = total + (cta_in_slab - first);
        total += last - first + 1;
    }
    if (total == 1) {
        epilogue(p, group, v, lane);
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
    float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t j = 0; j < total; ++j) {
        const float4* slot = reinterpret_cast<const float4*>(slots + static_cast<uint64_t>(j) * kSlotFloats) + lane * 2;
        const float4 a = __ldcg(slot), b = __ldcg(slot + 1);
        sum[0] += a.x; sum[1] += a.y; sum[2] += a.z; sum[3] += a.w;
        sum[4] += b.x; sum[5] += b.y; sum[6] += b.z; sum[7] += b.w;
    }
    epilogue(p, group, sum, lane);
    if (lane == 0) p.counters[group] = 0;  // leave the counter clean for the next launch
}

__global__ void __launch_bounds__(kWarps * 32, 1) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint4* act = reinterpret_cast<uint4*>(smem);                                   // [kbs*4][32] x 16 B
    float* warp_partial = reinterpret_cast<float*>(smem + kMaxSlabBlocks * 4 * 512);  // [warps][2][256]
    __shared__ float s_amax[kWarps];
    __shared__ float s_inv_scale[8];
    __shared__ float s_scale[8];

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t slab = blockIdx.x / p.ctas_per_slab, cta_in_slab = blockIdx.x % p.ctas_per_slab;
    const uint32_t kb_lo = slab * p.kb_count / p.slabs;
    const uint32_t kbs = (slab + 1) * p.kb_count / p.slabs - kb_lo;
    const uint64_t blocks = static_cast<uint64_t>(p.groups) * kbs;
    const uint64_t c0 = cta_in_slab * blocks / p.ctas_per_slab, c1 = (cta_in_slab + 1) * blocks / p.ctas_per_slab;
    const uint64_t len = c1 - c0;
    const uint64_t w0 = c0 + warp * len / kWarps, w1 = c0 + (warp + 1) * len / kWarps;

    auto block_ptr = [&](uint64_t at) {
        const uint64_t group = at / kbs, kbi = at % kbs;
        return p.weight + (group * p.kb_count + kb_lo + kbi) * kStreamBlockBytes;
    };

    // Weight loads go out first so that HBM is busy while the activations are staged.
    WeightRegs ring[kDepth];
#pragma unroll
    for (uint32_t d = 0; d < kDepth; ++d) {
        if (w0 + d < w1) load_block(ring[d], block_ptr(w0 + d), lane);
    }

    // ---- stage activations of this k-slab as f16 B fragments ----
    {
        constexpr uint32_t kThreadsPerToken = kWarps * 32 / 8;
        const uint32_t token = threadIdx.x / kThreadsPerToken, within = threadIdx.x % kThreadsPerToken;
        const uint32_t chunks = kbs * (kStreamBlockK / 8);  // 16-byte chunks of 8 bf16 per token row
        const uint4* row = reinterpret_cast<const uint4*>(p.x + static_cast<uint64_t>(token) * p.cols + kb_lo * kStreamBlockK);
        const bool live = token < p.tokens;
        float amax = 0.0f;
        if (live) {
            for (uint32_t c = within; c < chunks; c += kThreadsPerToken) {
                const uint4 v = __ldg(row + c);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    amax = fmaxf(amax, fabsf(__uint_as_float(w[i] << 16)));
                    amax = fmaxf(amax, fabsf(__uint_as_float(w[i] & 0xffff0000u)));
                }
            }
        }
#pragma unroll
        for (uint32_t o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) s_amax[warp] = amax;
        __syncthreads();
        if (threadIdx.x < 8) {
            constexpr uint32_t kWarpsPerToken = kWarps / 8;
            float m = 0.0f;
            for (uint32_t i = 0; i < kWarpsPerToken; ++i) m = fmaxf(m, s_amax[threadIdx.x * kWarpsPerToken + i]);
            // power of two e with m * 2^e in [2^14, 2^15); e = 0 for zero or non-finite rows
            int e = 0;
            const uint32_t field = (__float_as_uint(m) >> 23) & 0xff;
            if (m > 0.0f && field != 0xff) {
                e = 141 - static_cast<int>(field);
                e = e > 126 ? 126 : e;
            }
            s_scale[threadIdx.x] = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
            s_inv_scale[threadIdx.x] = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
        }
        __syncthreads();
        const float scale = s_scale[token];
        for (uint32_t c = within; c < chunks; c += kThreadsPerToken) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live) v = __ldg(row + c);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            // chunk c holds k = 8c..8c+7 of the slab: k-step c/2, fragment register c%2,
            // word i of the chunk is the pair k%16 = 8(c%2) + 2i, +1  -> lane token*4 + i
            const uint32_t kstep = c >> 1, reg = c & 1;
            uint32_t* dst = reinterpret_cast<uint32_t*>(act) + ((kstep >> 1) * 32 + token * 4) * 4 + (kstep & 1) * 2 + reg;
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                const float lo = __uint_as_float(w[i] << 16) * scale;
                const float hi = __uint_as_float(w[i] & 0xffff0000u) * scale;
                const __half2 h = __floats2half2_rn(lo, hi);
                dst[i * 4] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        __syncthreads();
    }

    const uint32_t t4 = lane & 3;
    const float inv0 = s_inv_scale[2 * t4], inv1 = s_inv_scale[2 * t4 + 1];
    const uint64_t first_group = w0 / kbs;

    // ---- stream this warp's span of blocks ----
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint64_t seg_group = first_group;
    uint32_t seg_first_kbi = static_cast<uint32_t>(w0 % kbs);

    auto flush = [&](uint64_t group, uint32_t first_kbi, uint32_t last_kbi) {
        float v[8];
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) v[i] = acc[i] * ((i & 1) ? inv1 : inv0);
        if (first_kbi == 0 && last_kbi + 1 == kbs) {
            contribute(p, static_cast<uint32_t>(group), slab, cta_in_slab, v, lane);
        } else {
            const uint32_t slot = group == first_group ? 0 : 1;
            float4* dst = reinterpret_cast<float4*>(warp_partial + (warp * 2 + slot) * kSlotFloats) + lane * 2;
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) acc[i] = 0.0f;
    };

    for (uint64_t base = w0; base < w1; base += kDepth) {
#pragma unroll
        for (uint32_t d = 0; d < kDepth; ++d) {
            const uint64_t at = base + d;
            if (at < w1) {
                const uint64_t group = at / kbs;
                const uint32_t kbi = static_cast<uint32_t>(at % kbs);
                if (group != seg_group) {
                    flush(seg_group, seg_first_kbi, kbs - 1);
                    seg_group = group;
                    seg_first_kbi = 0;
                }
                compute_block(acc, ring[d], act + kbi * 128, lane);
                if (at + kDepth < w1) load_block(ring[d], block_ptr(at + kDepth), lane);
            }
        }
    }
    if (w1 > w0) flush(seg_group, seg_first_kbi, static_cast<uint32_t>((w1 - 1) % kbs));
    __syncthreads();

    // ---- combine row groups that were split between warps of this CTA ----
    if (len == 0) return;
    const uint64_t cta_first_group = c0 / kbs;
    const uint32_t cta_groups = static_cast<uint32_t>((c1 - 1) / kbs - cta_first_group + 1);
    for (uint32_t index = warp; index < cta_groups; index += kWarps) {
        const uint64_t group = cta_first_group + index;
        const uint64_t lo = group * kbs > c0 ? group * kbs : c0;
        const uint64_t hi = (group + 1) * kbs < c1 ? (group + 1) * kbs : c1;
        const uint32_t w_lo = span_of(lo - c0, len, kWarps), w_hi = span_of(hi - 1 - c0, len, kWarps);
        if (w_lo == w_hi && lo == group * kbs && hi == (group + 1) * kbs) continue;  // one warp had it all
        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t w = w_lo; w <= w_hi; ++w) {
            const uint64_t b0 = c0 + w * len / kWarps, b1 = c0 + (w + 1) * len / kWarps;
            if (b1 == b0) continue;
            const uint32_t slot = (b0 / kbs == group) ? 0 : 1;
            const float4* src = reinterpret_cast<const float4*>(warp_partial + (w * 2 + slot) * kSlotFloats) + lane * 2;
            const float4 a = src[0], b = src[1];
            sum[0] += a.x; sum[1] += a.y; sum[2] += a.z; sum[3] += a.w;
            sum[4] += b.x; sum[5] += b.y; sum[6] += b.z; sum[7] += b.w;
        }
        contribute(p, static_cast<uint32_t>(group), slab, cta_in_slab, sum, lane);
    }
}

constexpr uint32_t kGemvSmemBytes = kMaxSlabBlocks * 4 * 512 + kWarps * 2 * kSlotFloats * 4;

// ---- validation ---------------------------------------------------------------------------
bool check_gemv_scalars(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, bool* pair) {
    if (a->reserved0 || a->reserved1 || a->epilogue > AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32) return false;
    *pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    if (!a->rows || !a->cols || a->rows > INT_MAX || a->cols > INT_MAX) return false;
    if (static_cast<uint64_t>(a->rows) * a->cols > UINT32_MAX) return false;
    if (a->cols % kStreamBlockK != 0 || a->rows % (*pair ? 16 : 32) != 0) return false;
    if (a->tokens < 1 || a->tokens > AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) return false;
    if (!scale_ok(a->global_scale)) return false;
    if (*pair ? !scale_ok(a->global_scale_b) : a->global_scale_b != 0.0f) return false;
    if (a->weight_len_bytes != stream_extent_bytes(*pair, a->rows, a->cols)) return false;
    if (a->input_len_bytes != static_cast<uint64_t>(a->tokens) * a->cols * 2) return false;
    const uint64_t out_elem = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32 ? 4 : 2;
    return a->output_len_bytes == static_cast<uint64_t>(a->tokens) * a->rows * out_elem;
}

void gemv_ranges(const augur_cuda_nvfp4_sm100_gemv_args_v1* a, Range (&r)[3]) {
    r[0] = {a->weight, a->weight_len_bytes, 256};
    r[1] = {a->input_bf16, a->input_len_bytes, 16};
    r[2] = {a->output, a->output_len_bytes, 4};
}

// `partial_offset`..`partial_limit` is the part of the plan scratch this launch may use for slots.
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
        partial_limit < partial_offset || g.partial_bytes > partial_limit - partial_offset) {
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

void launch_gemv(augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_plan_v1* plan,
                 const augur_cuda_nvfp4_sm100_gemv_args_v1* a, uint32_t member, uint64_t partial_offset) {
    const bool pair = a->epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16;
    const GemvGeometry g = geometry(a->rows, a->cols, pair, plan->sm_count);
    GemvParams p{};
    p.weight = reinterpret_cast<const uint8_t*>(a->weight);
    p.x = reinterpret_cast<const uint16_t*>(a->input_bf16);
    p.out = reinterpret_cast<void*>(a->output);
    p.counters = reinterpret_cast<uint32_t*>(plan->scratch + member * kCounterRegionBytes);
    p.partials = reinterpret_cast<float*>(plan->scratch + partial_offset);
    p.groups = g.groups; p.kb_count = g.kb_count; p.slabs = g.slabs; p.ctas_per_slab = g.ctas_per_slab;
    p.max_contrib = g.max_contrib;
    p.rows = a->rows; p.cols = a->cols; p.tokens = a->tokens; p.epilogue = a->epilogue;
    p.global_a = a->global_scale; p.global_b = a->global_scale_b;
    gemv_kernel<<<g.slabs * g.ctas_per_slab, kWarps * 32, kGemvSmemBytes, s->stream>>>(p);
    count_launch();
}

}  // namespace

// Called once per device from plan creation (a bind-time call): raises the kernel's
// dynamic shared-memory limit.
cudaError_t gemv_configure_device() {
    return cudaFuncSetAttribute(gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes);
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
            if (g.partial_bytes > worst) worst = g.partial_bytes;
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
        a->down.epilogue == AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16) {
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
    launch_gemv(s, plan, &a->gate_up, 0, kCounterBytes);
    augur_cuda_result_v1 first = submitted();
    if (first.status != AUGUR_CUDA_STATUS_OK) return first;
    launch_gemv(s, plan, &a->down, 1, down_offset);
    return submitted();
}
