// tcgen05 / TMA / mbarrier wrappers, shared-memory and instruction descriptors, and the BF16 -> NVFP4
// quantiser arithmetic shared by the tensor-memory kernels of this library (prefill GEMM and the
// small-token tensor-memory linear).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace augur_sm100 {
namespace tc {

constexpr uint32_t kTileM = 128;          // rows of the 128-row MMA operand per tile
constexpr uint32_t kWaitLimit = 20u * 1000u * 1000u;

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait. Returns false (after raising the abort flag) if the phase never completes
// or if another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status_word, uint32_t code) {
    for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status_word, 0u, code);
    return false;
}

// The same with the hardware's suspended wait: the thread gives up its issue slots until the phase completes
// or about a microsecond has passed, instead of polling. For roles that have nothing else to do.
__device__ __forceinline__ bool mbar_wait_suspended(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                    uint32_t* status_word, uint32_t code) {
    for (uint32_t spin = 0; spin < (1u << 21); ++spin) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(bar), "r"(parity), "r"(1000u)
            : "memory");
        if (done) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status_word, 0u, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_copy_sf(uint32_t tmem, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_load32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (64-bit): start address >> 4 in bits [0,14), leading
// byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in
// [46,48), swizzle mode in [61,64) (0 = none, 2 = 128-byte).
// K-major 128-byte-swizzled operand tile: rows are 128 bytes apart, 8-row groups 1024 bytes.
__device__ __forceinline__ uint64_t operand_desc(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Scale-factor atom for tcgen05.cp 32x128b: 32 rows of 16 bytes, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
}
// Instruction descriptor, block-scaled: A/B format E2M1 (1) at bits [7,10) / [10,13), both
// K-major, N >> 3 at [17,23), scale format UE4M3 (0) at bit 23, M >> 4 at [24,29), K = 64.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((kTileM >> 4) << 24);
}


// max(a, b, c), NaN if any is.
__device__ __forceinline__ float max_or_nan(float a, float b, float c) {
    float d;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Smallest positive E4M3 code whose value is >= d (d > 0), 126 if none.
__device__ __forceinline__ uint32_t e4m3_ceil_code(float d) {
    if (d > 448.0f) return 126;
    if (d <= 0x1p-6f) {                          // subnormal range: multiples of 2^-9, and 2^-6 itself
        const float steps = d * 512.0f;          // exact
        uint32_t m = static_cast<uint32_t>(ceilf(steps));
        return m < 1 ? 1 : m;                     // m == 8 is code 8 = 2^-6
    }
    const uint32_t bits = __float_as_uint(d);
    uint32_t exponent = (bits >> 23) - 127 + 7;  // E4M3 biased exponent, >= 1 here
    uint32_t mantissa = (bits >> 20) & 7;
    if (bits & 0xfffffu) ++mantissa;             // round up
    if (mantissa == 8) { mantissa = 0; ++exponent; }
    return exponent * 8 + mantissa;
}

__device__ __forceinline__ float e4m3_positive_value(uint32_t code) {
    const uint32_t exponent = code >> 3, mantissa = code & 7;
    return exponent == 0 ? static_cast<float>(mantissa) * 0x1p-9f
                         : __uint_as_float(((exponent + 120) << 23) | (mantissa << 20));
}

// Nearest E2M1 level; a tie goes to the smaller magnitude; zero is always code 0. |v| <= 6.
// From 1 upward E2M1 is a float with one mantissa bit, so rounding the f32 pattern to that bit with
// "ties down" (add half an ulp minus one, truncate) gives exponent and mantissa at once:
// 1 -> code 2, 1.5 -> 3, 2 -> 4, 3 -> 5, 4 -> 6, 6 -> 7. Below 1 the levels are 0, 0.5 and 1.
// `v` is the quotient as computed; the clamp to [-6, 6] is folded in: the magnitude is cut at 6, and a NaN
// quotient, which fmin(fmax(v, -6), 6) sends to -6, is negative here as well.
__device__ __forceinline__ uint32_t e2m1_nearest(float v, float* level) {
    const float a = fminf(fabsf(v), 6.0f);
    uint32_t m;
    if (a < 1.0f) {
        m = (a > 0.25f ? 1u : 0u) + (a > 0.75f ? 1u : 0u);
    } else {
        m = (__float_as_uint(a) + (0x1fffffu - (252u << 22))) >> 22;   // round to one mantissa bit, ties toward zero
    }
    const float l = m < 2 ? 0.5f * static_cast<float>(m) : __uint_as_float((m + 252u) << 22);
    const bool negative = !(v >= 0.0f) && m != 0;
    *level = negative ? -l : l;
    return negative ? (m | 8u) : m;
}

// Eight quotients -> eight codes, element i in nibble i, by the hardware converter: round to nearest even,
// magnitudes above 6 (infinities too) to 6. It differs from "nearest, ties toward zero, zero always code 0" in
// three places, put right here. At 0.75, 1.75 and 3.5 "even" is the larger level. A tie is a value of at most
// three significant bits; every quotient that short (low 21 bits of the pattern zero) goes in one or two ulps
// nearer to zero, which takes a tie to the level below and changes nothing else: the values passed over
// are not short, so none of them is a tie, and a zero stays a zero. A negative quotient that rounds to zero
// comes out as code 8. And a NaN comes out as +6 (the caller keeps groups with a NaN off this path).
__device__ __forceinline__ float off_the_tie(float q) {
    return (__float_as_uint(q) & 0x1fffffu) == 0 ? __fmul_rn(q, 0x1.fffffcp-1f) : q;   // q * (1 - 2^-23)
}
__device__ __forceinline__ uint32_t e2m1x8_nearest(const float2 (&q)[4]) {
    uint32_t codes;
    asm("{\n .reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n}"
        : "=r"(codes)
        : "f"(off_the_tie(q[0].x)), "f"(off_the_tie(q[0].y)), "f"(off_the_tie(q[1].x)), "f"(off_the_tie(q[1].y)),
          "f"(off_the_tie(q[2].x)), "f"(off_the_tie(q[2].y)), "f"(off_the_tie(q[3].x)), "f"(off_the_tie(q[3].y)));
    const uint32_t nonzero = (codes | (codes >> 1) | (codes >> 2)) & 0x11111111u;   // bit 0 of every nibble with a magnitude
    return codes & ((nonzero << 3) | 0x77777777u);
}

// The signed levels of eight codes (hardware E2M1 -> F16 pairs, widened).
__device__ __forceinline__ void e2m1x8_levels(uint32_t codes, float2 (&level)[4]) {
    uint32_t pair[4];
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(pair[0]), "=r"(pair[1]), "=r"(pair[2]), "=r"(pair[3])
        : "r"(codes));
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) level[i] = __half22float2(*reinterpret_cast<const __half2*>(&pair[i]));
}

// The 16 quotients of a group share one divisor. With y = RN(1/d), two Newton steps on the quotient (each
// an exact FMA residual) end on the correctly rounded x / d whenever d and x are well inside the normal
// range and d is not of the all-ones mantissa form; the kernel checks that once per group and otherwise
// divides. An x so small that a residual of the steps is subnormal (below 2^-103) has a quotient under
// 2^-40 (d is at least 2^-63 here), and the error that the lost bits leave in it is under 2^-87: code 0
// either way. This path holds no NaN (the caller checks), works on pairs of elements with the two-wide
// F32 instructions and rounds with the hardware converter.
template <bool kMoreTerms>
__device__ __forceinline__ void quantise_group_fast(float2 (&residual)[8], float divisor, float reciprocal, uint32_t (&packed)[2]) {
    const float2 y = make_float2(reciprocal, reciprocal), minus_d = make_float2(-divisor, -divisor);
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {
        float2 x[4], quotient[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            x[i] = residual[4 * half + i];
            float2 q = __fmul2_rn(x[i], y);
            float2 r = __ffma2_rn(q, minus_d, x[i]);
            q = __ffma2_rn(r, y, q);
            r = __ffma2_rn(q, minus_d, x[i]);
            quotient[i] = __ffma2_rn(r, y, q);
        }
        packed[half] = e2m1x8_nearest(quotient);
        if (kMoreTerms) {
            float2 level[4];
            e2m1x8_levels(packed[half], level);
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                // x - RN(level * d). The product is rounded one element at a time: a two-wide product feeding a
                // two-wide sum came out fused into one operation (one rounding), however it was written.
                const float2 product = make_float2(__fmul_rn(level[i].x, -divisor), __fmul_rn(level[i].y, -divisor));
                residual[4 * half + i] = __fadd2_rn(x[i], product);
            }
        }
    }
}

// The same without those conditions: IEEE division, rounding in software, NaN quotients included.
template <bool kMoreTerms>
__device__ __forceinline__ float quantise_element_any(float x, float divisor, uint32_t shift, uint32_t* packed) {
    const float normalized = divisor == 0.0f ? 0.0f : __fdiv_rn(x, divisor);
    float level;
    const uint32_t code = e2m1_nearest(normalized, &level);
    *packed += code << shift;   // disjoint fields: a sum, so that shift and add fuse
    return kMoreTerms ? __fsub_rn(x, __fmul_rn(level, divisor)) : x;
}
template <bool kMoreTerms>
__device__ __forceinline__ void quantise_group_any(float2 (&residual)[8], float divisor, uint32_t (&packed)[2]) {
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        residual[i].x = quantise_element_any<kMoreTerms>(residual[i].x, divisor, 8 * (i & 3), &packed[i >> 2]);
        residual[i].y = quantise_element_any<kMoreTerms>(residual[i].y, divisor, 8 * (i & 3) + 4, &packed[i >> 2]);
    }
}

// Block scale of a group with largest magnitude `maximum`: the smallest E4M3 value >= maximum / (6 g) and its
// code; returns the divisor scale * g.
__device__ __forceinline__ float group_divisor(float maximum, float global_scale, uint32_t* scale_code_out) {
    const float desired = __fdiv_rn(maximum, __fmul_rn(6.0f, global_scale));
    uint32_t scale_code = 0;
    float scale = 0.0f;
    if (desired > 0.0f) {
        scale_code = e4m3_ceil_code(desired);
        scale = e4m3_positive_value(scale_code);
    }
    *scale_code_out = scale_code;
    return __fmul_rn(scale, global_scale);
}

// One residual term of one 16-element group: the block scale, the 16 codes (nearest level of x / (scale * g),
// ties toward zero) and, if another term follows, the residual it quantises.
// `kMoreTerms` is a compile-time choice: the last term of a group needs neither the levels nor the residual.
template <bool kMoreTerms>
__device__ __forceinline__ void quantise_term_as(float2 (&residual)[8], float global_scale, uint32_t (&packed)[2],
                                                 uint32_t* scale_code_out) {
    // This maximum carries a NaN along, which keeps the group off the fast path; the reference's maximum
    // leaves NaNs out, and only the other path computes it.
    float maximum = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) maximum = max_or_nan(maximum, fabsf(residual[i].x), fabsf(residual[i].y));
    float divisor = group_divisor(maximum, global_scale, scale_code_out);
    const uint32_t divisor_field = (__float_as_uint(divisor) >> 23) & 0xffu, largest_field = (__float_as_uint(maximum) >> 23) & 0xffu;
    const bool fast = divisor_field >= 64u && divisor_field <= 190u && (__float_as_uint(divisor) & 0x7fffffu) != 0x7fffffu &&
                      largest_field <= 190u;
    packed[0] = packed[1] = 0;
    if (fast) {
        quantise_group_fast<kMoreTerms>(residual, divisor, __frcp_rn(divisor), packed);
    } else {
        maximum = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) maximum = fmaxf(maximum, fmaxf(fabsf(residual[i].x), fabsf(residual[i].y)));
        divisor = group_divisor(maximum, global_scale, scale_code_out);
        quantise_group_any<kMoreTerms>(residual, divisor, packed);
    }
}
__device__ __forceinline__ void quantise_term(float2 (&residual)[8], float global_scale, bool more_terms, uint32_t (&packed)[2],
                                              uint32_t* scale_code_out) {
    if (more_terms) {
        quantise_term_as<true>(residual, global_scale, packed, scale_code_out);
    } else {
        quantise_term_as<false>(residual, global_scale, packed, scale_code_out);
    }
}

}  // namespace tc
}  // namespace augur_sm100
