// BF16 vocabulary head for 1..8 token rows on sm_100a: logits[token][row] = sum_k w[row][k] * x[token][k] with
// BF16 weights read in place, F32 activations and F32 results.
//
// What it replaces: the register-blocked FP32 kernel of the reference
// (crates/augur-cuda-sys/native/augur_dflash_llama_bf16_head.cuh:24-72, f32_rw4: BF16 widened exactly to F32,
// exact F32 products, F32 accumulation). At 8 token rows the head is bandwidth-bound on a B200 only if the
// inner product is cheap: 3.2e12 weights per second at HBM rate would need 26e12 FP32 FMAs per second, most of
// what the FP32 pipes have. Here the weights go to the tensor cores as they are (mma.sync m16n8k16, BF16 A
// operand straight from global memory in fragment order, the 8 token rows on n), and the F32 activations are
// split on the fly into three BF16 terms x = hi + mid + lo (8 + 8 + 8 significand bits: exact), one MMA per term.
// Every product is exact, as in the reference; only the order of the F32 additions differs.
//
// A warp owns 16-row tiles over the whole k range (no reduction between warps); a lane's weight loads are
// 16-byte vectors, two per row and 64-k step, kept four steps ahead in registers, so that a CTA of 16 warps has
// 128 KB in flight. The activations sit in shared memory as F32, each token row padded so that a quarter warp's
// 16-byte reads fall in different banks, with the 16-byte pieces of a 64-k block ordered the way the lanes
// consume them.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "nvfp4_internal.h"

namespace augur_sm100 {
namespace {

static_assert(sizeof(augur_cuda_nvfp4_sm100_bf16_head_args_v1) == 64, "bf16 head ABI");

constexpr uint32_t kHeadWarps = 16;
constexpr uint32_t kHeadThreads = kHeadWarps * 32;
constexpr uint32_t kHeadAhead = 4;          // 64-k steps of weights a lane keeps in flight
constexpr uint32_t kHeadRowPad = 16;        // floats between token rows in shared memory beyond cols (64 bytes)
constexpr uint32_t kHeadMaxSmem = 200 * 1024;

__device__ __forceinline__ void mma_bf16_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two F32 values -> their three BF16 terms, packed (low half = first value). x = hi + mid + lo exactly: each
// subtraction is exact, and after two of them at most 8 significand bits are left.
__device__ __forceinline__ void split3(float x0, float x1, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(x1), "f"(x0));
    const float r0 = x0 - __uint_as_float(hi << 16), r1 = x1 - __uint_as_float(hi & 0xffff0000u);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(mid) : "f"(r1), "f"(r0));
    const float s0 = r0 - __uint_as_float(mid << 16), s1 = r1 - __uint_as_float(mid & 0xffff0000u);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(s1), "f"(s0));
}

__device__ __forceinline__ uint4 load_weights(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(kHeadThreads, 1)
bf16_head_kernel(const uint16_t* __restrict__ weight, const float* __restrict__ x, float* __restrict__ out, uint32_t rows,
                 uint32_t cols, uint32_t tokens) {
    extern __shared__ __align__(16) float staged[];     // [8 token rows][cols + pad], the 16-byte pieces of a 64-k block reordered
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t4 = lane & 3;
    const uint32_t stride = cols + kHeadRowPad;
    // Lane (g, t4) takes the weights k = 64c + 16 t4 .. + 15 of a 64-k block c; MMA step j of the block contracts
    // its k = 64c + 16 t4 + 4j .. + 3 with the same k of token g, which therefore sit at piece j * 4 + t4.
    for (uint32_t i = threadIdx.x; i < 8 * (cols / 4); i += kHeadThreads) {
        const uint32_t token = i / (cols / 4), piece = i - token * (cols / 4);          // 16-byte piece of the row
        const uint32_t block = piece >> 4, owner = (piece >> 2) & 3, step = piece & 3;   // k = 64 block + 16 owner + 4 step
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (token < tokens) v = __ldcg(reinterpret_cast<const float4*>(x + static_cast<uint64_t>(token) * cols) + piece);
        *reinterpret_cast<float4*>(staged + token * stride + block * 64 + (step * 4 + owner) * 4) = v;
    }
    __syncthreads();

    // this warp's 16-row tiles: equal contiguous shares of all tiles over all warps of the grid
    const uint32_t tiles = rows / 16, warps = gridDim.x * kHeadWarps, me = blockIdx.x * kHeadWarps + warp;
    const uint32_t tile0 = static_cast<uint32_t>(static_cast<uint64_t>(me) * tiles / warps);
    const uint32_t tile1 = static_cast<uint32_t>(static_cast<uint64_t>(me + 1) * tiles / warps);
    const uint32_t blocks = cols / 64;
    const uint32_t total = (tile1 - tile0) * blocks;       // 64-k steps of this warp
    const float* mine = staged + g * stride + t4 * 4;      // token g, this lane's piece of step 0

    // weights of step s: rows g and g + 8 of its tile, 16 k each (two 16-byte vectors per row)
    auto fetch = [&](uint32_t s, uint4 (&w)[4]) {
        const uint32_t tile = tile0 + s / blocks, block = s - (s / blocks) * blocks;
        const uint4* row = reinterpret_cast<const uint4*>(weight + (static_cast<uint64_t>(tile) * 16 + g) * cols + block * 64 + t4 * 16);
        const uint4* other = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(row) + static_cast<uint64_t>(8) * cols);
        w[0] = load_weights(row);
        w[1] = load_weights(row + 1);
        w[2] = load_weights(other);
        w[3] = load_weights(other + 1);
    };
    uint4 ring[kHeadAhead][4];
#pragma unroll
    for (uint32_t a = 0; a < kHeadAhead; ++a) {
        if (a < total) fetch(a, ring[a]);
    }
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint32_t block = 0, tile = tile0;
    for (uint32_t s0 = 0; s0 < total; s0 += kHeadAhead) {
#pragma unroll
        for (uint32_t a = 0; a < kHeadAhead; ++a) {
            const uint32_t s = s0 + a;
            if (s >= total) break;
            const uint4 (&w)[4] = ring[a];
            const uint32_t row_g[8] = {w[0].x, w[0].y, w[0].z, w[0].w, w[1].x, w[1].y, w[1].z, w[1].w};
            const uint32_t row_h[8] = {w[2].x, w[2].y, w[2].z, w[2].w, w[3].x, w[3].y, w[3].z, w[3].w};
            const float* base = mine + block * 64;
            // The tensor core adds into its accumulator without rounding to nearest, so the sum of a 64-k block is
            // formed in a register set of its own (twelve MMAs deep) and added to the running sum with ordinary
            // round-to-nearest additions: the error grows like that of the reference's F32 chain.
            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                const float4 v = *reinterpret_cast<const float4*>(base + j * 16);
                uint32_t hi0, mid0, lo0, hi1, mid1, lo1;
                split3(v.x, v.y, hi0, mid0, lo0);
                split3(v.z, v.w, hi1, mid1, lo1);
                // the smallest terms first, so that they are not lost against a large partial sum
                mma_bf16_acc(part, row_g[2 * j], row_h[2 * j], row_g[2 * j + 1], row_h[2 * j + 1], lo0, lo1);
                mma_bf16_acc(part, row_g[2 * j], row_h[2 * j], row_g[2 * j + 1], row_h[2 * j + 1], mid0, mid1);
                mma_bf16_acc(part, row_g[2 * j], row_h[2 * j], row_g[2 * j + 1], row_h[2 * j + 1], hi0, hi1);
            }
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) acc[i] += part[i];
            if (s + kHeadAhead < total) fetch(s + kHeadAhead, ring[a]);
            if (++block == blocks) {
                // acc: rows g (first two) and g + 8 (last two) of the tile, tokens 2 t4 and 2 t4 + 1
                const uint32_t row = tile * 16 + g;
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const uint32_t token = 2 * t4 + (i & 1);
                    if (token < tokens) out[static_cast<uint64_t>(token) * rows + row + (i >> 1) * 8] = acc[i];
                    acc[i] = 0.0f;
                }
                block = 0;
                ++tile;
            }
        }
    }
}

bool check_head(int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_bf16_head_args_v1* a, bool full, uint32_t* tokens,
                augur_cuda_result_v1* failure) {
    *failure = invalid();
    if (!header_ok(d, s, a)) {
        if (a && s && d >= 0 && s->ordinal == d && a->abi_version != AUGUR_CUDA_ABI_VERSION_V1) {
            *failure = make_result(AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH);
        }
        return false;
    }
    if (!a->rows || !a->cols || a->rows % 16 != 0 || a->cols % 64 != 0 || a->rows > (1u << 30) || a->cols > (1u << 20)) return false;
    if (a->weight_len_bytes != static_cast<uint64_t>(a->rows) * a->cols * 2) return false;
    const uint64_t row_bytes = static_cast<uint64_t>(a->cols) * 4;
    if (a->input_len_bytes % row_bytes != 0) return false;
    const uint64_t count = a->input_len_bytes / row_bytes;
    if (count < 1 || count > AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) return false;
    *tokens = static_cast<uint32_t>(count);
    if (a->output_len_bytes != count * a->rows * 4) return false;
    if (8ull * (a->cols + kHeadRowPad) * 4 > kHeadMaxSmem) return false;   // the activations must fit shared memory
    // 16-byte vector loads of weights and activations (the reference's rw4 entry asks the same)
    const Range r[3] = {{a->weight, a->weight_len_bytes, 16}, {a->input, a->input_len_bytes, 16}, {a->output, a->output_len_bytes, 4}};
    if (!all_disjoint(r, 3)) return false;
    return !full || inspect_device_ranges(d, r, 3, failure);
}

uint32_t head_smem_bytes(uint32_t cols) { return 8 * (cols + kHeadRowPad) * 4; }

}  // namespace
}  // namespace augur_sm100

using namespace augur_sm100;

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_bf16_head_preflight_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_bf16_head_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint32_t tokens = 0;
    if (!check_head(d, s, a, true, &tokens, &failure)) return failure;
    // a bind-time call: the kernel's shared-memory limit for this width
    const cudaError_t e = cudaFuncSetAttribute(bf16_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHeadMaxSmem);
    return e == cudaSuccess ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_bf16_head_prevalidated_submit_v1(
    int32_t d, augur_cuda_stream_t s, const augur_cuda_nvfp4_sm100_bf16_head_args_v1* a) {
    augur_cuda_result_v1 failure;
    uint32_t tokens = 0;
    if (!check_head(d, s, a, false, &tokens, &failure)) return failure;
    if (consume_injected_fault()) return make_result(AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED);
    cudaError_t e = cudaSetDevice(d);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    static int sm_count[64];               // per device, looked up once (a host-side attribute query, no allocation)
    if (d >= 64) return invalid();
    if (!sm_count[d]) {
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(bf16_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kHeadMaxSmem);
        if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
        sm_count[d] = sms;
    }
    const int sms = sm_count[d];
    const uint32_t tiles = a->rows / 16;
    uint32_t grid = static_cast<uint32_t>(sms);
    if (grid * kHeadWarps > tiles) grid = (tiles + kHeadWarps - 1) / kHeadWarps;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t config{};
    config.stream = s->stream;
    config.attrs = &attribute;
    config.numAttrs = 1;
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kHeadThreads);
    config.dynamicSmemBytes = head_smem_bytes(a->cols);
    cudaLaunchKernelEx(&config, bf16_head_kernel, reinterpret_cast<const uint16_t*>(a->weight), reinterpret_cast<const float*>(a->input),
                       reinterpret_cast<float*>(a->output), a->rows, a->cols, tokens);
    count_launch();
    return submitted();
}
