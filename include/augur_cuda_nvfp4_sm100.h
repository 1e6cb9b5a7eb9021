/* B200 (sm_100a) NVFP4 quantized-linear C ABI.
 *
 * A drop-in for the quantized-linear path of Augur's native CUDA layer
 * (crates/augur-cuda-sys). It keeps that layer's calling contract:
 *   - every operation is a pair  X_preflight_v1 / X_prevalidated_submit_v1
 *     (contract: crates/augur-cuda-sys/native/augur_qwen35_nvfp4_qpn_abi.h:134-139);
 *   - preflight (once per binding) validates the descriptor header, shapes,
 *     exact byte extents, alignment and pairwise disjointness of every range,
 *     then asks the driver who owns each range; it enqueues and allocates nothing;
 *   - prevalidated_submit (hot) repeats the scalar/extent/overlap checks, skips
 *     the driver queries, enqueues on the caller's stream and returns; it never
 *     synchronises and never allocates;
 *   - results are {status, raw_cuda_status}
 *     (crates/augur-cuda-sys/native/augur_cuda_runtime.h:31-55);
 *   - device addresses are opaque uint64 tokens, never dereferenced on the host
 *     (augur_cuda_runtime.h:66-72); the ABI retains nothing the caller owns
 *     (augur_cuda_runtime.h:4-12).
 *
 * The types shared with the reference header keep their names and layouts, so
 * this header can be included next to it (guards below).
 */
#ifndef AUGUR_CUDA_NVFP4_SM100_H
#define AUGUR_CUDA_NVFP4_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifndef AUGUR_CUDA_RUNTIME_H /* shared vocabulary of augur_cuda_runtime.h:17-72 */
#if defined(_WIN32)
#define AUGUR_CUDA_CALL __cdecl
#else
#define AUGUR_CUDA_CALL
#endif
#define AUGUR_CUDA_ABI_VERSION_V1 UINT32_C(1)
typedef int32_t augur_cuda_status_t;
enum {
    AUGUR_CUDA_STATUS_OK = 0,
    AUGUR_CUDA_STATUS_INVALID_ARGUMENT = -1,
    AUGUR_CUDA_STATUS_UNSUPPORTED_DEVICE = -2,
    AUGUR_CUDA_STATUS_OUT_OF_MEMORY = -3,
    AUGUR_CUDA_STATUS_RUNTIME_FAILURE = -4,
    AUGUR_CUDA_STATUS_SUBMISSION_FAILURE = -5,
    AUGUR_CUDA_STATUS_COMPLETION_FAILURE = -6,
    AUGUR_CUDA_STATUS_ABI_VERSION_MISMATCH = -7,
    AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED = -8
};
typedef struct augur_cuda_result_v1 {
    augur_cuda_status_t status;
    int32_t raw_cuda_status;
} augur_cuda_result_v1;
/* Opaque stream handle; its private layout is {int32 ordinal; cudaStream_t stream}
 * (crates/augur-cuda-sys/native/augur_cuda_internal.h:39-42). */
typedef struct augur_cuda_stream_handle augur_cuda_stream_handle;
typedef augur_cuda_stream_handle* augur_cuda_stream_t;
typedef uint64_t augur_cuda_device_ptr_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- physical layouts --------------------------------------------------- */
/* COMPACT is what a checkpoint loader hands over (crates/augur-formats/src/fp4.rs:17-21,
 * crates/augur-model-qwen35/src/checkpoint_quant.rs:93-152): codes [rows][cols/2]
 * (even k in the low nibble), scales [rows][cols/16], one f32 global scale.
 * The other three are lossless permutations of the same bits. */
#define AUGUR_NVFP4_SM100_LAYOUT_COMPACT UINT32_C(0)
/* 32-row x 128-k blocks of 2304 bytes in mma fragment order, codes bit-permuted so that each
 * fragment register is one shift-and-mask away: the decode/verify stream. */
#define AUGUR_NVFP4_SM100_LAYOUT_STREAM UINT32_C(1)
/* Same, with 16 gate rows and the matching 16 up rows in each block (fused SwiGLU). */
#define AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR UINT32_C(2)
/* Codes untouched (K-major rows, TMA-loadable) followed by block scales tiled into
 * 128-row x 4-scale atoms for tcgen05 block-scaled MMA. */
#define AUGUR_NVFP4_SM100_LAYOUT_TCGEN05 UINT32_C(3)

#define AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16 UINT32_C(0)
#define AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16 UINT32_C(1)
#define AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32 UINT32_C(2)

#define AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS UINT32_C(8)

/* ---- identity ------------------------------------------------------------ */
/* Replaces augur_cuda_abi_version (augur_cuda_runtime.h:74). */
uint32_t AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_abi_version(void);
/* Replaces augur_cuda_nvfp4_sm120_build_capability_v1
 * (crates/augur-cuda-sys/native/augur_nvfp4_stub.cu:10-13): 100 when the
 * library holds sm_100a code, 0 otherwise. */
uint32_t AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_build_capability_v1(void);

/* ---- stream handles (stand-alone use) -------------------------------------- */
/* Inside Augur the handles come from augur_cuda_stream_create
 * (augur_cuda_runtime.h:116-131) and are passed through unchanged. These three
 * exist so the library can be used and tested without the rest of the runtime. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_create_v1(
    int32_t ordinal, augur_cuda_stream_t* out_stream);
/* Wraps an existing cudaStream_t (for example the framework's current stream);
 * destroying the handle does not destroy the wrapped stream. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_adopt_v1(
    int32_t ordinal, void* raw_cuda_stream, augur_cuda_stream_t* out_stream);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_synchronize_v1(
    augur_cuda_stream_t stream);
/* Order of destruction: plans first, then the handle they were made on. A handle that still has
 * live plans is not destroyed (INVALID_ARGUMENT), because every plan call checks the plan against
 * the handle it was made on. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_destroy_v1(
    augur_cuda_stream_t stream);

/* ---- plan: stream-owned scratch ------------------------------------------- */
/* Replaces augur_cuda_qwen35_prefill_cublas_plan_v1 (augur_cuda_runtime.h:2019-2034):
 * created once per stream at bind time, owns the scratch the kernels need
 * (split-K partials, arrival counters, quantised-activation staging), and is
 * only accepted together with the stream that created it. Creation and
 * destruction are the only calls of this library that allocate device memory. */
typedef struct augur_cuda_nvfp4_sm100_plan_v1 augur_cuda_nvfp4_sm100_plan_v1;

typedef struct augur_cuda_nvfp4_sm100_plan_snapshot_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t scratch;
    uint64_t scratch_len_bytes;
    uint32_t sm_count;
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_plan_snapshot_v1;

/* Bytes of plan scratch needed by a small-token linear / a prefill linear. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_scratch_extent_host_v1(
    uint32_t rows, uint32_t cols, uint32_t tokens, uint64_t* out_bytes);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_scratch_extent_host_v1(
    uint32_t rows, uint32_t cols, uint32_t tokens, uint32_t activation_terms, uint64_t* out_bytes);
/* Bytes of plan scratch with which the prefill GEMM balances its last round of tiles on a device of
 * `sm_count` SMs: when the 256 x 256 tiles are not a multiple of the CTA pairs, the tiles left over are cut
 * along k between all pairs and the partial accumulators pass through the plan's scratch (one 256 KB slot
 * per pair behind the counter regions). With a smaller plan the GEMM keeps every tile whole; results agree
 * to f32 summation order. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_plan_scratch_extent_host_v1(
    uint32_t sm_count, uint64_t* out_bytes);

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_create_v1(
    int32_t ordinal, augur_cuda_stream_t stream, uint64_t scratch_len_bytes,
    augur_cuda_nvfp4_sm100_plan_v1** out_plan);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_describe_v1(
    const augur_cuda_nvfp4_sm100_plan_v1* plan, augur_cuda_nvfp4_sm100_plan_snapshot_v1* out);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_destroy_v1(
    augur_cuda_nvfp4_sm100_plan_v1* plan);

/* ---- repack: compact planes -> hot layout ---------------------------------- */
/* Replaces the pack_checkpoint pair (augur_qwen35_nvfp4_qpn_abi.h:14-18,146-148;
 * CPU counterpart crates/augur-repack/src/fp4_cpu.rs:45-55). Scale bytes >= 127
 * (sign bit or NaN) are the caller's to reject before upload, as the reference
 * loader does (crates/augur-backend/src/cuda_qwen35_qpn.rs:59-72); the host
 * repack below rejects them itself. */
typedef struct augur_cuda_nvfp4_sm100_repack_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t codes;      /* [rows][cols/2] */
    uint64_t codes_len_bytes;
    augur_cuda_device_ptr_t scales;     /* [rows][cols/16] */
    uint64_t scales_len_bytes;
    augur_cuda_device_ptr_t codes_b;    /* second matrix (up) for STREAM_PAIR, else 0 */
    uint64_t codes_b_len_bytes;
    augur_cuda_device_ptr_t scales_b;
    uint64_t scales_b_len_bytes;
    augur_cuda_device_ptr_t destination;
    uint64_t destination_len_bytes;
    uint32_t rows;                      /* of each source matrix */
    uint32_t cols;
    uint32_t layout;                    /* STREAM, STREAM_PAIR or TCGEN05 */
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_repack_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_extent_host_v1(
    uint32_t layout, uint32_t rows, uint32_t cols, uint64_t* out_bytes);
/* Host-memory twin of the device repack (same permutation, byte for byte) and its inverse. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_host_v1(
    uint32_t layout, uint32_t rows, uint32_t cols,
    const uint8_t* codes, const uint8_t* scales, const uint8_t* codes_b, const uint8_t* scales_b,
    uint8_t* destination, uint64_t destination_len_bytes);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_unpack_host_v1(
    uint32_t layout, uint32_t rows, uint32_t cols,
    const uint8_t* source, uint64_t source_len_bytes,
    uint8_t* codes, uint8_t* scales, uint8_t* codes_b, uint8_t* scales_b);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_repack_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_repack_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_repack_args_v1* args);

/* ---- checkpoint formats (host side, load time) -------------------------------------- */
/* How a checkpoint's per-tensor scalar enters the value
 * (crates/augur-model-qwen35/src/checkpoint_quant.rs:10-58): compressed-tensors divides by
 * weight_global_scale, ModelOpt (W4A4 and W4A16 exports alike) multiplies by weight_scale_2.
 * Activation scales of either format are not part of the weight and are not touched here. */
#define AUGUR_NVFP4_SM100_SCALE_COMPRESSED_TENSORS UINT32_C(0)
#define AUGUR_NVFP4_SM100_SCALE_MODELOPT UINT32_C(1)
/* The multiplier the kernels of this library take as global_scale. Rejects non-finite or
 * non-positive scalars (checkpoint_quant.rs:27-47) and results outside [2^-32, 24]. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_checkpoint_global_scale_host_v1(
    uint32_t convention, float checkpoint_scalar, float* out_global_scale);
/* CheckpointNvfp4Matrix::new's checks (checkpoint_quant.rs:113-133): non-empty, cols % 16,
 * exact plane extents, every block scale byte < 127. Rows need not be a tile multiple here. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_checkpoint_validate_host_v1(
    uint64_t rows, uint64_t cols, const uint8_t* codes, uint64_t codes_len_bytes,
    const uint8_t* scales, uint64_t scales_len_bytes);
/* Planes <-> GGML36 wire blocks (to_ggml_planes_into, checkpoint_quant.rs:157-189, and its
 * inverse): 36 bytes per 64 elements, lossless, cols % 64. The inverse rejects scale bytes >= 127. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_planes_to_ggml36_host_v1(
    uint64_t rows, uint64_t cols, const uint8_t* codes, const uint8_t* scales,
    uint8_t* wire, uint64_t wire_len_bytes);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_ggml36_to_planes_host_v1(
    uint64_t rows, uint64_t cols, const uint8_t* wire, uint64_t wire_len_bytes,
    uint8_t* codes, uint8_t* scales);

/* ---- dequantise to f32 (verification entry) -------------------------------- */
/* Replaces the expand pair (augur_qwen35_nvfp4_qpn_abi.h:23-29,153). Output is
 * bit-identical to Nvfp4CompactBlock::decode_ref (crates/augur-formats/src/fp4.rs:105-125):
 * fl(e2m1 * fl(e4m3 * global)), code 8 -> +0.0. `layout` says how `weight` is laid out. */
typedef struct augur_cuda_nvfp4_sm100_dequant_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t weight;     /* COMPACT: codes plane; otherwise the repacked tensor */
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t scales;     /* COMPACT only, else 0 */
    uint64_t scales_len_bytes;
    augur_cuda_device_ptr_t output_f32; /* [rows][cols]; STREAM_PAIR: gate rows then up rows */
    uint64_t output_len_bytes;
    uint32_t rows;
    uint32_t cols;
    uint32_t layout;
    float global_scale;
    float global_scale_b;               /* STREAM_PAIR: scale of the second matrix, else 0 */
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_dequant_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_dequant_f32_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_dequant_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_dequant_f32_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_dequant_args_v1* args);

/* ---- small-token linear: tokens 1..8 (decode and the fixed B8 verify batch) -- */
/* Replaces the project / prefill pairs for tokens <= 8
 * (augur_qwen35_nvfp4_qpn_abi.h:30-36,60-70,154) and the fused gate+up / SiLU
 * entries (same file :68-73,130-133). y[t][n] = bf16(global * sum_k w[n][k] x[t][k]),
 * BF16 activations, f32 accumulation. With EPILOGUE_SWIGLU the weight is a
 * STREAM_PAIR tensor and the output is bf16(silu(gate) * up), rows = intermediate size.
 * With EPILOGUE_LINEAR_F32 the unrounded f32 sums are written (tensor-parallel partials). */
typedef struct augur_cuda_nvfp4_sm100_gemv_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t weight;
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t input_bf16;   /* [tokens][cols] */
    uint64_t input_len_bytes;
    augur_cuda_device_ptr_t output;       /* [tokens][rows] bf16, or f32 for LINEAR_F32 */
    uint64_t output_len_bytes;
    uint32_t rows;
    uint32_t cols;
    uint32_t tokens;
    uint32_t epilogue;
    float global_scale;
    float global_scale_b;                 /* SWIGLU: scale of the up matrix, else 0 */
    uint32_t stored_rows;                 /* 0: all rows. Else (LINEAR epilogues) only the first stored_rows rows are written and
                                           * output is [tokens][stored_rows]: the weight's remaining rows are padding, as for the
                                           * 48-row gates of the reference's grouped projections, stored trimmed by the same write
                                           * (docs/AUGUR_GDN_GLUE_B8_20261016.md:18-23) */
    uint32_t reserved1;
} augur_cuda_nvfp4_sm100_gemv_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_args_v1* args);

/* The same small-token linear on the tensor-memory path: `weight` is in AUGUR_NVFP4_SM100_LAYOUT_TCGEN05
 * (for EPILOGUE_SWIGLU_BF16: one tensor of 2 * rows physical rows, 16 gate rows alternating with the
 * matching 16 up rows, as interleave_gate_up_host_v1 makes it), rows (physical) a multiple of 128, cols a
 * multiple of 64. The weights reach the tensor cores (tcgen05.mma kind::mxf4nvf4) as TMA delivers them;
 * the BF16 activations are split inside the launch into eight NVFP4 terms (radix-8 digits with power-of-two
 * scales), exact for every element within 2^-14 of its 16-element group's largest magnitude and to 2^-23 of that
 * magnitude below; a token row with a non-finite element gives NaN outputs. The CTAs of the launch meet through
 * counters in the plan's header: it needs all of them (at most two per SM) resident, so keep other long-running
 * kernels off the device meanwhile; a wait that runs out sets the plan's status word to 0x301..0x309, and reading
 * the status word then also clears the counters. Replaces the same reference entry points as
 * gemv_bf16_*_v1 (augur_qwen35_nvfp4_qpn_abi.h:134-156), with one weight layout for every token count. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_scratch_extent_host_v1(
    uint32_t rows, uint32_t cols, uint32_t epilogue, uint64_t* out_bytes);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tc_bf16_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_args_v1* args);


/* No counterpart in the reference. The same small-token linear for callers that may not allocate:
 * plan creation calls cudaMalloc, which a host cannot do once it has handed all device memory to
 * its own arena, or while it runs under an audited no-allocation rule (the discipline Augur's own
 * runtime applies to its serving loop). This entry needs no plan: its scratch is a fixed array of
 * AUGUR_NVFP4_SM100_STATIC_SCRATCH_BYTES inside the library image, held by every GPU that loads the
 * library until the process exits. It calls no cudaMalloc / cudaFree and no allocating library
 * routine. The first call on a device looks the array's device address up and sets the kernel's
 * shared-memory attribute; make that first call before any stream capture. Shapes whose scratch need
 * is larger than the array return AUGUR_CUDA_STATUS_INVALID_ARGUMENT with nothing enqueued (the two
 * MLP projections of the 27B profile, 17408 x 5120 and 5120 x 17408, fit). All calls share the one
 * array, which keeps the previous call's contents (the arrival counters are cleared on the stream
 * at the start of every call): two calls that overlap on the GPU race - keep them on one stream or
 * order them with events. Same descriptor and same checks as gemv_bf16_prevalidated_submit_v1,
 * without the driver queries of a preflight. */
#define AUGUR_NVFP4_SM100_STATIC_SCRATCH_BYTES (UINT32_C(4) << 20)
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_bf16_static_scratch_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_gemv_args_v1* args);
/* No counterpart in the reference. The device-side status word of that entry (0 = clean): the kernel's
 * bounded waits record where they gave up in the first four bytes of the fixed array, as they do in a
 * plan's status word. Copies the word to `out_status` on `stream` and waits for the stream; a non-zero
 * word is set back to zero afterwards, so a give-up is reported once. Allocates nothing. Devices other
 * than compute capability 10.x get AUGUR_CUDA_STATUS_UNSUPPORTED_DEVICE from both entries. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_static_scratch_status_v1(
    int32_t ordinal, augur_cuda_stream_t stream, uint32_t* out_status);

/* ---- MLP program: gate|up + SwiGLU, then down ------------------------------- */
/* Replaces CudaQwen35QpnFfnProgramV1's two native steps
 * (crates/augur-backend/src/cuda_qwen35_prefill_cublas/qpn.rs:391-394,465-492;
 * native augur_qwen35_qpn_prefill.cuh:97-147): both members and every cross alias
 * are validated before the first enqueue; down.input must be gate_up.output. */
typedef struct augur_cuda_nvfp4_sm100_mlp_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_nvfp4_sm100_gemv_args_v1 gate_up;
    augur_cuda_nvfp4_sm100_gemv_args_v1 down;
} augur_cuda_nvfp4_sm100_mlp_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_args_v1* args);

/* The MLP block on the tensor-memory path as ONE launch: gate|up with SiLU(gate) * up (the interleaved
 * TCGEN05 weight), then down (TCGEN05), with the intermediate handed on inside the launch and the weight
 * stream of the down projection already running while the intermediate is completed. Same descriptor and
 * the same cross-member checks as mlp_*_v1 (both members validated before the one enqueue); replaces
 * CudaQwen35QpnFfnProgramV1 (crates/augur-backend/src/cuda_qwen35_prefill_cublas/qpn.rs:391-492) for
 * 1..8 token rows. The plan needs gemv_tc_scratch_extent of each member, side by side. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tc_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tc_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_args_v1* args);

/* How a tensor-memory launch is laid out on a device with `sm_count` SMs: a host-side computation (no device
 * access, no allocation) for diagnostics and for tests of the split. A launch is a list of steps; a step is a set
 * of items (tile, part) dealt round-robin over the CTAs (item i goes to CTA i mod ctas): tiles [tile0, tile0 + tiles)
 * of 128 physical weight rows of product `phase`, each over the 256-deep k blocks [kb0, kb1) cut into `parts` equal
 * ranges (part p: [kb0 + p * (kb1 - kb0) / parts, kb0 + (p + 1) * (kb1 - kb0) / parts)); the partial sums of a tile
 * meet in contributor slots slot0 + part of `contributors[phase]`. Its activations are job `job`: the 16-element
 * groups [group0, group0 + groups) of every token row of the input of product `phase`, split inside the launch;
 * `feeds` names the job that this step's outputs become (0: none), `keeps` says that every CTA has at most one item
 * of the step and splits its own outputs from registers. `rows_b` = 0 describes a linear (`epilogue_a` as in the
 * gemv arguments, `rows_a` logical rows), otherwise the MLP block `rows_a` = intermediate, `cols_a` = hidden,
 * `rows_b` = hidden, `cols_b` = intermediate. */
typedef struct augur_cuda_nvfp4_sm100_tc_step_v1 {
    uint32_t phase, job, tile0, tiles, kb0, kb1, parts, slot0, feeds, keeps;
} augur_cuda_nvfp4_sm100_tc_step_v1;
typedef struct augur_cuda_nvfp4_sm100_tc_job_v1 {
    uint32_t phase, group0, groups;
} augur_cuda_nvfp4_sm100_tc_job_v1;
typedef struct augur_cuda_nvfp4_sm100_tc_program_v1 {
    uint32_t steps, jobs, ctas;
    uint32_t contributors[2];
    augur_cuda_nvfp4_sm100_tc_step_v1 step[4];
    augur_cuda_nvfp4_sm100_tc_job_v1 job[3];
} augur_cuda_nvfp4_sm100_tc_program_v1;
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_tc_program_describe_host_v1(
    uint32_t rows_a, uint32_t cols_a, uint32_t epilogue_a, uint32_t rows_b, uint32_t cols_b, uint32_t sm_count,
    augur_cuda_nvfp4_sm100_tc_program_v1* out);

/* ---- norm group: [residual add] -> RMSNorm -> BF16 stage -> 1..4 small-token projections ----- */
/* Replaces augur_cuda_qwen35_qpn_norm_group_b8_{preflight,prevalidated_submit}_v1
 * (native augur_qwen35_gdn_input_b8.cuh:19-49,50-110): GDN input (norm, then the in-projections)
 * and post-attention (residual add, norm, then gate|up or separate projections) as one validated
 * program. The norm stage keeps the reference kernel's arithmetic order (per-lane serial sums over
 * columns l, l+256, ..., halving-stride fold, y = value * scale * weight left to right), with
 * scale = 1 / sqrt(mean + epsilon) correctly rounded (the reference uses the approximate rsqrtf)
 * and a BF16 staged copy instead of FP16. With `residual` the value add_a + add_b is stored to
 * input_f32 first. Every projection must take staged_bf16 as its input (same tokens and cols);
 * unused members are zero. tokens 1..8, cols a multiple of 256. Two launches, as in the reference: the
 * norm stage, which also writes the activations in the form the projections' MMAs consume (so that no
 * member stages them again), and ONE grid for all members, the SMs dealt out in proportion to the members'
 * rows. A member may store trimmed (stored_rows), e.g. 48 of 64 padded rows. */
typedef struct augur_cuda_nvfp4_sm100_norm_group_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t add_a;         /* residual only, else 0: [tokens][cols] f32 */
    augur_cuda_device_ptr_t add_b;
    uint64_t add_len_bytes;
    augur_cuda_device_ptr_t input_f32;     /* [tokens][cols]; read, or written when residual */
    uint64_t input_len_bytes;
    augur_cuda_device_ptr_t weight_f32;    /* [cols] */
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t output_f32;    /* [tokens][cols] normalised */
    uint64_t output_len_bytes;
    augur_cuda_device_ptr_t staged_bf16;   /* [tokens][cols] = bf16(output): the projections' input */
    uint64_t staged_len_bytes;
    uint32_t tokens;
    uint32_t cols;
    float epsilon;
    uint32_t residual;
    uint32_t count;
    uint32_t reserved;
    augur_cuda_nvfp4_sm100_gemv_args_v1 projections[4];
} augur_cuda_nvfp4_sm100_norm_group_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_norm_group_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_norm_group_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_norm_group_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_norm_group_args_v1* args);

/* ---- BF16 vocabulary head for 1..8 token rows ------------------------------------ */
/* Replaces augur_cuda_dflash_bf16_head_f32_rw4_{preflight,submit}_v1 (augur_cuda_runtime.h:2499-2502, struct
 * augur_cuda_bf16_f32_matvec_args_v1 at :1689-1700, kernel native/augur_dflash_llama_bf16_head.cuh:24-72): the
 * shared 248320 x 5120 BF16 head of the draft and the verifier, read in place. Same members as the reference
 * struct; weights [rows][cols] BF16, activations [tokens][cols] F32 (tokens = input_len_bytes / (4 cols),
 * 1..8), logits [tokens][rows] F32; 16-byte aligned weights and activations as the rw4 entry asks; rows a
 * multiple of 16, cols a multiple of 64 (any such shape, not only the one vocabulary). Products are exact
 * (BF16 x BF16 terms of the exactly split F32 activation on the tensor cores), accumulation is F32. */
typedef struct augur_cuda_nvfp4_sm100_bf16_head_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t weight;
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t input;
    uint64_t input_len_bytes;
    augur_cuda_device_ptr_t output;
    uint64_t output_len_bytes;
    uint32_t rows;
    uint32_t cols;
} augur_cuda_nvfp4_sm100_bf16_head_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_bf16_head_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_bf16_head_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_bf16_head_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_bf16_head_args_v1* args);

/* ---- tensor-parallel MLP program: the all-reduce inside the down launch --------- */
/* No counterpart in the reference (it has no multi-GPU code). Column-parallel gate|up and
 * row-parallel down over up to 8 GPUs of one box, one process per GPU: every rank passes its
 * own shard in `gate_up` / `down` exactly as for mlp_*_v1, plus the exchange buffers of all
 * ranks as they are mapped into this process (peer-accessible device memory of
 * exchange_len_bytes each, zero-filled once before the first submit; exchange[rank] is this
 * rank's own). The warp that completes a 32-row group of the down projection stores its f32
 * tile, each value paired with `sequence` as its flag, into every other rank's buffer over
 * NVLink, waits (bounded) for the same group of every other rank in its own buffer and writes
 * bf16(sum over ranks, in rank order) to down.output: all ranks end up with the same
 * full-width [tokens][rows] result and no collective is launched. `sequence` = 0 lets the
 * launches count their own sequence in the last 256 bytes of this rank's exchange buffer
 * (zero-filled with the rest): nothing that changes from submit to submit is then part of the
 * launch parameters, so a program captured into a CUDA graph can be replayed, which is how the
 * reference's serving loop drives its programs
 * (crates/augur-backend/src/cuda_qwen35_prefill_cublas/qpn.rs:507-515). A non-zero `sequence`
 * is counted by the caller instead: it starts at 1 and grows by exactly 1 with every submit
 * that uses these buffers, in step on all ranks (1, ..., 0xFFFFFFFE, 1, ...); the two ways of
 * counting are not mixed on one set of buffers. All ranks' kernels must be able to run at the
 * same time (one process and one GPU per rank). A wait that runs out sets the plan's status
 * word to 0x203.
 * Peer buffers cannot be inspected from this process: preflight checks them for alignment,
 * size and overlap only. */
#define AUGUR_NVFP4_SM100_MAX_TP_RANKS 8
typedef struct augur_cuda_nvfp4_sm100_mlp_tp_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_nvfp4_sm100_gemv_args_v1 gate_up;
    augur_cuda_nvfp4_sm100_gemv_args_v1 down;
    augur_cuda_device_ptr_t exchange[AUGUR_NVFP4_SM100_MAX_TP_RANKS];  /* entries >= world are 0 */
    uint64_t exchange_len_bytes;
    uint32_t world;
    uint32_t rank;
    uint32_t sequence;
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_mlp_tp_args_v1;

/* Bytes of one rank's exchange buffer for a down projection with `rows` output rows. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tp_exchange_extent_host_v1(
    uint32_t rows, uint32_t world, uint64_t* out_bytes);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tp_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_tp_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_mlp_tp_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_mlp_tp_args_v1* args);

/* A single row-parallel small-token linear with the same exchange: every rank holds a k-slice of the
 * weight (`linear`, epilogue LINEAR_BF16) and its matching slice of the activations, and every rank
 * ends up with bf16(sum over ranks) in linear.output. For the projections outside the MLP block
 * (attention / GDN output projections). No counterpart in the reference. */
typedef struct augur_cuda_nvfp4_sm100_gemv_tp_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_nvfp4_sm100_gemv_args_v1 linear;
    augur_cuda_device_ptr_t exchange[AUGUR_NVFP4_SM100_MAX_TP_RANKS];  /* entries >= world are 0 */
    uint64_t exchange_len_bytes;
    uint32_t world;
    uint32_t rank;
    uint32_t sequence;                    /* as in mlp_tp_args_v1 */
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_gemv_tp_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tp_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_tp_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemv_tp_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemv_tp_args_v1* args);

/* ---- prefill: activation quantiser + tcgen05 block-scaled GEMM --------------- */
/* Replaces the W4A4 interstage quantiser (augur_cuda_runtime.h:6983 ff.;
 * native augur_nvfp4_cutlass_sm120.cu:455-503): BF16 rows -> E2M1 codes with one
 * E4M3 scale per 16 (smallest scale >= amax/(6*global); nearest level, ties to
 * the smaller magnitude). `terms` > 1 writes a residual series. */
typedef struct augur_cuda_nvfp4_sm100_act_quant_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t input_bf16;   /* [tokens][cols] */
    uint64_t input_len_bytes;
    augur_cuda_device_ptr_t destination;  /* [terms] x TCGEN05 layout of a ceil128(tokens) x cols tensor */
    uint64_t destination_len_bytes;
    uint32_t tokens;
    uint32_t cols;
    uint32_t terms;                       /* 1..3 */
    float global_scale;
} augur_cuda_nvfp4_sm100_act_quant_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_act_quant_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_act_quant_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, const augur_cuda_nvfp4_sm100_act_quant_args_v1* args);

/* Replaces the CUTLASS W4A4 shape launches and the W4A16 kernel
 * (augur_cuda_runtime.h:6930-6964,7631-7643; native augur_nvfp4_cutlass_sm120.cu:36-203,320-378)
 * and the wide prefill projection (augur_qwen35_qpn_prefill.cuh:53-88):
 * y[t][n] = bf16(g_w * g_a * sum_terms sum_k w[n][k] a_term[t][k]) on tcgen05
 * kind::mxf4nvf4 with TMEM accumulators. Any token count >= 1: the staged activations hold whole
 * 128-row tiles per term (gemm_scratch_extent_host_v1 gives the size act_quant writes and the GEMM
 * reads), rows past `tokens` are computed and never stored; input and output have exactly
 * `tokens` rows. */
typedef struct augur_cuda_nvfp4_sm100_gemm_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t weight;        /* TCGEN05 layout, rows x cols */
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t activation;    /* output of act_quant */
    uint64_t activation_len_bytes;
    augur_cuda_device_ptr_t output_bf16;   /* [tokens][rows] */
    uint64_t output_len_bytes;
    uint32_t rows;
    uint32_t cols;
    uint32_t tokens;
    uint32_t activation_terms;
    float weight_global_scale;
    float activation_global_scale;
} augur_cuda_nvfp4_sm100_gemm_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_args_v1* args);

/* The gate|up projection of an MLP at prefill with SiLU(gate) * up in the GEMM epilogue; the
 * counterpart of the reference's interstage step (native augur_nvfp4_cutlass_sm120.cu:455-503 computes
 * silu(gate) * up from two GEMM outputs in a separate pass; augur_qwen35_qpn_prefill.cuh:120-147 fuses
 * it with the staging of the down projection's input). `weight` is the TCGEN05 layout of ONE matrix of
 * 2 * rows physical rows in which 16 gate rows alternate with the matching 16 up rows
 * (interleave_gate_up_host_v1 builds its compact planes), so that 32 consecutive accumulator columns
 * of a token hold the gate and up sums of 16 intermediate columns:
 * out[t][n] = bf16(silu(g_gate * g_a * sum gate) * (g_up * g_a * sum up)), rows = intermediate size
 * (a multiple of 64). Nothing of the 2 * rows wide gate|up tensor is ever written to memory. */
typedef struct augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t weight;        /* TCGEN05 layout, (2 * rows) x cols, gate/up interleaved by 16 rows */
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t activation;    /* output of act_quant */
    uint64_t activation_len_bytes;
    augur_cuda_device_ptr_t output_bf16;   /* [tokens][rows] */
    uint64_t output_len_bytes;
    uint32_t rows;
    uint32_t cols;
    uint32_t tokens;
    uint32_t activation_terms;
    float gate_global_scale;
    float up_global_scale;
    float activation_global_scale;
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1* args);
/* The same fused gate|up projection, with its result also - or only - quantised for the down
 * projection inside the epilogue (the reference's interstage step produces the quantised tensor
 * directly from the two GEMM outputs, augur_nvfp4_cutlass_sm120.cu:455-503): `destination` receives
 * exactly what act_quant would write for the BF16 intermediate (same rule, same layout,
 * `destination_terms` residual terms, `destination_global_scale`), while the next tile's MMAs run.
 * `output_bf16` may be 0 (with output_len_bytes 0): the BF16 intermediate is then never written.
 * Runs on the two-CTA tiles only: rows must be a multiple of 128 (any token count); other shapes get
 * INVALID_ARGUMENT and use gemm_swiglu_bf16 followed by act_quant. */
typedef struct augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1 {
    uint32_t abi_version;
    uint32_t struct_size;
    augur_cuda_device_ptr_t weight;        /* TCGEN05 layout, (2 * rows) x cols, gate/up interleaved by 16 rows */
    uint64_t weight_len_bytes;
    augur_cuda_device_ptr_t activation;    /* output of act_quant */
    uint64_t activation_len_bytes;
    augur_cuda_device_ptr_t output_bf16;   /* [tokens][rows], or 0 */
    uint64_t output_len_bytes;
    augur_cuda_device_ptr_t destination;   /* [destination_terms] x TCGEN05 layout of a ceil128(tokens) x rows tensor */
    uint64_t destination_len_bytes;
    uint32_t rows;
    uint32_t cols;
    uint32_t tokens;
    uint32_t activation_terms;
    float gate_global_scale;
    float up_global_scale;
    float activation_global_scale;
    float destination_global_scale;
    uint32_t destination_terms;
    uint32_t reserved;
} augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1;

augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_quant_preflight_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1* args);
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_gemm_swiglu_quant_prevalidated_submit_v1(
    int32_t ordinal, augur_cuda_stream_t stream, augur_cuda_nvfp4_sm100_plan_v1* plan,
    const augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1* args);
/* Compact planes of the interleaved gate|up matrix: physical row 32 j + i is gate row 16 j + i for
 * i < 16 and up row 16 j + i - 16 otherwise. rows % 16 == 0, cols % 16 == 0; outputs hold 2 * rows rows. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_interleave_gate_up_host_v1(
    uint32_t rows, uint32_t cols, const uint8_t* gate_codes, const uint8_t* gate_scales,
    const uint8_t* up_codes, const uint8_t* up_scales, uint8_t* out_codes, uint8_t* out_scales);

/* ---- diagnostics ------------------------------------------------------------ */
/* Host-side fault injection (the reference injects with a device trap,
 * native augur_m306_k14_async_fault_sm70.cu:7-9,61; here nothing touches the GPU):
 * the next `count` submits return AUGUR_CUDA_STATUS_DIAGNOSTIC_FAULT_INJECTED
 * before any enqueue. */
void AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_diagnostic_inject_submit_fault_v1(uint32_t count);
/* Device allocations / frees made by this library so far; the counterpart of
 * cuda_device_allocation_snapshot (crates/augur-backend/src/cuda_runtime.rs:528-535),
 * used to prove the hot path allocates nothing. */
void AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_allocation_snapshot_v1(
    uint64_t* out_allocations, uint64_t* out_frees);
/* Kernel launches enqueued by this library so far. */
uint64_t AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_launch_count_v1(void);
/* Device-side status word of the plan (0 = clean). Bounded waits inside the
 * kernels record where they gave up here instead of spinning for ever; reading
 * it synchronises the plan's stream. */
augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_device_status_v1(
    augur_cuda_nvfp4_sm100_plan_v1* plan, uint32_t* out_status);

#ifdef __cplusplus
}
#endif
#endif
