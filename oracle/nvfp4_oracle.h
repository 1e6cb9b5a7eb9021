/* CPU oracle for the NVFP4 quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * CPU arithmetic for the NVFP4 linear (Augur crates augur-formats,
 * augur-repack, augur-kernels, augur-reference). It exists so that the CUDA
 * path can be checked against it; nothing in the shipped library links,
 * imports or calls it. Parity status: PINNED against the known-answer
 * vectors held by the reference's own unit tests (see tests/test_oracle_kat.py).
 *
 * Build: gcc -O2 -ffp-contract=off (no FMA contraction: Rust never contracts
 * a*b+c, so neither may this file).
 */
#ifndef AUGUR_NVFP4_ORACLE_H
#define AUGUR_NVFP4_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors Nvfp4CompactBlock (crates/augur-formats/src/fp4.rs:91-96). */
typedef struct augur_oracle_nvfp4_compact_block {
    uint8_t qs[8];
    uint8_t scale_e4m3;
    uint8_t pad[3];
    float global_scale;
} augur_oracle_nvfp4_compact_block;

/* Mirrors Nvfp4HotCpuBlock (crates/augur-kernel-api/src/hot/fp4_portable.rs:15-19). */
typedef struct augur_oracle_nvfp4_hot_block {
    float scale;
    uint8_t qs[8];
} augur_oracle_nvfp4_hot_block;

/* Error vocabulary: FormatError / ReferenceQ8Error / KernelError collapsed to ints. */
enum {
    AUGUR_ORACLE_OK = 0,
    AUGUR_ORACLE_NON_FINITE_VALUE = 1,     /* FormatError::NonFiniteValue */
    AUGUR_ORACLE_OUTPUT_TOO_SMALL = 2,     /* FormatError::OutputTooSmall */
    AUGUR_ORACLE_BAD_WEIGHT_SHAPE = 3,     /* ReferenceQ8Error::BadWeightShape */
    AUGUR_ORACLE_BAD_ACTIVATION_LENGTH = 4,
    AUGUR_ORACLE_BAD_OUTPUT_LENGTH = 5,
    AUGUR_ORACLE_BAD_WEIGHT_BLOCK_COUNT = 6,
    AUGUR_ORACLE_BAD_WEIGHT = 7
};

float augur_oracle_decode_e2m1(uint8_t value);
int augur_oracle_decode_e4m3fn(uint8_t value, float* out);
float augur_oracle_bf16_round(float value);
uint16_t augur_oracle_f32_to_bf16_bits(float value);
float augur_oracle_bf16_bits_to_f32(uint16_t bits);

int augur_oracle_nvfp4_block_decode_ref(const augur_oracle_nvfp4_compact_block* block,
                                        float* destination, size_t destination_len);

int augur_oracle_qmatvec_nvfp4_f32_ref(const augur_oracle_nvfp4_compact_block* blocks,
                                       size_t block_count, size_t rows, size_t cols,
                                       const float* activation, size_t activation_len,
                                       float* output, size_t output_len);

int augur_oracle_repack_nvfp4_block_cpu(const augur_oracle_nvfp4_compact_block* source,
                                        augur_oracle_nvfp4_hot_block* out);
int augur_oracle_repack_nvfp4_tensor_cpu(const augur_oracle_nvfp4_compact_block* source,
                                         size_t block_count, size_t rows, size_t cols,
                                         augur_oracle_nvfp4_hot_block* out);
int augur_oracle_qmatvec_nvfp4_f32_cpu_portable(const augur_oracle_nvfp4_hot_block* blocks,
                                                size_t block_count, size_t rows, size_t cols,
                                                const float* activation, size_t activation_len,
                                                float* output, size_t output_len);

/* Plane form (codes [rows][cols/2], scales [rows][cols/16], one global): the
 * layout a checkpoint loader hands over (checkpoint_quant.rs:95-152). */
int augur_oracle_planes_to_blocks(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                  size_t rows, size_t cols,
                                  augur_oracle_nvfp4_compact_block* out);
int augur_oracle_dequant_planes_f32(const uint8_t* codes, const uint8_t* scales,
                                    float global_scale, size_t rows, size_t cols, float* out);

/* y[m][n] = bf16_round( f32 sequential sum_k w[n][k] * widen(x[m][k]) ).
 * threads > 1 splits weight rows across threads; per-row order is unchanged,
 * so the result is bit-identical to threads == 1. */
int augur_oracle_linear_bf16(const uint8_t* codes, const uint8_t* scales, float global_scale,
                             size_t rows, size_t cols, const uint16_t* x_bf16, size_t tokens,
                             uint16_t* y_bf16, float* y_f32_or_null, int threads);

/* fp64 oracle: y64[m][n] = sum_k double(w_f32[n][k]) * double(x[m][k]). */
int augur_oracle_linear_f64(const uint8_t* codes, const uint8_t* scales, float global_scale,
                            size_t rows, size_t cols, const uint16_t* x_bf16, size_t tokens,
                            double* y64, int threads);

/* Same, but activations already given as doubles (used for the block-scaled
 * GEMM, whose activations are quantised first). */
int augur_oracle_linear_f64_xf64(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                 size_t rows, size_t cols, const double* x, size_t tokens,
                                 double* y64, int threads);

/* SwiGLU MLP: h = bf16_round(silu(g)*u) with g,u the f32 sums; y = linear_bf16(down, h). */
int augur_oracle_mlp_bf16(const uint8_t* gate_codes, const uint8_t* gate_scales, float gate_global,
                          const uint8_t* up_codes, const uint8_t* up_scales, float up_global,
                          const uint8_t* down_codes, const uint8_t* down_scales, float down_global,
                          size_t hidden, size_t intermediate, const uint16_t* x_bf16, size_t tokens,
                          uint16_t* h_bf16, uint16_t* y_bf16, int threads);
int augur_oracle_mlp_f64(const uint8_t* gate_codes, const uint8_t* gate_scales, float gate_global,
                         const uint8_t* up_codes, const uint8_t* up_scales, float up_global,
                         const uint8_t* down_codes, const uint8_t* down_scales, float down_global,
                         size_t hidden, size_t intermediate, const uint16_t* x_bf16, size_t tokens,
                         double* h64, double* y64, int threads);

/* Activation quantiser (BF16 -> NVFP4 residual terms), the CPU statement of
 * the rule the CUDA quantiser implements. See nvfp4_oracle.c. */
int augur_oracle_act_quant(const uint16_t* x_bf16, size_t tokens, size_t cols, float global_scale,
                           int terms, uint8_t* codes, uint8_t* scales);
int augur_oracle_act_dequant_f64(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                 size_t tokens, size_t cols, int terms, double* out);

/* [residual add] -> RMSNorm -> F32 output + BF16 staged copy; see nvfp4_oracle.c. cols % 256 == 0. */
int augur_oracle_rmsnorm_stage(const float* add_a, const float* add_b, float* input, const float* weight,
                               size_t tokens, size_t cols, float epsilon, int residual,
                               float* output_f32, uint16_t* staged_bf16);

int augur_oracle_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
