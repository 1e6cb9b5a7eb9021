/* CPU oracle for the NVFP4 quantized-linear path. TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU arithmetic; every function
 * cites the reference file:line it follows (paths inside the Augur project).
 * Parity status: PINNED — tests/test_oracle_kat.py checks it against the
 * known-answer vectors of the reference's own unit tests.
 *
 * Must be built with -ffp-contract=off: the reference (Rust) never fuses
 * a*b+c, and bit-exactness of the f32 path depends on that.
 */
#include "nvfp4_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

/* crates/augur-formats/src/fp4.rs:7-9 — note code 8 is +0.0, not -0.0. */
static const float E2M1_VALUES[16] = {
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f,
};

/* crates/augur-formats/src/fp4.rs:34-37 */
float augur_oracle_decode_e2m1(uint8_t value) { return E2M1_VALUES[value & 0x0f]; }

/* crates/augur-formats/src/fp4.rs:46-59 — signed E4M3FN; 0x7f/0xff are NaN. */
int augur_oracle_decode_e4m3fn(uint8_t value, float* out) {
    const float sign = (value & 0x80) == 0 ? 1.0f : -1.0f;
    const int exponent = (value >> 3) & 0x0f;
    const int mantissa = value & 0x07;
    if (exponent == 0x0f && mantissa == 0x07) {
        return AUGUR_ORACLE_NON_FINITE_VALUE;
    }
    float magnitude;
    if (exponent == 0) {
        magnitude = ldexpf(1.0f, -6) * ((float)mantissa / 8.0f);
    } else {
        magnitude = ldexpf(1.0f, exponent - 7) * (1.0f + (float)mantissa / 8.0f);
    }
    *out = sign * magnitude;
    return AUGUR_ORACLE_OK;
}

/* crates/augur-model-qwen35/src/reference.rs:819-826 — f32 -> BF16, RNE. */
float augur_oracle_bf16_round(float value) {
    if (!isfinite(value)) {
        return value;
    }
    uint32_t bits;
    memcpy(&bits, &value, 4);
    bits = (bits + (0x7fffu + ((bits >> 16) & 1u))) & 0xffff0000u;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

uint16_t augur_oracle_f32_to_bf16_bits(float value) {
    uint32_t bits;
    if (isnan(value)) {
        memcpy(&bits, &value, 4);
        return (uint16_t)((bits >> 16) | 0x0040u);
    }
    const float rounded = augur_oracle_bf16_round(value);
    memcpy(&bits, &rounded, 4);
    return (uint16_t)(bits >> 16);
}

float augur_oracle_bf16_bits_to_f32(uint16_t bits) {
    const uint32_t wide = (uint32_t)bits << 16;
    float out;
    memcpy(&out, &wide, 4);
    return out;
}

/* crates/augur-formats/src/fp4.rs:105-125 — two roundings: scale = fl(e4m3*global),
 * value = fl(e2m1*scale); element i sits in byte i/2, low nibble for even i. */
int augur_oracle_nvfp4_block_decode_ref(const augur_oracle_nvfp4_compact_block* block,
                                        float* destination, size_t destination_len) {
    if (destination_len < 16) {
        return AUGUR_ORACLE_OUTPUT_TOO_SMALL;
    }
    if (!isfinite(block->global_scale)) {
        return AUGUR_ORACLE_NON_FINITE_VALUE;
    }
    float e4m3;
    const int status = augur_oracle_decode_e4m3fn(block->scale_e4m3, &e4m3);
    if (status != AUGUR_ORACLE_OK) {
        return status;
    }
    const float scale = e4m3 * block->global_scale;
    if (!isfinite(scale)) {
        return AUGUR_ORACLE_NON_FINITE_VALUE;
    }
    for (size_t index = 0; index < 16; ++index) {
        const uint8_t byte = block->qs[index / 2];
        const uint8_t nibble = (index % 2 == 0) ? byte : (uint8_t)(byte >> 4);
        destination[index] = augur_oracle_decode_e2m1(nibble) * scale;
    }
    return AUGUR_ORACLE_OK;
}

/* crates/augur-reference/src/m46_fp4.rs:128-177 — validation order and the
 * strictly sequential f32 sum over k. */
int augur_oracle_qmatvec_nvfp4_f32_ref(const augur_oracle_nvfp4_compact_block* blocks,
                                       size_t block_count, size_t rows, size_t cols,
                                       const float* activation, size_t activation_len,
                                       float* output, size_t output_len) {
    const size_t block_len = 16;
    if (rows == 0 || cols == 0 || cols % block_len != 0) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    if (activation_len != cols) {
        return AUGUR_ORACLE_BAD_ACTIVATION_LENGTH;
    }
    if (output_len < rows) {
        return AUGUR_ORACLE_BAD_OUTPUT_LENGTH;
    }
    const size_t blocks_per_row = cols / block_len;
    if (blocks_per_row != 0 && rows > SIZE_MAX / blocks_per_row) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    if (block_count != rows * blocks_per_row) {
        return AUGUR_ORACLE_BAD_WEIGHT_BLOCK_COUNT;
    }
    float decoded[16];
    for (size_t row = 0; row < rows; ++row) {
        float sum = 0.0f;
        for (size_t block_index = 0; block_index < blocks_per_row; ++block_index) {
            if (augur_oracle_nvfp4_block_decode_ref(&blocks[row * blocks_per_row + block_index],
                                                    decoded, 16) != AUGUR_ORACLE_OK) {
                return AUGUR_ORACLE_BAD_WEIGHT;
            }
            const size_t start = block_index * block_len;
            for (size_t lane = 0; lane < block_len; ++lane) {
                sum += decoded[lane] * activation[start + lane];
            }
        }
        output[row] = sum;
    }
    return AUGUR_ORACLE_OK;
}

/* crates/augur-repack/src/fp4_cpu.rs:19-31 */
int augur_oracle_repack_nvfp4_block_cpu(const augur_oracle_nvfp4_compact_block* source,
                                        augur_oracle_nvfp4_hot_block* out) {
    if (!isfinite(source->global_scale)) {
        return AUGUR_ORACLE_NON_FINITE_VALUE;
    }
    float e4m3;
    const int status = augur_oracle_decode_e4m3fn(source->scale_e4m3, &e4m3);
    if (status != AUGUR_ORACLE_OK) {
        return status;
    }
    const float scale = e4m3 * source->global_scale;
    if (!isfinite(scale)) {
        return AUGUR_ORACLE_NON_FINITE_VALUE;
    }
    out->scale = scale;
    memcpy(out->qs, source->qs, 8);
    return AUGUR_ORACLE_OK;
}

/* crates/augur-repack/src/fp4_cpu.rs:45-55 plus the shape contract of
 * crates/augur-kernel-api/src/hot/fp4_portable.rs:27-87. */
int augur_oracle_repack_nvfp4_tensor_cpu(const augur_oracle_nvfp4_compact_block* source,
                                         size_t block_count, size_t rows, size_t cols,
                                         augur_oracle_nvfp4_hot_block* out) {
    for (size_t index = 0; index < block_count; ++index) {
        const int status = augur_oracle_repack_nvfp4_block_cpu(&source[index], &out[index]);
        if (status != AUGUR_ORACLE_OK) {
            return status;
        }
    }
    if (rows == 0 || cols == 0 || cols % 16 != 0) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    if (block_count != rows * (cols / 16)) {
        return AUGUR_ORACLE_BAD_WEIGHT_BLOCK_COUNT;
    }
    return AUGUR_ORACLE_OK;
}

/* crates/augur-kernels/src/portable/m46_fp4.rs:18-56 — sum += e2m1*scale*act,
 * left-associated, which yields the same bits as the reference oracle. */
int augur_oracle_qmatvec_nvfp4_f32_cpu_portable(const augur_oracle_nvfp4_hot_block* blocks,
                                                size_t block_count, size_t rows, size_t cols,
                                                const float* activation, size_t activation_len,
                                                float* output, size_t output_len) {
    if (rows == 0 || cols == 0 || cols % 16 != 0 || block_count != rows * (cols / 16)) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    if (activation_len != cols) {
        return AUGUR_ORACLE_BAD_ACTIVATION_LENGTH;
    }
    if (output_len < rows) {
        return AUGUR_ORACLE_BAD_OUTPUT_LENGTH;
    }
    const size_t blocks_per_row = cols / 16;
    for (size_t row = 0; row < rows; ++row) {
        float sum = 0.0f;
        for (size_t block_index = 0; block_index < blocks_per_row; ++block_index) {
            const augur_oracle_nvfp4_hot_block* block = &blocks[row * blocks_per_row + block_index];
            const size_t start = block_index * 16;
            for (size_t lane = 0; lane < 16; ++lane) {
                const uint8_t byte = block->qs[lane / 2];
                const uint8_t nibble = (lane % 2 == 0) ? byte : (uint8_t)(byte >> 4);
                sum += augur_oracle_decode_e2m1(nibble) * block->scale * activation[start + lane];
            }
        }
        output[row] = sum;
    }
    return AUGUR_ORACLE_OK;
}

/* Plane form -> block form. Layout per crates/augur-model-qwen35/src/checkpoint_quant.rs:93-152:
 * codes [rows][cols/2] (low nibble = even k), scales [rows][cols/16]. */
int augur_oracle_planes_to_blocks(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                  size_t rows, size_t cols,
                                  augur_oracle_nvfp4_compact_block* out) {
    if (rows == 0 || cols == 0 || cols % 16 != 0) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    const size_t count = rows * (cols / 16);
    for (size_t index = 0; index < count; ++index) {
        memcpy(out[index].qs, codes + index * 8, 8);
        out[index].scale_e4m3 = scales[index];
        memset(out[index].pad, 0, sizeof out[index].pad);
        out[index].global_scale = global_scale;
    }
    return AUGUR_ORACLE_OK;
}

static int decode_row_f32(const uint8_t* codes, const uint8_t* scales, float global_scale,
                          size_t cols, float* out) {
    augur_oracle_nvfp4_compact_block block;
    memset(&block, 0, sizeof block);
    block.global_scale = global_scale;
    for (size_t group = 0; group < cols / 16; ++group) {
        memcpy(block.qs, codes + group * 8, 8);
        block.scale_e4m3 = scales[group];
        const int status = augur_oracle_nvfp4_block_decode_ref(&block, out + group * 16, 16);
        if (status != AUGUR_ORACLE_OK) {
            return status;
        }
    }
    return AUGUR_ORACLE_OK;
}

int augur_oracle_dequant_planes_f32(const uint8_t* codes, const uint8_t* scales,
                                    float global_scale, size_t rows, size_t cols, float* out) {
    if (rows == 0 || cols == 0 || cols % 16 != 0) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    for (size_t row = 0; row < rows; ++row) {
        const int status = decode_row_f32(codes + row * (cols / 2), scales + row * (cols / 16),
                                          global_scale, cols, out + row * cols);
        if (status != AUGUR_ORACLE_OK) {
            return AUGUR_ORACLE_BAD_WEIGHT;
        }
    }
    return AUGUR_ORACLE_OK;
}

/* [residual add] -> RMSNorm -> F32 output and its BF16 rounding: the CPU statement of the
 * reference's norm stage (crates/augur-cuda-sys/native/augur_qwen35_gdn_input_b8.cuh:19-49, which
 * keeps prefill_rmsnorm_kernel's order, augur_qwen35_prefill_cublas_sm70.cu:1008-1029): 256 lanes
 * per token row, lane l adds value*value over columns l, l+256, ... in that order (a multiply and
 * an add, no fused operation), the 256 partial sums are folded by halving strides
 * (partial[l] += partial[l + stride], stride 128 .. 1), y = value * scale * weight[col] evaluated
 * left to right. Two deliberate differences: scale = 1 / sqrt(mean + epsilon) with correctly
 * rounded division and square root (the reference's rsqrtf is a hardware approximation that no
 * CPU code can restate bit for bit), and the staged copy is BF16 (bf16_round), not FP16, because
 * the B200 kernels take BF16 activations. With `residual` the value is add_a + add_b and is stored
 * to `input` first (one F32 add per element, as the reference does). */
int augur_oracle_rmsnorm_stage(const float* add_a, const float* add_b, float* input, const float* weight,
                               size_t tokens, size_t cols, float epsilon, int residual,
                               float* output_f32, uint16_t* staged_bf16) {
    if (!input || !weight || !output_f32 || !staged_bf16 || tokens == 0 || cols == 0 || cols % 256 != 0) return -1;
    if (residual && (!add_a || !add_b)) return -1;
    for (size_t token = 0; token < tokens; ++token) {
        const size_t base = token * cols;
        float partial[256];
        for (size_t lane = 0; lane < 256; ++lane) {
            float sum = 0.0f;
            for (size_t col = lane; col < cols; col += 256) {
                float value;
                if (residual) {
                    value = add_a[base + col] + add_b[base + col];
                    input[base + col] = value;
                } else {
                    value = input[base + col];
                }
                const float square = value * value;
                sum = sum + square;
            }
            partial[lane] = sum;
        }
        for (size_t stride = 128; stride != 0; stride >>= 1) {
            for (size_t lane = 0; lane < stride; ++lane) partial[lane] = partial[lane] + partial[lane + stride];
        }
        const float mean = partial[0] / (float)cols;
        const float scale = 1.0f / sqrtf(mean + epsilon);
        for (size_t col = 0; col < cols; ++col) {
            const float scaled = input[base + col] * scale;
            const float y = scaled * weight[col];
            output_f32[base + col] = y;
            const float rounded = augur_oracle_bf16_round(y);
            uint32_t bits;
            memcpy(&bits, &rounded, 4);
            staged_bf16[base + col] = (uint16_t)(bits >> 16);
        }
    }
    return 0;
}

int augur_oracle_max_threads(void) {
    const long count = sysconf(_SC_NPROCESSORS_ONLN);
    return count < 1 ? 1 : (int)count;
}

/* Row-parallel driver: rows [0, rows) are cut into `threads` contiguous
 * ranges, one pthread each. Every row is computed by exactly one thread with
 * the serial per-row code, so the output does not depend on `threads`. */
typedef struct row_job {
    const uint8_t* codes;
    const uint8_t* scales;
    float global_scale;
    size_t rows, cols, tokens;
    const float* x_f32;
    const double* x_f64;
    uint16_t* y_bf16;
    float* y_f32;
    double* y_f64;
    size_t row_begin, row_end;
    int failed;
} row_job;

static void* row_worker(void* argument) {
    row_job* job = (row_job*)argument;
    const size_t cols = job->cols;
    float* decoded = (float*)malloc(sizeof(float) * cols);
    if (decoded == NULL) {
        job->failed = 1;
        return NULL;
    }
    for (size_t row = job->row_begin; row < job->row_end; ++row) {
        if (decode_row_f32(job->codes + row * (cols / 2), job->scales + row * (cols / 16),
                           job->global_scale, cols, decoded) != AUGUR_ORACLE_OK) {
            job->failed = 1;
            continue;
        }
        for (size_t token = 0; token < job->tokens; ++token) {
            if (job->x_f32 != NULL) {
                const float* act = job->x_f32 + token * cols;
                float sum = 0.0f;
                for (size_t k = 0; k < cols; ++k) {
                    sum += decoded[k] * act[k];
                }
                if (job->y_f32 != NULL) {
                    job->y_f32[token * job->rows + row] = sum;
                }
                job->y_bf16[token * job->rows + row] = augur_oracle_f32_to_bf16_bits(sum);
            } else {
                const double* act = job->x_f64 + token * cols;
                double sum = 0.0;
                for (size_t k = 0; k < cols; ++k) {
                    sum += (double)decoded[k] * act[k];
                }
                job->y_f64[token * job->rows + row] = sum;
            }
        }
    }
    free(decoded);
    return NULL;
}

static int run_rows(row_job base, int threads) {
    if (threads < 1) {
        threads = 1;
    }
    if ((size_t)threads > base.rows) {
        threads = (int)base.rows;
    }
    row_job* jobs = (row_job*)malloc(sizeof(row_job) * (size_t)threads);
    pthread_t* handles = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    if (jobs == NULL || handles == NULL) {
        free(jobs);
        free(handles);
        return 1;
    }
    int failed = 0;
    for (int index = 0; index < threads; ++index) {
        jobs[index] = base;
        jobs[index].row_begin = base.rows * (size_t)index / (size_t)threads;
        jobs[index].row_end = base.rows * (size_t)(index + 1) / (size_t)threads;
        jobs[index].failed = 0;
        if (index + 1 == threads) {
            row_worker(&jobs[index]);
        } else if (pthread_create(&handles[index], NULL, row_worker, &jobs[index]) != 0) {
            row_worker(&jobs[index]);
            handles[index] = pthread_self();
        }
    }
    for (int index = 0; index + 1 < threads; ++index) {
        if (!pthread_equal(handles[index], pthread_self())) {
            pthread_join(handles[index], NULL);
        }
    }
    for (int index = 0; index < threads; ++index) {
        failed |= jobs[index].failed;
    }
    free(jobs);
    free(handles);
    return failed;
}

/* Per token this is exactly qmatvec_ref above (decode once, then the same
 * sequential f32 sum), followed by bf16_round. Rows are independent, so a
 * row-parallel run is bit-identical to the serial one. */
int augur_oracle_linear_bf16(const uint8_t* codes, const uint8_t* scales, float global_scale,
                             size_t rows, size_t cols, const uint16_t* x_bf16, size_t tokens,
                             uint16_t* y_bf16, float* y_f32_or_null, int threads) {
    if (rows == 0 || cols == 0 || cols % 16 != 0) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    float* x = (float*)malloc(sizeof(float) * tokens * cols);
    if (x == NULL) {
        return AUGUR_ORACLE_BAD_WEIGHT;
    }
    for (size_t index = 0; index < tokens * cols; ++index) {
        x[index] = augur_oracle_bf16_bits_to_f32(x_bf16[index]);
    }
    row_job job;
    memset(&job, 0, sizeof job);
    job.codes = codes;
    job.scales = scales;
    job.global_scale = global_scale;
    job.rows = rows;
    job.cols = cols;
    job.tokens = tokens;
    job.x_f32 = x;
    job.y_bf16 = y_bf16;
    job.y_f32 = y_f32_or_null;
    const int failed = run_rows(job, threads);
    free(x);
    return failed ? AUGUR_ORACLE_BAD_WEIGHT : AUGUR_ORACLE_OK;
}

int augur_oracle_linear_f64_xf64(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                 size_t rows, size_t cols, const double* x, size_t tokens,
                                 double* y64, int threads) {
    if (rows == 0 || cols == 0 || cols % 16 != 0) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    row_job job;
    memset(&job, 0, sizeof job);
    job.codes = codes;
    job.scales = scales;
    job.global_scale = global_scale;
    job.rows = rows;
    job.cols = cols;
    job.tokens = tokens;
    job.x_f64 = x;
    job.y_f64 = y64;
    const int failed = run_rows(job, threads);
    return failed ? AUGUR_ORACLE_BAD_WEIGHT : AUGUR_ORACLE_OK;
}

int augur_oracle_linear_f64(const uint8_t* codes, const uint8_t* scales, float global_scale,
                            size_t rows, size_t cols, const uint16_t* x_bf16, size_t tokens,
                            double* y64, int threads) {
    double* x = (double*)malloc(sizeof(double) * tokens * cols);
    if (x == NULL) {
        return AUGUR_ORACLE_BAD_WEIGHT;
    }
    for (size_t index = 0; index < tokens * cols; ++index) {
        x[index] = (double)augur_oracle_bf16_bits_to_f32(x_bf16[index]);
    }
    const int status = augur_oracle_linear_f64_xf64(codes, scales, global_scale, rows, cols, x,
                                                    tokens, y64, threads);
    free(x);
    return status;
}

/* SiLU(g)*u as the reference's fused MLP states it: gated / (1 + exp(-gated)) * up
 * (crates/augur-reference/src/m46_fp4.rs:117-121), in f32. */
static float silu_mul_f32(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }

int augur_oracle_mlp_bf16(const uint8_t* gate_codes, const uint8_t* gate_scales, float gate_global,
                          const uint8_t* up_codes, const uint8_t* up_scales, float up_global,
                          const uint8_t* down_codes, const uint8_t* down_scales, float down_global,
                          size_t hidden, size_t intermediate, const uint16_t* x_bf16, size_t tokens,
                          uint16_t* h_bf16, uint16_t* y_bf16, int threads) {
    const size_t count = tokens * intermediate;
    float* gate = (float*)malloc(sizeof(float) * count);
    float* up = (float*)malloc(sizeof(float) * count);
    uint16_t* scratch = (uint16_t*)malloc(sizeof(uint16_t) * count);
    int status = AUGUR_ORACLE_BAD_WEIGHT;
    if (gate != NULL && up != NULL && scratch != NULL) {
        status = augur_oracle_linear_bf16(gate_codes, gate_scales, gate_global, intermediate,
                                          hidden, x_bf16, tokens, scratch, gate, threads);
        if (status == AUGUR_ORACLE_OK) {
            status = augur_oracle_linear_bf16(up_codes, up_scales, up_global, intermediate, hidden,
                                              x_bf16, tokens, scratch, up, threads);
        }
        if (status == AUGUR_ORACLE_OK) {
            for (size_t index = 0; index < count; ++index) {
                h_bf16[index] = augur_oracle_f32_to_bf16_bits(silu_mul_f32(gate[index], up[index]));
            }
            status = augur_oracle_linear_bf16(down_codes, down_scales, down_global, hidden,
                                              intermediate, h_bf16, tokens, y_bf16, NULL, threads);
        }
    }
    free(gate);
    free(up);
    free(scratch);
    return status;
}

int augur_oracle_mlp_f64(const uint8_t* gate_codes, const uint8_t* gate_scales, float gate_global,
                         const uint8_t* up_codes, const uint8_t* up_scales, float up_global,
                         const uint8_t* down_codes, const uint8_t* down_scales, float down_global,
                         size_t hidden, size_t intermediate, const uint16_t* x_bf16, size_t tokens,
                         double* h64, double* y64, int threads) {
    const size_t count = tokens * intermediate;
    double* gate = (double*)malloc(sizeof(double) * count);
    double* up = (double*)malloc(sizeof(double) * count);
    int status = AUGUR_ORACLE_BAD_WEIGHT;
    if (gate != NULL && up != NULL) {
        status = augur_oracle_linear_f64(gate_codes, gate_scales, gate_global, intermediate, hidden,
                                         x_bf16, tokens, gate, threads);
        if (status == AUGUR_ORACLE_OK) {
            status = augur_oracle_linear_f64(up_codes, up_scales, up_global, intermediate, hidden,
                                             x_bf16, tokens, up, threads);
        }
        if (status == AUGUR_ORACLE_OK) {
            for (size_t index = 0; index < count; ++index) {
                h64[index] = gate[index] / (1.0 + exp(-gate[index])) * up[index];
            }
            status = augur_oracle_linear_f64_xf64(down_codes, down_scales, down_global, hidden,
                                                  intermediate, h64, tokens, y64, threads);
        }
    }
    free(gate);
    free(up);
    return status;
}

/* ---- activation quantiser (BF16 -> NVFP4, optionally as a residual series) ----
 *
 * Rule, per 16-element group, following the reference's W4A4 interstage
 * quantiser (crates/augur-cuda-sys/native/augur_nvfp4_cutlass_sm120.cu:286-311,
 * 455-503): desired = amax / (6*global); block scale = the SMALLEST positive
 * E4M3 value >= desired (code 126 if none, code 0 when amax == 0); each
 * element becomes the E2M1 level nearest to value/(scale*global), a tie going
 * to the level listed first (so to the smaller magnitude, and never to -0).
 *
 * terms > 1 extends this to a residual series: term t quantises what terms
 * 0..t-1 left over, r_{t+1} = r_t - level*fl(scale*global), all in f32 with
 * single roundings (no fused multiply-add). Output planes are
 * codes [terms][tokens][cols/2] and scales [terms][tokens][cols/16].
 */
static float positive_e4m3(uint8_t code) {
    float out = 0.0f;
    augur_oracle_decode_e4m3fn(code, &out);
    return out;
}

static uint8_t e2m1_nearest_code(float value) {
    uint8_t best = 0;
    float best_distance = fabsf(value - E2M1_VALUES[0]);
    for (uint8_t code = 1; code < 16; ++code) {
        const float distance = fabsf(value - E2M1_VALUES[code]);
        if (distance < best_distance) {
            best = code;
            best_distance = distance;
        }
    }
    return best;
}

int augur_oracle_act_quant(const uint16_t* x_bf16, size_t tokens, size_t cols, float global_scale,
                           int terms, uint8_t* codes, uint8_t* scales) {
    if (tokens == 0 || cols == 0 || cols % 16 != 0 || terms < 1 || terms > 4 ||
        !isfinite(global_scale) || global_scale <= 0.0f) {
        return AUGUR_ORACLE_BAD_WEIGHT_SHAPE;
    }
    const size_t groups = cols / 16;
    for (size_t token = 0; token < tokens; ++token) {
        for (size_t group = 0; group < groups; ++group) {
            float residual[16];
            for (size_t lane = 0; lane < 16; ++lane) {
                residual[lane] = augur_oracle_bf16_bits_to_f32(x_bf16[token * cols + group * 16 + lane]);
            }
            for (int term = 0; term < terms; ++term) {
                float maximum = 0.0f;
                for (size_t lane = 0; lane < 16; ++lane) {
                    maximum = fmaxf(maximum, fabsf(residual[lane]));
                }
                const float desired = maximum / (6.0f * global_scale);
                uint8_t scale_code = 0;
                float scale = 0.0f;
                if (desired > 0.0f) {
                    for (unsigned candidate = 1; candidate <= 126; ++candidate) {
                        const float decoded = positive_e4m3((uint8_t)candidate);
                        if (decoded >= desired) {
                            scale_code = (uint8_t)candidate;
                            scale = decoded;
                            break;
                        }
                    }
                    if (scale_code == 0) {
                        scale_code = 126;
                        scale = positive_e4m3(126);
                    }
                }
                const float divisor = scale * global_scale;
                uint8_t packed[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (size_t lane = 0; lane < 16; ++lane) {
                    float normalized = divisor == 0.0f ? 0.0f : residual[lane] / divisor;
                    normalized = fminf(fmaxf(normalized, -6.0f), 6.0f);
                    const uint8_t code = e2m1_nearest_code(normalized);
                    packed[lane / 2] |= (uint8_t)(code << ((lane % 2) * 4));
                    const float dequantised = E2M1_VALUES[code] * divisor;
                    residual[lane] = residual[lane] - dequantised;
                }
                const size_t plane = ((size_t)term * tokens + token) * groups + group;
                memcpy(codes + plane * 8, packed, 8);
                scales[plane] = scale_code;
            }
        }
    }
    return AUGUR_ORACLE_OK;
}

int augur_oracle_act_dequant_f64(const uint8_t* codes, const uint8_t* scales, float global_scale,
                                 size_t tokens, size_t cols, int terms, double* out) {
    const size_t groups = cols / 16;
    for (size_t index = 0; index < tokens * cols; ++index) {
        out[index] = 0.0;
    }
    for (int term = 0; term < terms; ++term) {
        for (size_t token = 0; token < tokens; ++token) {
            for (size_t group = 0; group < groups; ++group) {
                const size_t plane = ((size_t)term * tokens + token) * groups + group;
                const double scale = (double)positive_e4m3(scales[plane]) * (double)global_scale;
                for (size_t lane = 0; lane < 16; ++lane) {
                    const uint8_t byte = codes[plane * 8 + lane / 2];
                    const uint8_t nibble = (lane % 2 == 0) ? (byte & 0x0f) : (byte >> 4);
                    out[token * cols + group * 16 + lane] += (double)E2M1_VALUES[nibble] * scale;
                }
            }
        }
    }
    return AUGUR_ORACLE_OK;
}
