// Host-side C++ view of augur_cuda_nvfp4_sm100.h: the owner types a backend crate keeps above
// the C ABI, restated in C++17 (header-only).
//
// It mirrors the safe wrappers Augur's backend puts above its native layer
// (crates/augur-backend/src/cuda_qwen35_prefill_cublas/qpn.rs:51-105,391-492 and
// crates/augur-backend/src/cuda_nvfp4_sm70.rs:226-289):
//   * a binding is made once with `bind(...)`, which runs the preflight; after that it is
//     immutable and `submit_for_plan()` only calls the prevalidated submit;
//   * a binding keeps shared owners (the Rust side uses Rc) of its plan, stream, weight, input
//     and output, so nothing a submitted kernel touches can be freed under it; dropping the last
//     owner of a stream synchronises it first;
//   * one serial stream per owner, single-threaded submission; a plan is only accepted with the
//     stream that created it, and the wrappers check that identity before the C call does;
//   * every failure is an exception that carries {status, raw_cuda_status} and the call's name
//     (the counterpart of CudaRuntimeError, crates/augur-backend/src/cuda_runtime.rs).
// Nothing here computes: every number comes from the library's kernels.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "augur_cuda_nvfp4_sm100.h"

namespace augur {
namespace nvfp4_sm100 {

class CudaRuntimeError : public std::runtime_error {
public:
    CudaRuntimeError(const std::string& where, int32_t status, int32_t raw)
        : std::runtime_error(where + ": status " + std::to_string(status) + ", cuda " + std::to_string(raw)),
          status(status), raw_cuda_status(raw) {}
    int32_t status;
    int32_t raw_cuda_status;
};

inline void check(const char* where, augur_cuda_result_v1 result) {
    if (result.status != AUGUR_CUDA_STATUS_OK) throw CudaRuntimeError(where, result.status, result.raw_cuda_status);
}
inline void check_cuda(const char* where, cudaError_t e) {
    if (e != cudaSuccess) throw CudaRuntimeError(where, AUGUR_CUDA_STATUS_RUNTIME_FAILURE, static_cast<int32_t>(e));
}

// A serial stream on one device. Destroying it synchronises first.
class Stream {
public:
    explicit Stream(int32_t ordinal) : ordinal_(ordinal) {
        check("stream_create", augur_cuda_nvfp4_sm100_stream_create_v1(ordinal, &handle_));
    }
    Stream(const Stream&) = delete;
    Stream& operator=(const Stream&) = delete;
    ~Stream() {
        if (handle_) {
            augur_cuda_nvfp4_sm100_stream_synchronize_v1(handle_);
            augur_cuda_nvfp4_sm100_stream_destroy_v1(handle_);
        }
    }
    void synchronize() const { check("stream_synchronize", augur_cuda_nvfp4_sm100_stream_synchronize_v1(handle_)); }
    int32_t ordinal() const { return ordinal_; }
    augur_cuda_stream_t handle() const { return handle_; }
    // The raw CUDA stream behind the handle; the handle's first two fields are {int32 ordinal; cudaStream_t stream}.
    cudaStream_t raw() const {
        struct View { int32_t ordinal; cudaStream_t stream; };
        return reinterpret_cast<const View*>(handle_)->stream;
    }

private:
    int32_t ordinal_;
    augur_cuda_stream_t handle_ = nullptr;
};

// Device memory with one owner; shared between bindings through shared_ptr.
class DeviceBuffer {
public:
    DeviceBuffer(int32_t ordinal, uint64_t bytes) : ordinal_(ordinal), bytes_(bytes) {
        check_cuda("cudaSetDevice", cudaSetDevice(ordinal));
        check_cuda("cudaMalloc", cudaMalloc(&pointer_, bytes ? bytes : 1));
    }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() {
        if (pointer_) cudaFree(pointer_);
    }
    uint64_t address() const { return reinterpret_cast<uint64_t>(pointer_); }
    uint64_t bytes() const { return bytes_; }
    int32_t ordinal() const { return ordinal_; }
    void upload(const Stream& stream, const void* host, uint64_t bytes, uint64_t offset = 0) {
        if (offset + bytes > bytes_) throw std::invalid_argument("upload beyond the buffer");
        check_cuda("cudaMemcpyAsync", cudaMemcpyAsync(static_cast<uint8_t*>(pointer_) + offset, host, bytes,
                                                       cudaMemcpyHostToDevice, stream.raw()));
    }
    void download(const Stream& stream, void* host, uint64_t bytes, uint64_t offset = 0) const {
        if (offset + bytes > bytes_) throw std::invalid_argument("download beyond the buffer");
        check_cuda("cudaMemcpyAsync", cudaMemcpyAsync(host, static_cast<const uint8_t*>(pointer_) + offset, bytes,
                                                       cudaMemcpyDeviceToHost, stream.raw()));
        stream.synchronize();
    }

private:
    int32_t ordinal_;
    uint64_t bytes_;
    void* pointer_ = nullptr;
};

template <class Args>
Args header() {
    Args args{};
    args.abi_version = AUGUR_CUDA_ABI_VERSION_V1;
    args.struct_size = static_cast<uint32_t>(sizeof(Args));
    return args;
}

// Stream-owned scratch. Creation and destruction are the only allocating calls of the library.
class Plan {
public:
    Plan(std::shared_ptr<Stream> stream, uint64_t scratch_bytes) : stream_(std::move(stream)) {
        check("plan_create", augur_cuda_nvfp4_sm100_plan_create_v1(stream_->ordinal(), stream_->handle(), scratch_bytes, &plan_));
    }
    Plan(const Plan&) = delete;
    Plan& operator=(const Plan&) = delete;
    ~Plan() {
        if (plan_) {
            augur_cuda_nvfp4_sm100_stream_synchronize_v1(stream_->handle());
            augur_cuda_nvfp4_sm100_plan_destroy_v1(plan_);
        }
    }
    augur_cuda_nvfp4_sm100_plan_snapshot_v1 snapshot() const {
        auto out = header<augur_cuda_nvfp4_sm100_plan_snapshot_v1>();
        check("plan_describe", augur_cuda_nvfp4_sm100_plan_describe_v1(plan_, &out));
        return out;
    }
    // Synchronises the stream; 0 means every bounded device wait was satisfied.
    uint32_t device_status() const {
        uint32_t word = 0;
        check("plan_device_status", augur_cuda_nvfp4_sm100_plan_device_status_v1(plan_, &word));
        return word;
    }
    const std::shared_ptr<Stream>& stream() const { return stream_; }
    augur_cuda_nvfp4_sm100_plan_v1* raw() const { return plan_; }

private:
    std::shared_ptr<Stream> stream_;
    augur_cuda_nvfp4_sm100_plan_v1* plan_ = nullptr;
};

inline uint64_t gemv_scratch_bytes(uint32_t rows, uint32_t cols, uint32_t tokens = AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) {
    uint64_t bytes = 0;
    check("gemv_scratch_extent", augur_cuda_nvfp4_sm100_gemv_scratch_extent_host_v1(rows, cols, tokens, &bytes));
    return bytes;
}
// Scratch of an MLP program: both members, each in its own half of the slot area.
inline uint64_t mlp_scratch_bytes(uint32_t hidden, uint32_t intermediate, uint32_t tokens = AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS) {
    const uint64_t a = gemv_scratch_bytes(intermediate, hidden, tokens), b = gemv_scratch_bytes(hidden, intermediate, tokens);
    return 2 * (a > b ? a : b) + 4096;
}
inline uint64_t gemm_scratch_bytes(uint32_t rows, uint32_t cols, uint32_t tokens, uint32_t terms) {
    uint64_t bytes = 0;
    check("gemm_scratch_extent", augur_cuda_nvfp4_sm100_gemm_scratch_extent_host_v1(rows, cols, tokens, terms, &bytes));
    return bytes;
}
// Plan scratch with which the prefill GEMM can cut its leftover tiles along k on a device of `sm_count` SMs.
inline uint64_t gemm_plan_scratch_bytes(uint32_t sm_count) {
    uint64_t bytes = 0;
    check("gemm_plan_scratch_extent", augur_cuda_nvfp4_sm100_gemm_plan_scratch_extent_host_v1(sm_count, &bytes));
    return bytes;
}
inline uint64_t repack_extent(uint32_t layout, uint32_t rows, uint32_t cols) {
    uint64_t bytes = 0;
    check("repack_extent", augur_cuda_nvfp4_sm100_repack_extent_host_v1(layout, rows, cols, &bytes));
    return bytes;
}

// One matrix in checkpoint form (crates/augur-model-qwen35/src/checkpoint_quant.rs:95-152):
// codes [rows][cols/2], scales [rows][cols/16], one f32 global scale.
struct CheckpointNvfp4Matrix {
    const uint8_t* codes;
    const uint8_t* scales;
    float global_scale;
};

// A weight tensor resident on the device in one of the hot layouts.
class Nvfp4Sm100Weight {
public:
    // Validates the planes the way the reference loader does before upload
    // (crates/augur-backend/src/cuda_qwen35_qpn.rs:59-72: no negative or NaN scale byte, finite
    // positive global scale), uploads them, repacks on the device and drops the planes.
    // `second` is the up matrix of a STREAM_PAIR tensor.
    static std::shared_ptr<Nvfp4Sm100Weight> upload_checkpoint_nvfp4(const std::shared_ptr<Stream>& stream, uint32_t layout,
                                                                    uint32_t rows, uint32_t cols,
                                                                    const CheckpointNvfp4Matrix& first,
                                                                    const CheckpointNvfp4Matrix* second = nullptr) {
        const bool pair = layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR;
        if (pair != (second != nullptr)) throw std::invalid_argument("STREAM_PAIR takes two matrices, other layouts one");
        const uint64_t code_bytes = static_cast<uint64_t>(rows) * cols / 2, scale_bytes = static_cast<uint64_t>(rows) * cols / 16;
        const CheckpointNvfp4Matrix* sources[2] = {&first, second};
        for (const CheckpointNvfp4Matrix* m : sources) {
            if (!m) continue;
            if (!(m->global_scale > 0.0f) || m->global_scale > 3.0e38f) throw std::invalid_argument("global scale must be finite and positive");
            for (uint64_t i = 0; i < scale_bytes; ++i) {
                if (m->scales[i] >= 0x7f) throw std::invalid_argument("block scale byte is negative or NaN");
            }
        }
        const int32_t d = stream->ordinal();
        auto align = [](uint64_t v) { return (v + 255) / 256 * 256; };
        const uint64_t at_scales = align(code_bytes), at_codes_b = at_scales + align(scale_bytes), at_scales_b = at_codes_b + align(code_bytes);
        auto staged = std::make_shared<DeviceBuffer>(d, at_scales_b + align(scale_bytes));
        staged->upload(*stream, first.codes, code_bytes, 0);
        staged->upload(*stream, first.scales, scale_bytes, at_scales);
        if (pair) {
            staged->upload(*stream, second->codes, code_bytes, at_codes_b);
            staged->upload(*stream, second->scales, scale_bytes, at_scales_b);
        }
        auto weight = std::shared_ptr<Nvfp4Sm100Weight>(new Nvfp4Sm100Weight());
        weight->stream_ = stream;
        weight->layout_ = layout;
        weight->rows_ = rows;
        weight->cols_ = cols;
        weight->global_scale_ = first.global_scale;
        weight->global_scale_b_ = pair ? second->global_scale : 0.0f;
        weight->packed_ = std::make_shared<DeviceBuffer>(d, repack_extent(layout, rows, cols));
        auto args = header<augur_cuda_nvfp4_sm100_repack_args_v1>();
        args.codes = staged->address();
        args.codes_len_bytes = code_bytes;
        args.scales = staged->address() + at_scales;
        args.scales_len_bytes = scale_bytes;
        if (pair) {
            args.codes_b = staged->address() + at_codes_b;
            args.codes_b_len_bytes = code_bytes;
            args.scales_b = staged->address() + at_scales_b;
            args.scales_b_len_bytes = scale_bytes;
        }
        args.destination = weight->packed_->address();
        args.destination_len_bytes = weight->packed_->bytes();
        args.rows = rows;
        args.cols = cols;
        args.layout = layout;
        check("repack_preflight", augur_cuda_nvfp4_sm100_repack_preflight_v1(d, stream->handle(), &args));
        check("repack_submit", augur_cuda_nvfp4_sm100_repack_prevalidated_submit_v1(d, stream->handle(), &args));
        stream->synchronize();   // the staged planes are released when this function returns
        return weight;
    }

    uint32_t layout() const { return layout_; }
    uint32_t rows() const { return rows_; }   // rows of each source matrix (a pair tensor holds twice as many)
    uint32_t cols() const { return cols_; }
    float global_scale() const { return global_scale_; }
    float global_scale_b() const { return global_scale_b_; }
    const std::shared_ptr<DeviceBuffer>& packed() const { return packed_; }
    const std::shared_ptr<Stream>& stream() const { return stream_; }

private:
    Nvfp4Sm100Weight() = default;
    std::shared_ptr<Stream> stream_;
    std::shared_ptr<DeviceBuffer> packed_;
    uint32_t layout_ = 0, rows_ = 0, cols_ = 0;
    float global_scale_ = 0.0f, global_scale_b_ = 0.0f;
};

inline augur_cuda_nvfp4_sm100_gemv_args_v1 gemv_args(const Nvfp4Sm100Weight& weight, const DeviceBuffer& input,
                                                      const DeviceBuffer& output, uint32_t tokens, uint32_t epilogue) {
    auto args = header<augur_cuda_nvfp4_sm100_gemv_args_v1>();
    args.weight = weight.packed()->address();
    args.weight_len_bytes = weight.packed()->bytes();
    args.input_bf16 = input.address();
    args.input_len_bytes = static_cast<uint64_t>(tokens) * weight.cols() * 2;
    args.output = output.address();
    args.rows = weight.rows();
    args.output_len_bytes = static_cast<uint64_t>(tokens) * args.rows * (epilogue == AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_F32 ? 4 : 2);
    args.cols = weight.cols();
    args.tokens = tokens;
    args.epilogue = epilogue;
    args.global_scale = weight.global_scale();
    args.global_scale_b = weight.global_scale_b();
    return args;
}

// One small-token linear (tokens 1..8) bound to its buffers.
class Nvfp4Sm100Projection {
public:
    static std::unique_ptr<Nvfp4Sm100Projection> bind(std::shared_ptr<Plan> plan, std::shared_ptr<Nvfp4Sm100Weight> weight,
                                                      std::shared_ptr<DeviceBuffer> input, std::shared_ptr<DeviceBuffer> output,
                                                      uint32_t tokens, uint32_t epilogue = AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16) {
        if (plan->stream() != weight->stream()) throw std::invalid_argument("plan and weight belong to different streams");
        std::unique_ptr<Nvfp4Sm100Projection> binding(new Nvfp4Sm100Projection());
        binding->args_ = gemv_args(*weight, *input, *output, tokens, epilogue);
        const Stream& s = *plan->stream();
        check("gemv_bf16_preflight", augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(s.ordinal(), s.handle(), plan->raw(), &binding->args_));
        binding->plan_ = std::move(plan);
        binding->weight_ = std::move(weight);
        binding->input_ = std::move(input);
        binding->output_ = std::move(output);
        return binding;
    }
    // Enqueues on the plan's stream and returns; never synchronises, never allocates.
    void submit_for_plan() const {
        const Stream& s = *plan_->stream();
        check("gemv_bf16_submit", augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1(s.ordinal(), s.handle(), plan_->raw(), &args_));
    }
    const std::shared_ptr<DeviceBuffer>& output() const { return output_; }

private:
    Nvfp4Sm100Projection() = default;
    augur_cuda_nvfp4_sm100_gemv_args_v1 args_{};
    std::shared_ptr<Plan> plan_;
    std::shared_ptr<Nvfp4Sm100Weight> weight_;
    std::shared_ptr<DeviceBuffer> input_, output_;
};

// The MLP block for tokens 1..8: gate|up with fused SwiGLU, then down; one validated program.
class Nvfp4Sm100FfnProgram {
public:
    static std::unique_ptr<Nvfp4Sm100FfnProgram> bind(std::shared_ptr<Plan> plan, std::shared_ptr<Nvfp4Sm100Weight> gate_up,
                                                      std::shared_ptr<Nvfp4Sm100Weight> down, std::shared_ptr<DeviceBuffer> input,
                                                      std::shared_ptr<DeviceBuffer> output, uint32_t tokens) {
        if (gate_up->layout() != AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR || down->layout() != AUGUR_NVFP4_SM100_LAYOUT_STREAM) {
            throw std::invalid_argument("gate|up must be STREAM_PAIR and down STREAM");
        }
        if (plan->stream() != gate_up->stream() || plan->stream() != down->stream()) {
            throw std::invalid_argument("plan and weights belong to different streams");
        }
        std::unique_ptr<Nvfp4Sm100FfnProgram> program(new Nvfp4Sm100FfnProgram());
        const Stream& s = *plan->stream();
        program->intermediate_ = std::make_shared<DeviceBuffer>(s.ordinal(), static_cast<uint64_t>(tokens) * gate_up->rows() * 2);
        program->args_ = header<augur_cuda_nvfp4_sm100_mlp_args_v1>();
        program->args_.gate_up = gemv_args(*gate_up, *input, *program->intermediate_, tokens, AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16);
        program->args_.down = gemv_args(*down, *program->intermediate_, *output, tokens, AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16);
        check("mlp_preflight", augur_cuda_nvfp4_sm100_mlp_preflight_v1(s.ordinal(), s.handle(), plan->raw(), &program->args_));
        program->plan_ = std::move(plan);
        program->gate_up_ = std::move(gate_up);
        program->down_ = std::move(down);
        program->input_ = std::move(input);
        program->output_ = std::move(output);
        return program;
    }
    void submit_for_plan() const {
        const Stream& s = *plan_->stream();
        check("mlp_submit", augur_cuda_nvfp4_sm100_mlp_prevalidated_submit_v1(s.ordinal(), s.handle(), plan_->raw(), &args_));
    }
    const std::shared_ptr<DeviceBuffer>& intermediate() const { return intermediate_; }
    const std::shared_ptr<DeviceBuffer>& output() const { return output_; }

private:
    Nvfp4Sm100FfnProgram() = default;
    augur_cuda_nvfp4_sm100_mlp_args_v1 args_{};
    std::shared_ptr<Plan> plan_;
    std::shared_ptr<Nvfp4Sm100Weight> gate_up_, down_;
    std::shared_ptr<DeviceBuffer> input_, intermediate_, output_;
};

// The wide (tokens a multiple of 128) linear: activation quantiser, then the block-scaled GEMM.
class Nvfp4Sm100PrefillLinear {
public:
    static std::unique_ptr<Nvfp4Sm100PrefillLinear> bind(std::shared_ptr<Plan> plan, std::shared_ptr<Nvfp4Sm100Weight> weight,
                                                         std::shared_ptr<DeviceBuffer> input, std::shared_ptr<DeviceBuffer> output,
                                                         uint32_t tokens, uint32_t terms, float activation_global_scale) {
        if (weight->layout() != AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) throw std::invalid_argument("prefill takes a TCGEN05 weight");
        if (plan->stream() != weight->stream()) throw std::invalid_argument("plan and weight belong to different streams");
        std::unique_ptr<Nvfp4Sm100PrefillLinear> binding(new Nvfp4Sm100PrefillLinear());
        const Stream& s = *plan->stream();
        const uint64_t staged_bytes = gemm_scratch_bytes(weight->rows(), weight->cols(), tokens, terms);
        binding->staged_ = std::make_shared<DeviceBuffer>(s.ordinal(), staged_bytes);
        binding->quant_ = header<augur_cuda_nvfp4_sm100_act_quant_args_v1>();
        binding->quant_.input_bf16 = input->address();
        binding->quant_.input_len_bytes = static_cast<uint64_t>(tokens) * weight->cols() * 2;
        binding->quant_.destination = binding->staged_->address();
        binding->quant_.destination_len_bytes = staged_bytes;
        binding->quant_.tokens = tokens;
        binding->quant_.cols = weight->cols();
        binding->quant_.terms = terms;
        binding->quant_.global_scale = activation_global_scale;
        binding->gemm_ = header<augur_cuda_nvfp4_sm100_gemm_args_v1>();
        binding->gemm_.weight = weight->packed()->address();
        binding->gemm_.weight_len_bytes = weight->packed()->bytes();
        binding->gemm_.activation = binding->staged_->address();
        binding->gemm_.activation_len_bytes = staged_bytes;
        binding->gemm_.output_bf16 = output->address();
        binding->gemm_.output_len_bytes = static_cast<uint64_t>(tokens) * weight->rows() * 2;
        binding->gemm_.rows = weight->rows();
        binding->gemm_.cols = weight->cols();
        binding->gemm_.tokens = tokens;
        binding->gemm_.activation_terms = terms;
        binding->gemm_.weight_global_scale = weight->global_scale();
        binding->gemm_.activation_global_scale = activation_global_scale;
        check("act_quant_preflight", augur_cuda_nvfp4_sm100_act_quant_preflight_v1(s.ordinal(), s.handle(), &binding->quant_));
        check("gemm_bf16_preflight", augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(s.ordinal(), s.handle(), plan->raw(), &binding->gemm_));
        binding->plan_ = std::move(plan);
        binding->weight_ = std::move(weight);
        binding->input_ = std::move(input);
        binding->output_ = std::move(output);
        return binding;
    }
    void submit_for_plan() const {
        const Stream& s = *plan_->stream();
        check("act_quant_submit", augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(s.ordinal(), s.handle(), &quant_));
        check("gemm_bf16_submit", augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(s.ordinal(), s.handle(), plan_->raw(), &gemm_));
    }
    const std::shared_ptr<DeviceBuffer>& output() const { return output_; }

private:
    Nvfp4Sm100PrefillLinear() = default;
    augur_cuda_nvfp4_sm100_act_quant_args_v1 quant_{};
    augur_cuda_nvfp4_sm100_gemm_args_v1 gemm_{};
    std::shared_ptr<Plan> plan_;
    std::shared_ptr<Nvfp4Sm100Weight> weight_;
    std::shared_ptr<DeviceBuffer> input_, staged_, output_;
};

// The gate and up matrices as ONE tcgen05 weight of 2 * inter rows, 16 gate rows alternating with the matching
// 16 up rows: what the SwiGLU-fusing GEMM epilogue expects. rows() of the result is 2 * inter.
inline std::shared_ptr<Nvfp4Sm100Weight> upload_gate_up_interleaved(const std::shared_ptr<Stream>& stream, uint32_t inter,
                                                                   uint32_t hidden, const CheckpointNvfp4Matrix& gate,
                                                                   const CheckpointNvfp4Matrix& up, float* up_global_scale_out) {
    std::vector<uint8_t> codes(static_cast<size_t>(2) * inter * hidden / 2), scales(static_cast<size_t>(2) * inter * hidden / 16);
    check("interleave_gate_up", augur_cuda_nvfp4_sm100_interleave_gate_up_host_v1(inter, hidden, gate.codes, gate.scales, up.codes,
                                                                                 up.scales, codes.data(), scales.data()));
    if (!(up.global_scale > 0.0f) || up.global_scale > 3.0e38f) throw std::invalid_argument("global scale must be finite and positive");
    for (size_t i = static_cast<size_t>(inter) * hidden / 16; i-- > 0;) {
        if (up.scales[i] >= 0x7f) throw std::invalid_argument("block scale byte is negative or NaN");
    }
    const CheckpointNvfp4Matrix both{codes.data(), scales.data(), gate.global_scale};
    *up_global_scale_out = up.global_scale;
    return Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, 2 * inter, hidden, both);
}

// Plan scratch for the MLP block on the tensor-memory small-token kernel: both members' needs, side by side.
inline uint64_t mlp_tc_scratch_bytes(uint32_t hidden, uint32_t intermediate) {
    uint64_t first = 0, second = 0;
    check("gemv_tc_scratch_extent", augur_cuda_nvfp4_sm100_gemv_tc_scratch_extent_host_v1(intermediate, hidden, AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16, &first));
    check("gemv_tc_scratch_extent", augur_cuda_nvfp4_sm100_gemv_tc_scratch_extent_host_v1(hidden, intermediate, AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16, &second));
    return 2 * (first > second ? first : second) + 512;
}

// The MLP block for tokens 1..8 on the tensor-memory kernel: ONE launch; `gate_up` is the interleaved TCGEN05
// weight of `upload_gate_up_interleaved` (the weight the prefill program uses), `down` a TCGEN05 weight. Same
// contract as Nvfp4Sm100FfnProgram.
class Nvfp4Sm100TcFfnProgram {
public:
    static std::unique_ptr<Nvfp4Sm100TcFfnProgram> bind(std::shared_ptr<Plan> plan, std::shared_ptr<Nvfp4Sm100Weight> gate_up,
                                                        float up_global_scale, std::shared_ptr<Nvfp4Sm100Weight> down,
                                                        std::shared_ptr<DeviceBuffer> input, std::shared_ptr<DeviceBuffer> output, uint32_t tokens) {
        if (gate_up->layout() != AUGUR_NVFP4_SM100_LAYOUT_TCGEN05 || down->layout() != AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) {
            throw std::invalid_argument("gate|up and down must be TCGEN05 weights");
        }
        if (plan->stream() != gate_up->stream() || plan->stream() != down->stream()) {
            throw std::invalid_argument("plan and weights belong to different streams");
        }
        std::unique_ptr<Nvfp4Sm100TcFfnProgram> program(new Nvfp4Sm100TcFfnProgram());
        const Stream& s = *plan->stream();
        const uint32_t inter = gate_up->rows() / 2;
        program->intermediate_ = std::make_shared<DeviceBuffer>(s.ordinal(), static_cast<uint64_t>(tokens) * inter * 2);
        program->args_ = header<augur_cuda_nvfp4_sm100_mlp_args_v1>();
        program->args_.gate_up = gemv_args(*gate_up, *input, *program->intermediate_, tokens, AUGUR_NVFP4_SM100_EPILOGUE_SWIGLU_BF16);
        program->args_.gate_up.rows = inter;
        program->args_.gate_up.output_len_bytes = static_cast<uint64_t>(tokens) * inter * 2;
        program->args_.gate_up.global_scale_b = up_global_scale;
        program->args_.down = gemv_args(*down, *program->intermediate_, *output, tokens, AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16);
        check("mlp_tc_preflight", augur_cuda_nvfp4_sm100_mlp_tc_preflight_v1(s.ordinal(), s.handle(), plan->raw(), &program->args_));
        program->plan_ = std::move(plan);
        program->gate_up_ = std::move(gate_up);
        program->down_ = std::move(down);
        program->input_ = std::move(input);
        program->output_ = std::move(output);
        return program;
    }
    void submit_for_plan() const {
        const Stream& s = *plan_->stream();
        check("mlp_tc_submit", augur_cuda_nvfp4_sm100_mlp_tc_prevalidated_submit_v1(s.ordinal(), s.handle(), plan_->raw(), &args_));
    }
    const std::shared_ptr<DeviceBuffer>& intermediate() const { return intermediate_; }
    const std::shared_ptr<DeviceBuffer>& output() const { return output_; }

private:
    Nvfp4Sm100TcFfnProgram() = default;
    augur_cuda_nvfp4_sm100_mlp_args_v1 args_{};
    std::shared_ptr<Plan> plan_;
    std::shared_ptr<Nvfp4Sm100Weight> gate_up_, down_;
    std::shared_ptr<DeviceBuffer> input_, intermediate_, output_;
};

// The MLP block for wide inputs (any token count): quantise x, gate|up GEMM with SiLU(gate)*up in its epilogue,
// quantise the intermediate, down GEMM. Four launches; every member is preflighted at bind time.
class Nvfp4Sm100PrefillFfnProgram {
public:
    static std::unique_ptr<Nvfp4Sm100PrefillFfnProgram> bind(std::shared_ptr<Plan> plan, std::shared_ptr<Nvfp4Sm100Weight> gate_up,
                                                            float up_global_scale, std::shared_ptr<Nvfp4Sm100Weight> down,
                                                            std::shared_ptr<DeviceBuffer> input, std::shared_ptr<DeviceBuffer> output,
                                                            uint32_t tokens, uint32_t terms, float input_global_scale,
                                                            float intermediate_global_scale) {
        if (gate_up->layout() != AUGUR_NVFP4_SM100_LAYOUT_TCGEN05 || down->layout() != AUGUR_NVFP4_SM100_LAYOUT_TCGEN05) {
            throw std::invalid_argument("both weights must be in the tcgen05 layout");
        }
        if (plan->stream() != gate_up->stream() || plan->stream() != down->stream()) {
            throw std::invalid_argument("plan and weights belong to different streams");
        }
        const uint32_t hidden = gate_up->cols(), inter = gate_up->rows() / 2;
        if (down->cols() != inter) throw std::invalid_argument("gate|up and down shapes do not fit together");
        std::unique_ptr<Nvfp4Sm100PrefillFfnProgram> p(new Nvfp4Sm100PrefillFfnProgram());
        const Stream& s = *plan->stream();
        const int32_t d = s.ordinal();
        p->intermediate_ = std::make_shared<DeviceBuffer>(d, static_cast<uint64_t>(tokens) * inter * 2);
        p->staged_x_ = std::make_shared<DeviceBuffer>(d, gemm_scratch_bytes(gate_up->rows(), hidden, tokens, terms));
        p->staged_h_ = std::make_shared<DeviceBuffer>(d, gemm_scratch_bytes(down->rows(), inter, tokens, terms));
        auto quant = [&](const DeviceBuffer& source, const DeviceBuffer& staged, uint32_t cols, float scale) {
            auto q = header<augur_cuda_nvfp4_sm100_act_quant_args_v1>();
            q.input_bf16 = source.address();
            q.input_len_bytes = static_cast<uint64_t>(tokens) * cols * 2;
            q.destination = staged.address();
            q.destination_len_bytes = staged.bytes();
            q.tokens = tokens; q.cols = cols; q.terms = terms; q.global_scale = scale;
            return q;
        };
        p->quant_x_ = quant(*input, *p->staged_x_, hidden, input_global_scale);
        p->quant_h_ = quant(*p->intermediate_, *p->staged_h_, inter, intermediate_global_scale);
        p->gate_up_args_ = header<augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1>();
        p->gate_up_args_.weight = gate_up->packed()->address();
        p->gate_up_args_.weight_len_bytes = gate_up->packed()->bytes();
        p->gate_up_args_.activation = p->staged_x_->address();
        p->gate_up_args_.activation_len_bytes = p->staged_x_->bytes();
        p->gate_up_args_.output_bf16 = p->intermediate_->address();
        p->gate_up_args_.output_len_bytes = static_cast<uint64_t>(tokens) * inter * 2;
        p->gate_up_args_.rows = inter; p->gate_up_args_.cols = hidden; p->gate_up_args_.tokens = tokens;
        p->gate_up_args_.activation_terms = terms;
        p->gate_up_args_.gate_global_scale = gate_up->global_scale();
        p->gate_up_args_.up_global_scale = up_global_scale;
        p->gate_up_args_.activation_global_scale = input_global_scale;
        p->down_args_ = header<augur_cuda_nvfp4_sm100_gemm_args_v1>();
        p->down_args_.weight = down->packed()->address();
        p->down_args_.weight_len_bytes = down->packed()->bytes();
        p->down_args_.activation = p->staged_h_->address();
        p->down_args_.activation_len_bytes = p->staged_h_->bytes();
        p->down_args_.output_bf16 = output->address();
        p->down_args_.output_len_bytes = static_cast<uint64_t>(tokens) * down->rows() * 2;
        p->down_args_.rows = down->rows(); p->down_args_.cols = inter; p->down_args_.tokens = tokens;
        p->down_args_.activation_terms = terms;
        p->down_args_.weight_global_scale = down->global_scale();
        p->down_args_.activation_global_scale = intermediate_global_scale;
        // On the two-CTA tiles the gate|up GEMM quantises its result for the down GEMM in its own epilogue
        // (three launches instead of four; the BF16 intermediate is still written here).
        p->fused_ = inter % 128 == 0;
        check("act_quant_preflight", augur_cuda_nvfp4_sm100_act_quant_preflight_v1(d, s.handle(), &p->quant_x_));
        if (p->fused_) {
            p->fused_args_ = header<augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1>();
            p->fused_args_.weight = p->gate_up_args_.weight;
            p->fused_args_.weight_len_bytes = p->gate_up_args_.weight_len_bytes;
            p->fused_args_.activation = p->gate_up_args_.activation;
            p->fused_args_.activation_len_bytes = p->gate_up_args_.activation_len_bytes;
            p->fused_args_.output_bf16 = p->gate_up_args_.output_bf16;
            p->fused_args_.output_len_bytes = p->gate_up_args_.output_len_bytes;
            p->fused_args_.destination = p->staged_h_->address();
            p->fused_args_.destination_len_bytes = p->staged_h_->bytes();
            p->fused_args_.rows = inter; p->fused_args_.cols = hidden; p->fused_args_.tokens = tokens;
            p->fused_args_.activation_terms = terms;
            p->fused_args_.gate_global_scale = gate_up->global_scale();
            p->fused_args_.up_global_scale = up_global_scale;
            p->fused_args_.activation_global_scale = input_global_scale;
            p->fused_args_.destination_global_scale = intermediate_global_scale;
            p->fused_args_.destination_terms = terms;
            check("gemm_swiglu_quant_preflight",
                  augur_cuda_nvfp4_sm100_gemm_swiglu_quant_preflight_v1(d, s.handle(), plan->raw(), &p->fused_args_));
        } else {
            check("gemm_swiglu_preflight", augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_preflight_v1(d, s.handle(), plan->raw(), &p->gate_up_args_));
            check("act_quant_preflight", augur_cuda_nvfp4_sm100_act_quant_preflight_v1(d, s.handle(), &p->quant_h_));
        }
        check("gemm_bf16_preflight", augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(d, s.handle(), plan->raw(), &p->down_args_));
        p->plan_ = std::move(plan);
        p->gate_up_ = std::move(gate_up);
        p->down_ = std::move(down);
        p->input_ = std::move(input);
        p->output_ = std::move(output);
        return p;
    }
    void submit_for_plan() const {
        const Stream& s = *plan_->stream();
        const int32_t d = s.ordinal();
        check("act_quant_submit", augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(d, s.handle(), &quant_x_));
        if (fused_) {
            check("gemm_swiglu_quant_submit",
                  augur_cuda_nvfp4_sm100_gemm_swiglu_quant_prevalidated_submit_v1(d, s.handle(), plan_->raw(), &fused_args_));
        } else {
            check("gemm_swiglu_submit", augur_cuda_nvfp4_sm100_gemm_swiglu_bf16_prevalidated_submit_v1(d, s.handle(), plan_->raw(), &gate_up_args_));
            check("act_quant_submit", augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1(d, s.handle(), &quant_h_));
        }
        check("gemm_bf16_submit", augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1(d, s.handle(), plan_->raw(), &down_args_));
    }
    const std::shared_ptr<DeviceBuffer>& intermediate() const { return intermediate_; }
    const std::shared_ptr<DeviceBuffer>& output() const { return output_; }

private:
    Nvfp4Sm100PrefillFfnProgram() = default;
    augur_cuda_nvfp4_sm100_act_quant_args_v1 quant_x_{}, quant_h_{};
    augur_cuda_nvfp4_sm100_gemm_swiglu_args_v1 gate_up_args_{};
    augur_cuda_nvfp4_sm100_gemm_swiglu_quant_args_v1 fused_args_{};
    bool fused_ = false;
    augur_cuda_nvfp4_sm100_gemm_args_v1 down_args_{};
    std::shared_ptr<Plan> plan_;
    std::shared_ptr<Nvfp4Sm100Weight> gate_up_, down_;
    std::shared_ptr<DeviceBuffer> input_, intermediate_, staged_x_, staged_h_, output_;
};

// [residual add] -> RMSNorm -> BF16 stage -> one to four small-token projections as one validated program
// (the reference's GDN-input and post-attention groups, native augur_qwen35_gdn_input_b8.cuh).
class Nvfp4Sm100NormGroupProgram {
public:
    // `input_f32` is the residual stream [tokens][cols]; with `add_a` / `add_b` it is overwritten by their sum first.
    static std::unique_ptr<Nvfp4Sm100NormGroupProgram> bind(std::shared_ptr<Plan> plan,
                                                           std::vector<std::shared_ptr<Nvfp4Sm100Weight>> weights,
                                                           std::shared_ptr<DeviceBuffer> input_f32,
                                                           std::shared_ptr<DeviceBuffer> norm_weight_f32, uint32_t tokens, uint32_t cols,
                                                           float epsilon, std::shared_ptr<DeviceBuffer> add_a = nullptr,
                                                           std::shared_ptr<DeviceBuffer> add_b = nullptr) {
        if (weights.empty() || weights.size() > 4) throw std::invalid_argument("one to four projections");
        if (static_cast<bool>(add_a) != static_cast<bool>(add_b)) throw std::invalid_argument("the residual add takes both operands or none");
        std::unique_ptr<Nvfp4Sm100NormGroupProgram> p(new Nvfp4Sm100NormGroupProgram());
        const Stream& s = *plan->stream();
        const int32_t d = s.ordinal();
        const uint64_t elements = static_cast<uint64_t>(tokens) * cols;
        p->normalised_ = std::make_shared<DeviceBuffer>(d, elements * 4);
        p->staged_ = std::make_shared<DeviceBuffer>(d, elements * 2);
        p->args_ = header<augur_cuda_nvfp4_sm100_norm_group_args_v1>();
        if (add_a) {
            p->args_.add_a = add_a->address();
            p->args_.add_b = add_b->address();
            p->args_.add_len_bytes = elements * 4;
            p->args_.residual = 1;
        }
        p->args_.input_f32 = input_f32->address();
        p->args_.input_len_bytes = elements * 4;
        p->args_.weight_f32 = norm_weight_f32->address();
        p->args_.weight_len_bytes = static_cast<uint64_t>(cols) * 4;
        p->args_.output_f32 = p->normalised_->address();
        p->args_.output_len_bytes = elements * 4;
        p->args_.staged_bf16 = p->staged_->address();
        p->args_.staged_len_bytes = elements * 2;
        p->args_.tokens = tokens; p->args_.cols = cols; p->args_.epsilon = epsilon;
        p->args_.count = static_cast<uint32_t>(weights.size());
        for (size_t i = 0; i < weights.size(); ++i) {
            if (plan->stream() != weights[i]->stream()) throw std::invalid_argument("plan and weight belong to different streams");
            p->outputs_.push_back(std::make_shared<DeviceBuffer>(d, static_cast<uint64_t>(tokens) * weights[i]->rows() * 2));
            p->args_.projections[i] = gemv_args(*weights[i], *p->staged_, *p->outputs_[i], tokens, AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16);
        }
        check("norm_group_preflight", augur_cuda_nvfp4_sm100_norm_group_preflight_v1(d, s.handle(), plan->raw(), &p->args_));
        p->plan_ = std::move(plan);
        p->weights_ = std::move(weights);
        p->input_ = std::move(input_f32);
        p->norm_weight_ = std::move(norm_weight_f32);
        p->add_a_ = std::move(add_a);
        p->add_b_ = std::move(add_b);
        return p;
    }
    void submit_for_plan() const {
        const Stream& s = *plan_->stream();
        check("norm_group_submit", augur_cuda_nvfp4_sm100_norm_group_prevalidated_submit_v1(s.ordinal(), s.handle(), plan_->raw(), &args_));
    }
    const std::shared_ptr<DeviceBuffer>& normalised() const { return normalised_; }
    const std::shared_ptr<DeviceBuffer>& staged() const { return staged_; }
    const std::vector<std::shared_ptr<DeviceBuffer>>& outputs() const { return outputs_; }

private:
    Nvfp4Sm100NormGroupProgram() = default;
    augur_cuda_nvfp4_sm100_norm_group_args_v1 args_{};
    std::shared_ptr<Plan> plan_;
    std::vector<std::shared_ptr<Nvfp4Sm100Weight>> weights_;
    std::shared_ptr<DeviceBuffer> input_, norm_weight_, add_a_, add_b_, normalised_, staged_;
    std::vector<std::shared_ptr<DeviceBuffer>> outputs_;
};

// The reference's batch classes (crates/augur-kernel-api/src/key.rs:354-365): up to 8 token rows are the
// small-batch class (decode and the fixed B8 verify batch), anything wider is prefill.
enum class BatchClass { SmallBatch, Prefill };
inline BatchClass classify_tokens(uint32_t tokens) {
    if (tokens < 1) throw std::invalid_argument("at least one token row");
    return tokens <= AUGUR_NVFP4_SM100_MAX_SMALL_TOKENS ? BatchClass::SmallBatch : BatchClass::Prefill;
}

// One weight matrix in both hot layouts; `bind_*` picks the kernel the token count calls for.
class Nvfp4Sm100Linear {
public:
    Nvfp4Sm100Linear(const std::shared_ptr<Stream>& stream, uint32_t rows, uint32_t cols, const CheckpointNvfp4Matrix& matrix)
        : small_(Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_STREAM, rows, cols, matrix)),
          wide_(Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, rows, cols, matrix)) {}
    const std::shared_ptr<Nvfp4Sm100Weight>& small_batch_weight() const { return small_; }
    const std::shared_ptr<Nvfp4Sm100Weight>& prefill_weight() const { return wide_; }
    // tokens <= 8
    std::unique_ptr<Nvfp4Sm100Projection> bind_small_batch(std::shared_ptr<Plan> plan, std::shared_ptr<DeviceBuffer> input,
                                                           std::shared_ptr<DeviceBuffer> output, uint32_t tokens) const {
        if (classify_tokens(tokens) != BatchClass::SmallBatch) throw std::invalid_argument("more than 8 token rows: bind_prefill");
        return Nvfp4Sm100Projection::bind(std::move(plan), small_, std::move(input), std::move(output), tokens);
    }
    // tokens > 8 (any count)
    std::unique_ptr<Nvfp4Sm100PrefillLinear> bind_prefill(std::shared_ptr<Plan> plan, std::shared_ptr<DeviceBuffer> input,
                                                          std::shared_ptr<DeviceBuffer> output, uint32_t tokens, uint32_t terms = 3,
                                                          float activation_global_scale = 1.0f / 256.0f) const {
        return Nvfp4Sm100PrefillLinear::bind(std::move(plan), wide_, std::move(input), std::move(output), tokens, terms,
                                             activation_global_scale);
    }

private:
    std::shared_ptr<Nvfp4Sm100Weight> small_, wide_;
};

// Device allocations / frees made by the library so far (cuda_device_allocation_snapshot,
// crates/augur-backend/src/cuda_runtime.rs:528-535): equal before and after a hot loop.
inline std::pair<uint64_t, uint64_t> allocation_snapshot() {
    uint64_t allocations = 0, frees = 0;
    augur_cuda_nvfp4_sm100_allocation_snapshot_v1(&allocations, &frees);
    return {allocations, frees};
}
inline uint64_t launch_count() { return augur_cuda_nvfp4_sm100_launch_count_v1(); }

}  // namespace nvfp4_sm100
}  // namespace augur
