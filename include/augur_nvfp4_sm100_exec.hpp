// Execution-plan layer over the NVFP4 linear: the counterpart of what the reference's compiler and executor do
// for a quantised mat-mul node (lowering template crates/augur-compiler/src/lowering.rs:1139-1200; planned
// step and its execution crates/augur-exec/src/plan.rs:203-208,293,378-395; CUDA side
// crates/augur-exec/src/cuda_plan.rs:184-199), restated for the sm_100a library in C++17, header-only.
//
// Two stages, as in the reference:
//   * `lower(...)` is host-only and touches no device. It looks at a node (weight format, block size, format
//     version, shape, token rows), rejects what this backend does not run (`Unsupported`, the counterpart of
//     CompileError::BackendUnsupported) and selects the entry points by the batch class of the node
//     (crates/augur-kernel-api/src/key.rs:354-365): up to 8 token rows -> the small-token kernel
//     (`PlannedOp::Nvfp4LinearGemv`), more -> activation quantiser + block-scaled GEMM
//     (`PlannedOp::Nvfp4LinearGemm`). A compiled step stores the entry's address, so a test can check which
//     kernel was selected without running it.
//   * `bind(...)` resolves the weight requirements against uploaded weights, allocates the plan's buffers,
//     runs every step's preflight once and returns an `ExecutionPlan`. `submit_steps()` only enqueues (no
//     allocation, no synchronisation, no driver query); `execute()` adds the stream synchronisation;
//     `execute_profiled()` brackets every step with CUDA events and returns per-kind device times.
// The plan keeps shared owners of everything its steps touch; a weight's owner and payload address do not
// change between executions.
#pragma once

#include <map>
#include <variant>

#include "augur_nvfp4_sm100.hpp"

namespace augur {
namespace nvfp4_sm100 {
namespace exec {

// What a graph node says about its quantised weight (crates/augur-core: QuantFormatId, block size, format version).
enum class QuantFormat : uint32_t { NVFP4 = 1, MXFP4 = 2, Q8_0 = 3 };
constexpr uint32_t kNvfp4Block = 16;
constexpr uint16_t kNvfp4FormatVersion = 1;

struct WeightId {
    uint32_t value;
    bool operator<(const WeightId& other) const { return value < other.value; }
    bool operator==(const WeightId& other) const { return value == other.value; }
};

// A quantised mat-mul node: y[tokens][rows] = x[tokens][cols] * W^T, BF16 in and out.
struct QMatmulNode {
    WeightId weight;
    QuantFormat format;
    uint32_t block;
    uint16_t version;
    uint32_t rows, cols, tokens;
    uint32_t input_buffer, output_buffer;   // indices into the plan's buffer table
};

class Unsupported : public std::runtime_error {
public:
    explicit Unsupported(const std::string& why) : std::runtime_error("backend unsupported: " + why) {}
};

using GemvSubmit = augur_cuda_result_v1 (*)(int32_t, augur_cuda_stream_t, augur_cuda_nvfp4_sm100_plan_v1*,
                                             const augur_cuda_nvfp4_sm100_gemv_args_v1*);
using QuantSubmit = augur_cuda_result_v1 (*)(int32_t, augur_cuda_stream_t, const augur_cuda_nvfp4_sm100_act_quant_args_v1*);
using GemmSubmit = augur_cuda_result_v1 (*)(int32_t, augur_cuda_stream_t, augur_cuda_nvfp4_sm100_plan_v1*,
                                             const augur_cuda_nvfp4_sm100_gemm_args_v1*);

enum class StepKind : uint32_t { Nvfp4LinearGemv = 0, Nvfp4LinearGemm = 1 };

// A lowered step: which entry runs it and what it needs, nothing bound yet.
struct CompiledStep {
    StepKind kind;
    QMatmulNode node;
    uint32_t layout;                  // hot layout the weight must be resident in
    GemvSubmit gemv_submit;           // Nvfp4LinearGemv
    QuantSubmit quant_submit;         // Nvfp4LinearGemm: activation quantiser ...
    GemmSubmit gemm_submit;           // ... then the block-scaled GEMM
    uint32_t activation_terms;        // Nvfp4LinearGemm
};

struct WeightRequirement {
    WeightId weight;
    uint32_t layout, rows, cols;
};

struct CompiledPlan {
    std::vector<CompiledStep> steps;
    std::vector<WeightRequirement> weight_requirements;   // one per (weight, layout), in first-use order
    std::vector<uint64_t> buffer_bytes;                     // BF16 activations of every buffer index
    size_t step_count() const { return steps.size(); }
};

// Host-only: no device is touched.
inline CompiledPlan lower(const std::vector<QMatmulNode>& nodes, uint32_t prefill_activation_terms = 3) {
    CompiledPlan plan;
    for (const QMatmulNode& node : nodes) {
        if (node.format != QuantFormat::NVFP4) throw Unsupported("not an NVFP4 weight");
        if (node.block != kNvfp4Block) throw Unsupported("NVFP4 blocks hold 16 elements");
        if (node.version != kNvfp4FormatVersion) throw Unsupported("unknown NVFP4 format version");
        if (!node.rows || !node.cols || !node.tokens) throw Unsupported("empty shape");
        if (node.input_buffer == node.output_buffer) throw Unsupported("a step cannot write the buffer it reads");
        CompiledStep step{};
        step.node = node;
        if (classify_tokens(node.tokens) == BatchClass::SmallBatch) {
            if (node.rows % 32 != 0 || node.cols % 128 != 0) throw Unsupported("small-token kernel: rows % 32, cols % 128");
            step.kind = StepKind::Nvfp4LinearGemv;
            step.layout = AUGUR_NVFP4_SM100_LAYOUT_STREAM;
            step.gemv_submit = &augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1;
        } else {
            if (node.rows % 128 != 0 || node.cols % 64 != 0) throw Unsupported("prefill GEMM: rows % 128, cols % 64");
            if (prefill_activation_terms < 1 || prefill_activation_terms > 3) throw Unsupported("1..3 activation terms");
            step.kind = StepKind::Nvfp4LinearGemm;
            step.layout = AUGUR_NVFP4_SM100_LAYOUT_TCGEN05;
            step.quant_submit = &augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1;
            step.gemm_submit = &augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1;
            step.activation_terms = prefill_activation_terms;
        }
        bool known = false;
        for (const WeightRequirement& r : plan.weight_requirements) {
            if (r.weight == node.weight && r.layout == step.layout) {
                if (r.rows != node.rows || r.cols != node.cols) throw Unsupported("one weight used with two shapes");
                known = true;
            }
        }
        if (!known) plan.weight_requirements.push_back({node.weight, step.layout, node.rows, node.cols});
        const uint32_t highest = node.input_buffer > node.output_buffer ? node.input_buffer : node.output_buffer;
        if (plan.buffer_bytes.size() <= highest) plan.buffer_bytes.resize(highest + 1, 0);
        const uint64_t in_bytes = static_cast<uint64_t>(node.tokens) * node.cols * 2, out_bytes = static_cast<uint64_t>(node.tokens) * node.rows * 2;
        for (const auto& [index, bytes] : {std::pair<uint32_t, uint64_t>{node.input_buffer, in_bytes}, {node.output_buffer, out_bytes}}) {
            if (plan.buffer_bytes[index] && plan.buffer_bytes[index] != bytes) throw Unsupported("a buffer used with two extents");
            plan.buffer_bytes[index] = bytes;
        }
        plan.steps.push_back(step);
    }
    return plan;
}

// Uploaded weights by id and layout: what `bind` resolves the requirements against.
class WeightResources {
public:
    void add(WeightId id, std::shared_ptr<Nvfp4Sm100Weight> weight) { weights_[{id.value, weight->layout()}] = std::move(weight); }
    std::shared_ptr<Nvfp4Sm100Weight> find(WeightId id, uint32_t layout) const {
        const auto it = weights_.find({id.value, layout});
        return it == weights_.end() ? nullptr : it->second;
    }

private:
    std::map<std::pair<uint32_t, uint32_t>, std::shared_ptr<Nvfp4Sm100Weight>> weights_;
};

struct ResourceAccounting {
    size_t unique_weight_count = 0;
    size_t executable_weight_refs = 0;
    uint64_t hot_weight_payload_bytes = 0;
};

struct ExecutionTelemetry {
    size_t step_count = 0;
    double nvfp4_linear_gemv_ms = 0.0;
    double nvfp4_linear_gemm_ms = 0.0;
    double total_ms() const { return nvfp4_linear_gemv_ms + nvfp4_linear_gemm_ms; }
};

// A step with everything bound: the selected entry, its validated descriptor(s) and shared owners of its operands.
class PlannedOp {
public:
    StepKind kind() const { return kind_; }
    const std::shared_ptr<Nvfp4Sm100Weight>& weight() const { return weight_; }
    GemvSubmit gemv_submit() const { return gemv_submit_; }
    GemmSubmit gemm_submit() const { return gemm_submit_; }
    uint32_t input_buffer() const { return input_index_; }
    uint32_t output_buffer() const { return output_index_; }

private:
    friend class ExecutionPlan;
    StepKind kind_ = StepKind::Nvfp4LinearGemv;
    GemvSubmit gemv_submit_ = nullptr;
    QuantSubmit quant_submit_ = nullptr;
    GemmSubmit gemm_submit_ = nullptr;
    augur_cuda_nvfp4_sm100_gemv_args_v1 gemv_args_{};
    augur_cuda_nvfp4_sm100_act_quant_args_v1 quant_args_{};
    augur_cuda_nvfp4_sm100_gemm_args_v1 gemm_args_{};
    std::shared_ptr<Nvfp4Sm100Weight> weight_;
    std::shared_ptr<DeviceBuffer> input_, output_, staged_;
    uint32_t input_index_ = 0, output_index_ = 0;
};

class ExecutionPlan {
public:
    // Resolves weights, allocates buffers and scratch, preflights every step. The only allocating call.
    static std::unique_ptr<ExecutionPlan> bind(const CompiledPlan& compiled, const WeightResources& resources,
                                               const std::shared_ptr<Stream>& stream, float prefill_activation_global_scale = 1.0f / 256.0f) {
        std::unique_ptr<ExecutionPlan> plan(new ExecutionPlan());
        plan->stream_ = stream;
        const int32_t d = stream->ordinal();
        uint64_t scratch = 1 << 20;
        for (const CompiledStep& step : compiled.steps) {
            if (step.kind == StepKind::Nvfp4LinearGemv) {
                uint64_t need = 0;
                check("gemv_scratch_extent", augur_cuda_nvfp4_sm100_gemv_scratch_extent_host_v1(step.node.rows, step.node.cols, step.node.tokens, &need));
                if (need > scratch) scratch = need;
            }
        }
        plan->plan_ = std::make_shared<Plan>(stream, scratch);
        for (uint64_t bytes : compiled.buffer_bytes) plan->buffers_.push_back(std::make_shared<DeviceBuffer>(d, bytes));
        for (const WeightRequirement& r : compiled.weight_requirements) {
            const auto weight = resources.find(r.weight, r.layout);
            if (!weight) throw std::invalid_argument("a weight the plan needs was not uploaded in the layout it needs");
            if (weight->rows() != r.rows || weight->cols() != r.cols) throw std::invalid_argument("uploaded weight has another shape");
            if (weight->stream() != stream) throw std::invalid_argument("plan and weight belong to different streams");
            ++plan->accounting_.unique_weight_count;
            plan->accounting_.hot_weight_payload_bytes += weight->packed()->bytes();
        }
        for (const CompiledStep& step : compiled.steps) {
            PlannedOp op;
            op.kind_ = step.kind;
            op.weight_ = resources.find(step.node.weight, step.layout);
            op.input_ = plan->buffers_[step.node.input_buffer];
            op.output_ = plan->buffers_[step.node.output_buffer];
            op.input_index_ = step.node.input_buffer;
            op.output_index_ = step.node.output_buffer;
            ++plan->accounting_.executable_weight_refs;
            if (step.kind == StepKind::Nvfp4LinearGemv) {
                op.gemv_submit_ = step.gemv_submit;
                op.gemv_args_ = gemv_args(*op.weight_, *op.input_, *op.output_, step.node.tokens, AUGUR_NVFP4_SM100_EPILOGUE_LINEAR_BF16);
                check("gemv_bf16_preflight", augur_cuda_nvfp4_sm100_gemv_bf16_preflight_v1(d, stream->handle(), plan->plan_->raw(), &op.gemv_args_));
            } else {
                op.quant_submit_ = step.quant_submit;
                op.gemm_submit_ = step.gemm_submit;
                uint64_t staged_bytes = 0;
                check("gemm_scratch_extent", augur_cuda_nvfp4_sm100_gemm_scratch_extent_host_v1(step.node.rows, step.node.cols, step.node.tokens,
                                                                                               step.activation_terms, &staged_bytes));
                op.staged_ = std::make_shared<DeviceBuffer>(d, staged_bytes);
                op.quant_args_ = header<augur_cuda_nvfp4_sm100_act_quant_args_v1>();
                op.quant_args_.input_bf16 = op.input_->address();
                op.quant_args_.input_len_bytes = static_cast<uint64_t>(step.node.tokens) * step.node.cols * 2;
                op.quant_args_.destination = op.staged_->address();
                op.quant_args_.destination_len_bytes = staged_bytes;
                op.quant_args_.tokens = step.node.tokens;
                op.quant_args_.cols = step.node.cols;
                op.quant_args_.terms = step.activation_terms;
                op.quant_args_.global_scale = prefill_activation_global_scale;
                op.gemm_args_ = header<augur_cuda_nvfp4_sm100_gemm_args_v1>();
                op.gemm_args_.weight = op.weight_->packed()->address();
                op.gemm_args_.weight_len_bytes = op.weight_->packed()->bytes();
                op.gemm_args_.activation = op.staged_->address();
                op.gemm_args_.activation_len_bytes = staged_bytes;
                op.gemm_args_.output_bf16 = op.output_->address();
                op.gemm_args_.output_len_bytes = static_cast<uint64_t>(step.node.tokens) * step.node.rows * 2;
                op.gemm_args_.rows = step.node.rows;
                op.gemm_args_.cols = step.node.cols;
                op.gemm_args_.tokens = step.node.tokens;
                op.gemm_args_.activation_terms = step.activation_terms;
                op.gemm_args_.weight_global_scale = op.weight_->global_scale();
                op.gemm_args_.activation_global_scale = prefill_activation_global_scale;
                check("act_quant_preflight", augur_cuda_nvfp4_sm100_act_quant_preflight_v1(d, stream->handle(), &op.quant_args_));
                check("gemm_bf16_preflight", augur_cuda_nvfp4_sm100_gemm_bf16_preflight_v1(d, stream->handle(), plan->plan_->raw(), &op.gemm_args_));
            }
            plan->steps_.push_back(std::move(op));
        }
        check_cuda("cudaEventCreate", cudaEventCreate(&plan->started_));
        plan->stamps_.resize(plan->steps_.size());
        for (cudaEvent_t& stamp : plan->stamps_) check_cuda("cudaEventCreate", cudaEventCreate(&stamp));
        return plan;
    }
    ~ExecutionPlan() {
        if (stream_) augur_cuda_nvfp4_sm100_stream_synchronize_v1(stream_->handle());
        if (started_) cudaEventDestroy(started_);
        for (cudaEvent_t stamp : stamps_) cudaEventDestroy(stamp);
    }
    ExecutionPlan(const ExecutionPlan&) = delete;
    ExecutionPlan& operator=(const ExecutionPlan&) = delete;

    const std::vector<PlannedOp>& steps() const { return steps_; }
    const ResourceAccounting& resource_accounting() const { return accounting_; }
    const std::shared_ptr<DeviceBuffer>& buffer(uint32_t index) const { return buffers_.at(index); }
    const std::shared_ptr<Plan>& plan() const { return plan_; }

    void set_input_bf16(uint32_t buffer_index, const uint16_t* values, uint64_t count) {
        if (count * 2 != buffers_.at(buffer_index)->bytes()) throw std::invalid_argument("input extent");
        buffers_[buffer_index]->upload(*stream_, values, count * 2);
    }
    void output_bf16(uint32_t buffer_index, uint16_t* values, uint64_t count) const {
        if (count * 2 != buffers_.at(buffer_index)->bytes()) throw std::invalid_argument("output extent");
        buffers_[buffer_index]->download(*stream_, values, count * 2);
    }

    // Enqueues every step on the plan's stream: no allocation, no synchronisation.
    void submit_steps() const {
        for (const PlannedOp& op : steps_) submit_step(op);
    }
    void execute() const {
        submit_steps();
        stream_->synchronize();
    }
    // The same steps bracketed by CUDA events: device time per step kind.
    ExecutionTelemetry execute_profiled() const {
        ExecutionTelemetry telemetry;
        check_cuda("cudaEventRecord", cudaEventRecord(started_, stream_->raw()));
        for (size_t i = 0; i < steps_.size(); ++i) {
            submit_step(steps_[i]);
            check_cuda("cudaEventRecord", cudaEventRecord(stamps_[i], stream_->raw()));
        }
        stream_->synchronize();
        cudaEvent_t before = started_;
        for (size_t i = 0; i < steps_.size(); ++i) {
            float ms = 0.0f;
            check_cuda("cudaEventElapsedTime", cudaEventElapsedTime(&ms, before, stamps_[i]));
            (steps_[i].kind() == StepKind::Nvfp4LinearGemv ? telemetry.nvfp4_linear_gemv_ms : telemetry.nvfp4_linear_gemm_ms) += ms;
            before = stamps_[i];
            ++telemetry.step_count;
        }
        return telemetry;
    }

private:
    ExecutionPlan() = default;
    void submit_step(const PlannedOp& op) const {
        const int32_t d = stream_->ordinal();
        if (op.kind_ == StepKind::Nvfp4LinearGemv) {
            check("gemv_bf16_submit", op.gemv_submit_(d, stream_->handle(), plan_->raw(), &op.gemv_args_));
        } else {
            check("act_quant_submit", op.quant_submit_(d, stream_->handle(), &op.quant_args_));
            check("gemm_bf16_submit", op.gemm_submit_(d, stream_->handle(), plan_->raw(), &op.gemm_args_));
        }
    }
    std::shared_ptr<Stream> stream_;
    std::shared_ptr<Plan> plan_;
    std::vector<std::shared_ptr<DeviceBuffer>> buffers_;
    std::vector<PlannedOp> steps_;
    ResourceAccounting accounting_;
    cudaEvent_t started_ = nullptr;
    std::vector<cudaEvent_t> stamps_;
};

}  // namespace exec
}  // namespace nvfp4_sm100
}  // namespace augur
