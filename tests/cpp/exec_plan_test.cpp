// The execution-plan layer (include/augur_nvfp4_sm100_exec.hpp), tested in the shape of the reference's own
// execution-plan test of a quantised mat-mul node (crates/augur-compiler/tests/m47_mxfp4_execution_plan.rs):
// lowering selects the expected entry (checked by address), binding accounts for the weights, eight executions
// give the oracle's answer with the same weight owner and payload address every time, profiling reports device
// time per step kind, and nodes this backend does not run are rejected as unsupported.
//
//   exec_plan_test --cpu   lowering only: touches no device
//   exec_plan_test         the whole test on device 0; the CPU oracle (test infrastructure) is the checker
//
// Exit code 0 and a last line "ok" on success; any check that fails prints a line and exits 1.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "augur_nvfp4_sm100_exec.hpp"
#include "nvfp4_oracle.h"

using namespace augur::nvfp4_sm100;
using namespace augur::nvfp4_sm100::exec;

namespace {
int failures = 0;
void expect(bool condition, const char* what) {
    if (!condition) {
        std::printf("FAILED: %s\n", what);
        ++failures;
    }
}
template <class Call>
bool unsupported(Call call) {
    try {
        call();
    } catch (const Unsupported&) {
        return true;
    }
    return false;
}

constexpr uint32_t kRows = 64, kCols = 256;

// the reference test's generators, adapted to 16-element blocks and E4M3 scales
std::vector<uint8_t> codes(size_t rows, size_t cols) {
    std::vector<uint8_t> out(rows * cols / 2);
    for (size_t i = 0; i < out.size(); ++i) {
        const size_t block = i / 8, lane = i % 8;
        const uint8_t low = (block * 3 + lane * 5) & 0x0f, high = 15 - ((block * 7 + lane * 11) & 0x0f);
        out[i] = static_cast<uint8_t>(low | (high << 4));
    }
    return out;
}
std::vector<uint8_t> scales(size_t rows, size_t cols) {
    std::vector<uint8_t> out(rows * cols / 16);
    for (size_t i = 0; i < out.size(); ++i) out[i] = static_cast<uint8_t>(0x30 + i % 8);
    return out;
}
uint16_t to_bf16(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    bits += 0x7fff + ((bits >> 16) & 1);
    return static_cast<uint16_t>(bits >> 16);
}
double from_bf16(uint16_t bits) {
    const uint32_t wide = static_cast<uint32_t>(bits) << 16;
    float value;
    std::memcpy(&value, &wide, 4);
    return value;
}
std::vector<uint16_t> activation(size_t tokens, size_t cols) {
    std::vector<uint16_t> out(tokens * cols);
    for (size_t i = 0; i < out.size(); ++i) out[i] = to_bf16((static_cast<float>((i * 17) % 97) - 48.0f) / 32.0f);
    return out;
}
QMatmulNode node(uint32_t tokens, uint32_t rows = kRows, uint32_t cols = kCols) {
    return QMatmulNode{WeightId{7}, QuantFormat::NVFP4, 16, 1, rows, cols, tokens, 0, 1};
}

void lowering_checks() {
    // the verify batch: one step, the small-token entry, one weight in the stream layout
    const CompiledPlan small = lower({node(8)});
    expect(small.step_count() == 1 && small.steps[0].kind == StepKind::Nvfp4LinearGemv, "8 token rows lower to the small-token step");
    expect(small.steps[0].gemv_submit == &augur_cuda_nvfp4_sm100_gemv_bf16_prevalidated_submit_v1, "selected entry is the small-token submit");
    expect(small.weight_requirements.size() == 1 && small.weight_requirements[0].layout == AUGUR_NVFP4_SM100_LAYOUT_STREAM, "one weight, stream layout");
    expect(small.buffer_bytes.size() == 2 && small.buffer_bytes[0] == 8 * kCols * 2 && small.buffer_bytes[1] == 8 * kRows * 2, "buffer extents");
    // a prefill node: quantiser + GEMM on the tcgen05 layout
    const CompiledPlan wide = lower({node(512, 256, 256)});
    expect(wide.steps[0].kind == StepKind::Nvfp4LinearGemm, "512 token rows lower to the GEMM step");
    expect(wide.steps[0].gemm_submit == &augur_cuda_nvfp4_sm100_gemm_bf16_prevalidated_submit_v1 &&
               wide.steps[0].quant_submit == &augur_cuda_nvfp4_sm100_act_quant_prevalidated_submit_v1, "selected entries are quantiser and GEMM");
    expect(wide.weight_requirements[0].layout == AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, "tcgen05 layout");
    // one weight used twice is one requirement
    QMatmulNode again = node(8);
    again.input_buffer = 2;
    again.output_buffer = 3;
    expect(lower({node(8), again}).weight_requirements.size() == 1, "a shared weight is required once");
    // what this backend does not run (the reference rejects prefill shape, wrong block and wrong version the same way)
    QMatmulNode bad = node(8);
    bad.format = QuantFormat::MXFP4;
    expect(unsupported([&] { lower({bad}); }), "another format is unsupported");
    bad = node(8);
    bad.block = 32;
    expect(unsupported([&] { lower({bad}); }), "another block size is unsupported");
    bad = node(8);
    bad.version = 2;
    expect(unsupported([&] { lower({bad}); }), "another format version is unsupported");
    expect(unsupported([&] { lower({node(8, 8, 256)}); }), "8 weight rows are unsupported (the reference's toy shape)");
    expect(unsupported([&] { lower({node(8, 64, 200)}); }), "cols not a multiple of 128 are unsupported");
    expect(unsupported([&] { lower({node(512, 64, 256)}); }), "prefill rows not a multiple of 128 are unsupported");
    bad = node(8);
    bad.output_buffer = bad.input_buffer;
    expect(unsupported([&] { lower({bad}); }), "in-place steps are unsupported");
    expect(unsupported([&] { lower({node(8), node(8, 128, 256)}); }), "one weight with two shapes is unsupported");
    expect(unsupported([&] { lower({node(0)}); }), "no token rows are unsupported");
}

void device_checks() {
    auto stream = std::make_shared<Stream>(0);
    const std::vector<uint8_t> c = codes(kRows, kCols), s = scales(kRows, kCols);
    const float global = 0.125f;
    const CheckpointNvfp4Matrix matrix{c.data(), s.data(), global};
    WeightResources resources;
    resources.add(WeightId{7}, Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_STREAM, kRows, kCols, matrix));
    const CompiledPlan compiled = lower({node(8)});
    auto plan = ExecutionPlan::bind(compiled, resources, stream);
    expect(plan->resource_accounting().unique_weight_count == 1 && plan->resource_accounting().executable_weight_refs == 1, "one weight, one reference");
    expect(plan->resource_accounting().hot_weight_payload_bytes == static_cast<uint64_t>(kRows) * kCols * 9 / 16, "hot payload bytes");
    const PlannedOp& op = plan->steps()[0];
    expect(op.kind() == StepKind::Nvfp4LinearGemv && op.gemv_submit() == compiled.steps[0].gemv_submit, "the planned step runs the compiled entry");

    const std::vector<uint16_t> x = activation(8, kCols);
    std::vector<double> want(8 * kRows);
    expect(augur_oracle_linear_f64(c.data(), s.data(), global, kRows, kCols, x.data(), 8, want.data(), 2) == 0, "oracle");
    plan->set_input_bf16(op.input_buffer(), x.data(), x.size());
    const Nvfp4Sm100Weight* owner = op.weight().get();
    const uint64_t payload = op.weight()->packed()->address();
    std::vector<uint16_t> first, got(8 * kRows);
    const auto before = allocation_snapshot();
    for (int round = 0; round < 8; ++round) {
        plan->execute();
        plan->output_bf16(op.output_buffer(), got.data(), got.size());
        if (round == 0) first = got;
        expect(got == first, "every execution gives the same bits");
        expect(op.weight().get() == owner && op.weight()->packed()->address() == payload, "weight owner and payload stay put");
    }
    expect(allocation_snapshot() == before, "executing allocates nothing");
    double worst = 0.0, sum = 0.0;
    for (double w : want) sum += w * w;
    const double floor = 1e-3 * std::sqrt(sum / want.size());
    for (size_t i = 0; i < want.size(); ++i) {
        const double scale = std::fabs(want[i]) > floor ? std::fabs(want[i]) : floor;
        worst = std::fmax(worst, std::fabs(from_bf16(got[i]) - want[i]) / scale);
    }
    std::printf("small-token step: max rel err %.3e\n", worst);
    expect(worst <= 2e-2, "within 2e-2 of the fp64 oracle");
    const ExecutionTelemetry telemetry = plan->execute_profiled();
    expect(telemetry.step_count == 1 && telemetry.nvfp4_linear_gemv_ms > 0.0 && telemetry.total_ms() == telemetry.nvfp4_linear_gemv_ms,
           "profiling reports the one step's device time under its kind");
    expect(plan->plan()->device_status() == 0, "device status word clean");

    // two kinds in one plan: the verify batch and a prefill node on another weight
    const uint32_t wide_rows = 256, wide_cols = 256, wide_tokens = 200;
    const std::vector<uint8_t> wc = codes(wide_rows, wide_cols), ws = scales(wide_rows, wide_cols);
    const CheckpointNvfp4Matrix wide_matrix{wc.data(), ws.data(), global};
    resources.add(WeightId{9}, Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, wide_rows, wide_cols, wide_matrix));
    QMatmulNode wide{WeightId{9}, QuantFormat::NVFP4, 16, 1, wide_rows, wide_cols, wide_tokens, 2, 3};
    auto both = ExecutionPlan::bind(lower({node(8), wide}), resources, stream);
    expect(both->resource_accounting().unique_weight_count == 2, "two weights");
    both->set_input_bf16(0, x.data(), x.size());
    const std::vector<uint16_t> wide_x = activation(wide_tokens, wide_cols);
    both->set_input_bf16(2, wide_x.data(), wide_x.size());
    const ExecutionTelemetry mixed = both->execute_profiled();
    expect(mixed.step_count == 2 && mixed.nvfp4_linear_gemv_ms > 0.0 && mixed.nvfp4_linear_gemm_ms > 0.0, "both kinds are timed");
    std::vector<uint16_t> wide_got(wide_tokens * wide_rows);
    both->output_bf16(3, wide_got.data(), wide_got.size());
    std::vector<double> wide_want(wide_got.size());
    expect(augur_oracle_linear_f64(wc.data(), ws.data(), global, wide_rows, wide_cols, wide_x.data(), wide_tokens, wide_want.data(), 2) == 0, "oracle");
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < wide_want.size(); ++i) {
        num += (from_bf16(wide_got[i]) - wide_want[i]) * (from_bf16(wide_got[i]) - wide_want[i]);
        den += wide_want[i] * wide_want[i];
    }
    std::printf("prefill step (three activation terms): rms err %.3e\n", std::sqrt(num / den));
    expect(std::sqrt(num / den) <= 2e-2, "prefill step within 2e-2 (rms) of the BF16-activation oracle");

    // a requirement that was never uploaded
    bool refused = false;
    try {
        ExecutionPlan::bind(lower({QMatmulNode{WeightId{11}, QuantFormat::NVFP4, 16, 1, kRows, kCols, 8, 0, 1}}), resources, stream);
    } catch (const std::invalid_argument&) {
        refused = true;
    }
    expect(refused, "binding without the weight is refused");
}
}  // namespace

int main(int argc, char** argv) {
    const bool cpu_only = argc > 1 && std::strcmp(argv[1], "--cpu") == 0;
    try {
        lowering_checks();
        if (!cpu_only) device_checks();
    } catch (const std::exception& error) {
        std::printf("FAILED: exception: %s\n", error.what());
        return 1;
    }
    if (failures) return 1;
    std::printf("ok\n");
    return 0;
}
