// Drives the library through the C++ owner types (include/augur_nvfp4_sm100.hpp) and checks the
// results against the CPU oracle (test infrastructure; linked by tests only).
//
// Shaped after the reference's own backend tests of the retained FFN program
// (crates/augur-backend/src/cuda_qwen35_qpn.rs:690-707): bind once, submit repeatedly, compare
// with the CPU statement, and prove with the allocation snapshot that the hot loop allocates
// nothing.
//
// Exit code 0 and a last line "ok" on success; any check that fails prints a line and exits 1.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "augur_nvfp4_sm100.hpp"
#include "nvfp4_oracle.h"

using namespace augur::nvfp4_sm100;

namespace {
struct Lcg {
    uint64_t state;
    uint32_t next() {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<uint32_t>(state >> 33);
    }
    double uniform() { return (next() & 0xffffff) / double(0x1000000); }
    double normal() {
        double u = uniform(), v = uniform();
        if (u < 1e-12) u = 1e-12;
        return std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586 * v);
    }
};

struct Planes {
    std::vector<uint8_t> codes, scales;
    float global;
};

Planes make_planes(Lcg& rng, size_t rows, size_t cols) {
    Planes p;
    p.codes.resize(rows * cols / 2);
    p.scales.resize(rows * cols / 16);
    for (auto& b : p.codes) b = static_cast<uint8_t>(rng.next());
    for (auto& b : p.scales) b = static_cast<uint8_t>(0x28 + rng.next() % 0x20);   // 2^-4 .. 2^0, all finite and positive
    p.global = 1.0f / 64.0f;
    return p;
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

int failures = 0;
void expect(bool condition, const char* what) {
    if (!condition) {
        std::printf("FAILED: %s\n", what);
        ++failures;
    }
}

// Largest |got - want| relative to max(|want|, 1e-3 * rms(want)).
double rel_error(const std::vector<double>& got, const std::vector<double>& want) {
    double sum = 0.0;
    for (double w : want) sum += w * w;
    const double floor = 1e-3 * std::sqrt(sum / want.size());
    double worst = 0.0;
    for (size_t i = 0; i < want.size(); ++i) {
        const double scale = std::fabs(want[i]) > floor ? std::fabs(want[i]) : floor;
        const double e = std::fabs(got[i] - want[i]) / scale;
        if (e > worst) worst = e;
    }
    return worst;
}
double rms_error(const std::vector<double>& got, const std::vector<double>& want) {
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < want.size(); ++i) {
        num += (got[i] - want[i]) * (got[i] - want[i]);
        den += want[i] * want[i];
    }
    return std::sqrt(num / den);
}
}  // namespace

int main() {
    try {
        expect(augur_cuda_nvfp4_sm100_abi_version() == 1, "abi version");
        expect(augur_cuda_nvfp4_sm100_build_capability_v1() == 100, "library holds sm_100a code");
        Lcg rng{20260101};
        const uint32_t hidden = 512, inter = 1024, tokens = 8;
        const int threads = augur_oracle_max_threads();
        auto stream = std::make_shared<Stream>(0);

        // ---- FFN program, tokens = 8 ----
        Planes gate = make_planes(rng, inter, hidden), up = make_planes(rng, inter, hidden), down = make_planes(rng, hidden, inter);
        std::vector<uint16_t> x(tokens * hidden);
        for (auto& v : x) v = to_bf16(static_cast<float>(rng.normal()));
        const CheckpointNvfp4Matrix gate_m{gate.codes.data(), gate.scales.data(), gate.global};
        const CheckpointNvfp4Matrix up_m{up.codes.data(), up.scales.data(), up.global};
        const CheckpointNvfp4Matrix down_m{down.codes.data(), down.scales.data(), down.global};
        auto gate_up_w = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_STREAM_PAIR, inter, hidden, gate_m, &up_m);
        auto down_w = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_STREAM, hidden, inter, down_m);
        auto plan = std::make_shared<Plan>(stream, mlp_scratch_bytes(hidden, inter));
        auto x_dev = std::make_shared<DeviceBuffer>(0, x.size() * 2);
        auto y_dev = std::make_shared<DeviceBuffer>(0, static_cast<uint64_t>(tokens) * hidden * 2);
        x_dev->upload(*stream, x.data(), x.size() * 2);
        auto program = Nvfp4Sm100FfnProgram::bind(plan, gate_up_w, down_w, x_dev, y_dev, tokens);
        program->submit_for_plan();
        stream->synchronize();
        const auto before = allocation_snapshot();
        const uint64_t launches_before = launch_count();
        for (int i = 0; i < 10; ++i) program->submit_for_plan();
        stream->synchronize();
        expect(allocation_snapshot() == before, "the submit loop allocates nothing");
        expect(launch_count() - launches_before == 20, "two launches per program");
        expect(plan->device_status() == 0, "device status word clean");
        std::vector<uint16_t> y(tokens * hidden), h(tokens * inter);
        y_dev->download(*stream, y.data(), y.size() * 2);
        program->intermediate()->download(*stream, h.data(), h.size() * 2);
        std::vector<double> h64(h.size()), y64(y.size());
        expect(augur_oracle_mlp_f64(gate.codes.data(), gate.scales.data(), gate.global, up.codes.data(), up.scales.data(), up.global,
                                    down.codes.data(), down.scales.data(), down.global, hidden, inter, x.data(), tokens,
                                    h64.data(), y64.data(), threads) == 0, "oracle mlp");
        std::vector<double> got_h(h.size()), got_y(y.size());
        for (size_t i = 0; i < h.size(); ++i) got_h[i] = from_bf16(h[i]);
        for (size_t i = 0; i < y.size(); ++i) got_y[i] = from_bf16(y[i]);
        const double e_h = rel_error(got_h, h64), e_y = rms_error(got_y, y64);
        std::printf("ffn: intermediate max rel err %.3e, output rms err %.3e\n", e_h, e_y);
        expect(e_h <= 2e-2, "SwiGLU intermediate within 2e-2 of the fp64 oracle");
        expect(e_y <= 2e-2, "MLP output within 2e-2 (rms) of the fp64 oracle");

        // ---- one projection, tokens = 3 ----
        {
            const uint32_t t3 = 3;
            auto out = std::make_shared<DeviceBuffer>(0, static_cast<uint64_t>(t3) * hidden * 2);
            auto h_dev = std::make_shared<DeviceBuffer>(0, static_cast<uint64_t>(t3) * inter * 2);
            h_dev->upload(*stream, h.data(), static_cast<uint64_t>(t3) * inter * 2);
            auto linear_plan = std::make_shared<Plan>(stream, gemv_scratch_bytes(hidden, inter, t3));
            auto projection = Nvfp4Sm100Projection::bind(linear_plan, down_w, h_dev, out, t3);
            projection->submit_for_plan();
            std::vector<uint16_t> got(t3 * hidden);
            out->download(*stream, got.data(), got.size() * 2);
            std::vector<double> want(got.size()), have(got.size());
            expect(augur_oracle_linear_f64(down.codes.data(), down.scales.data(), down.global, hidden, inter, h.data(), t3,
                                           want.data(), threads) == 0, "oracle linear");
            for (size_t i = 0; i < got.size(); ++i) have[i] = from_bf16(got[i]);
            const double e = rel_error(have, want);
            std::printf("projection: max rel err %.3e\n", e);
            expect(e <= 2e-2, "projection within 2e-2 of the fp64 oracle");
            // tokens beyond the small-token limit are refused at bind time, before anything runs
            bool refused = false;
            try {
                auto wide_in = std::make_shared<DeviceBuffer>(0, 9ull * inter * 2);
                auto wide_out = std::make_shared<DeviceBuffer>(0, 9ull * hidden * 2);
                Nvfp4Sm100Projection::bind(linear_plan, down_w, wide_in, wide_out, 9);
            } catch (const CudaRuntimeError& error) {
                refused = error.status == AUGUR_CUDA_STATUS_INVALID_ARGUMENT;
            }
            expect(refused, "nine tokens refused with INVALID_ARGUMENT");
            // a plan is only accepted with the stream that created it
            bool wrong_stream = false;
            try {
                auto other = std::make_shared<Stream>(0);
                auto other_plan = std::make_shared<Plan>(other, gemv_scratch_bytes(hidden, inter, t3));
                Nvfp4Sm100Projection::bind(other_plan, down_w, h_dev, out, t3);
            } catch (const std::invalid_argument&) {
                wrong_stream = true;
            }
            expect(wrong_stream, "a plan of another stream is refused");
        }

        // ---- prefill linear, tokens = 128, three activation terms ----
        {
            const uint32_t rows = 256, cols = 512, wide = 128, terms = 3;
            Planes w = make_planes(rng, rows, cols);
            const CheckpointNvfp4Matrix w_m{w.codes.data(), w.scales.data(), w.global};
            auto weight = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, rows, cols, w_m);
            std::vector<uint16_t> a(wide * cols);
            for (auto& v : a) v = to_bf16(static_cast<float>(rng.normal()));
            auto a_dev = std::make_shared<DeviceBuffer>(0, a.size() * 2);
            auto out = std::make_shared<DeviceBuffer>(0, static_cast<uint64_t>(wide) * rows * 2);
            a_dev->upload(*stream, a.data(), a.size() * 2);
            auto gemm_plan = std::make_shared<Plan>(stream, gemm_scratch_bytes(rows, cols, wide, terms) + 256);
            auto linear = Nvfp4Sm100PrefillLinear::bind(gemm_plan, weight, a_dev, out, wide, terms, 1.0f / 256.0f);
            linear->submit_for_plan();
            std::vector<uint16_t> got(wide * rows);
            out->download(*stream, got.data(), got.size() * 2);
            expect(gemm_plan->device_status() == 0, "prefill device status word clean");
            std::vector<double> want(got.size()), have(got.size());
            expect(augur_oracle_linear_f64(w.codes.data(), w.scales.data(), w.global, rows, cols, a.data(), wide, want.data(), threads) == 0,
                   "oracle prefill linear");
            for (size_t i = 0; i < got.size(); ++i) have[i] = from_bf16(got[i]);
            const double e = rms_error(have, want);
            std::printf("prefill: rms err %.3e\n", e);
            expect(e <= 2e-2, "prefill (3 terms) within 2e-2 (rms) of the fp64 oracle");
        }
        // ---- prefill FFN program with the SwiGLU fused into the gate|up GEMM, 200 token rows (ragged last tile) ----
        {
            const uint32_t wide = 200, terms = 3;   // padded to 256: the fused-quantiser path on a pair tile, ragged rows
            std::vector<uint16_t> a(wide * hidden);
            for (auto& v : a) v = to_bf16(static_cast<float>(rng.normal()));
            std::vector<double> h64(static_cast<size_t>(wide) * inter), y64(static_cast<size_t>(wide) * hidden);
            expect(augur_oracle_mlp_f64(gate.codes.data(), gate.scales.data(), gate.global, up.codes.data(), up.scales.data(), up.global,
                                        down.codes.data(), down.scales.data(), down.global, hidden, inter, a.data(), wide,
                                        h64.data(), y64.data(), threads) == 0, "oracle prefill mlp");
            double x_max = 0.0, h_max = 0.0;
            for (uint16_t v : a) x_max = std::fmax(x_max, std::fabs(from_bf16(v)));
            for (double v : h64) h_max = std::fmax(h_max, std::fabs(v));
            float up_scale = 0.0f;
            auto wide_gate_up = upload_gate_up_interleaved(stream, inter, hidden, gate_m, up_m, &up_scale);
            auto wide_down = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, hidden, inter, down_m);
            auto a_dev = std::make_shared<DeviceBuffer>(0, a.size() * 2);
            auto out = std::make_shared<DeviceBuffer>(0, static_cast<uint64_t>(wide) * hidden * 2);
            a_dev->upload(*stream, a.data(), a.size() * 2);
            auto wide_plan = std::make_shared<Plan>(stream, 4096);
            auto ffn = Nvfp4Sm100PrefillFfnProgram::bind(wide_plan, wide_gate_up, up_scale, wide_down, a_dev, out, wide, terms,
                                                         static_cast<float>(x_max / (448.0 * 6.0)),
                                                         static_cast<float>(h_max * 1.05 / (448.0 * 6.0)));
            ffn->submit_for_plan();
            std::vector<uint16_t> got(static_cast<size_t>(wide) * hidden);
            out->download(*stream, got.data(), got.size() * 2);
            expect(wide_plan->device_status() == 0, "prefill FFN device status word clean");
            std::vector<double> have(got.size());
            for (size_t i = 0; i < got.size(); ++i) have[i] = from_bf16(got[i]);
            const double e = rms_error(have, y64);
            std::printf("prefill ffn: rms err %.3e\n", e);
            expect(e <= 2e-2, "prefill FFN within 2e-2 (rms) of the fp64 oracle");
        }
        // ---- the same FFN, 8 token rows, as ONE launch of the tensor-memory kernel on the prefill program's weights ----
        {
            float up_scale = 0.0f;
            auto tc_gate_up = upload_gate_up_interleaved(stream, inter, hidden, gate_m, up_m, &up_scale);
            auto tc_down = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_TCGEN05, hidden, inter, down_m);
            auto tc_plan = std::make_shared<Plan>(stream, mlp_tc_scratch_bytes(hidden, inter));
            auto tc_out = std::make_shared<DeviceBuffer>(0, static_cast<uint64_t>(tokens) * hidden * 2);
            auto tc_program = Nvfp4Sm100TcFfnProgram::bind(tc_plan, tc_gate_up, up_scale, tc_down, x_dev, tc_out, tokens);
            tc_program->submit_for_plan();
            stream->synchronize();
            const auto before_tc = allocation_snapshot();
            const uint64_t launches_tc = launch_count();
            for (int i = 0; i < 10; ++i) tc_program->submit_for_plan();
            stream->synchronize();
            expect(allocation_snapshot() == before_tc, "the tensor-memory submit loop allocates nothing");
            expect(launch_count() - launches_tc == 10, "one launch per program");
            expect(tc_plan->device_status() == 0, "tensor-memory device status word clean");
            std::vector<uint16_t> tc_y(tokens * hidden), tc_h(tokens * inter);
            tc_out->download(*stream, tc_y.data(), tc_y.size() * 2);
            tc_program->intermediate()->download(*stream, tc_h.data(), tc_h.size() * 2);
            std::vector<double> h64(tc_h.size()), y64(tc_y.size()), have_h(tc_h.size()), have_y(tc_y.size());
            expect(augur_oracle_mlp_f64(gate.codes.data(), gate.scales.data(), gate.global, up.codes.data(), up.scales.data(), up.global,
                                        down.codes.data(), down.scales.data(), down.global, hidden, inter, x.data(), tokens,
                                        h64.data(), y64.data(), threads) == 0, "oracle mlp");
            for (size_t i = 0; i < tc_h.size(); ++i) have_h[i] = from_bf16(tc_h[i]);
            for (size_t i = 0; i < tc_y.size(); ++i) have_y[i] = from_bf16(tc_y[i]);
            const double eh = rel_error(have_h, h64), ey = rms_error(have_y, y64);
            std::printf("tensor-memory ffn: h rel err %.3e, y rms err %.3e\n", eh, ey);
            expect(eh <= 2e-2, "tensor-memory FFN intermediate within 2e-2 of the fp64 oracle");
            expect(ey <= 2e-2, "tensor-memory FFN output within 2e-2 (rms) of the fp64 oracle");
        }
        // ---- norm group: residual add -> RMSNorm -> BF16 stage -> two projections, 8 token rows ----
        {
            const uint32_t rows_a = 256, rows_b = 64;
            Planes wa = make_planes(rng, rows_a, hidden), wb = make_planes(rng, rows_b, hidden);
            const CheckpointNvfp4Matrix wa_m{wa.codes.data(), wa.scales.data(), wa.global}, wb_m{wb.codes.data(), wb.scales.data(), wb.global};
            auto weight_a = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_STREAM, rows_a, hidden, wa_m);
            auto weight_b = Nvfp4Sm100Weight::upload_checkpoint_nvfp4(stream, AUGUR_NVFP4_SM100_LAYOUT_STREAM, rows_b, hidden, wb_m);
            std::vector<float> add_a(tokens * hidden), add_b(tokens * hidden), norm_weight(hidden), used(tokens * hidden), want_y(tokens * hidden);
            for (auto& v : add_a) v = static_cast<float>(rng.normal() * 3.0);
            for (auto& v : add_b) v = static_cast<float>(rng.normal());
            for (auto& v : norm_weight) v = static_cast<float>(1.0 + 0.1 * rng.normal());
            std::vector<uint16_t> want_staged(tokens * hidden);
            expect(augur_oracle_rmsnorm_stage(add_a.data(), add_b.data(), used.data(), norm_weight.data(), tokens, hidden, 1e-6f, 1,
                                              want_y.data(), want_staged.data()) == 0, "oracle norm stage");
            auto a_dev = std::make_shared<DeviceBuffer>(0, add_a.size() * 4), b_dev = std::make_shared<DeviceBuffer>(0, add_b.size() * 4);
            auto x_dev32 = std::make_shared<DeviceBuffer>(0, used.size() * 4), w_dev = std::make_shared<DeviceBuffer>(0, norm_weight.size() * 4);
            a_dev->upload(*stream, add_a.data(), add_a.size() * 4);
            b_dev->upload(*stream, add_b.data(), add_b.size() * 4);
            w_dev->upload(*stream, norm_weight.data(), norm_weight.size() * 4);
            auto group_plan = std::make_shared<Plan>(stream, gemv_scratch_bytes(rows_a, hidden, tokens));
            auto group = Nvfp4Sm100NormGroupProgram::bind(group_plan, {weight_a, weight_b}, x_dev32, w_dev, tokens, hidden, 1e-6f, a_dev, b_dev);
            group->submit_for_plan();
            std::vector<float> got_x(used.size()), got_y(want_y.size());
            std::vector<uint16_t> got_staged(want_staged.size());
            x_dev32->download(*stream, got_x.data(), got_x.size() * 4);
            group->normalised()->download(*stream, got_y.data(), got_y.size() * 4);
            group->staged()->download(*stream, got_staged.data(), got_staged.size() * 2);
            expect(std::memcmp(got_x.data(), used.data(), used.size() * 4) == 0, "residual sum bit-exact");
            expect(std::memcmp(got_y.data(), want_y.data(), want_y.size() * 4) == 0, "normalised output bit-exact");
            expect(std::memcmp(got_staged.data(), want_staged.data(), want_staged.size() * 2) == 0, "staged BF16 bit-exact");
            std::vector<uint16_t> out_a(tokens * rows_a);
            group->outputs()[0]->download(*stream, out_a.data(), out_a.size() * 2);
            std::vector<double> want(out_a.size()), have(out_a.size());
            expect(augur_oracle_linear_f64(wa.codes.data(), wa.scales.data(), wa.global, rows_a, hidden, want_staged.data(), tokens,
                                           want.data(), threads) == 0, "oracle group projection");
            for (size_t i = 0; i < out_a.size(); ++i) have[i] = from_bf16(out_a[i]);
            const double e = rel_error(have, want);
            std::printf("norm group: projection max rel err %.3e\n", e);
            expect(e <= 2e-2 && group_plan->device_status() == 0, "norm group projection within 2e-2 of the fp64 oracle");
        }
    } catch (const std::exception& error) {
        std::printf("FAILED: exception: %s\n", error.what());
        return 1;
    }
    if (failures) return 1;
    std::printf("ok\n");
    return 0;
}
