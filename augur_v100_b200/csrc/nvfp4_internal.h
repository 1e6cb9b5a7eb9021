// Private definitions shared by the translation units of the sm_100a NVFP4 library.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <climits>
#include <cmath>
#include <cstdint>

#include "augur_cuda_nvfp4_sm100.h"

// Same private layout as the reference runtime's handle
// (crates/augur-cuda-sys/native/augur_cuda_internal.h:39-42), so handles made by
// either library are interchangeable. `owned` lives past the shared prefix.
struct augur_cuda_stream_handle {
    int32_t ordinal;
    cudaStream_t stream;
    int32_t owned;
    int32_t plans;   // live plans made on this handle; the handle is not destroyed while any exist
};

struct augur_cuda_nvfp4_sm100_plan_v1 {
    uint32_t magic;
    int32_t ordinal;
    augur_cuda_stream_t owner;
    uint8_t* scratch;          // device
    uint64_t scratch_bytes;
    uint32_t* status_word;     // device, 256 bytes reserved in front of scratch
    uint32_t sm_count;
    // Copied from the owner when the plan is made: destroy and status read-back must not dereference a
    // stream handle that its owner may already have closed. `owner` itself only serves the identity check.
    cudaStream_t owner_stream;
    uint32_t pair_clusters;    // two-CTA clusters of the pair GEMM that can be resident at once on this device
};

namespace augur_sm100 {

constexpr uint32_t kPlanMagic = 0x4e56'4634u;  // "NVF4"
constexpr uint64_t kPlanHeaderBytes = 256;     // status word + padding in front of the scratch
constexpr uint64_t kPlanTrailerBytes = 16384;  // behind the scratch, outside what `scratch_bytes` counts: words that only the
                                               // tensor-memory small-token kernel writes (one per CTA, four sets)

struct Range {
    uint64_t address, bytes, alignment;
};

inline bool valid(Range r) {
    return r.address && r.bytes && r.alignment && r.address % r.alignment == 0 &&
           r.bytes <= UINT64_MAX - r.address;
}
inline bool disjoint(Range a, Range b) {
    return valid(a) && valid(b) &&
           (a.address + a.bytes <= b.address || b.address + b.bytes <= a.address);
}
inline bool all_disjoint(const Range* r, size_t count) {
    for (size_t i = 0; i < count; ++i) {
        if (!valid(r[i])) return false;
        for (size_t j = i + 1; j < count; ++j) {
            if (!disjoint(r[i], r[j])) return false;
        }
    }
    return true;
}
// Conservative scalar range of the reference's checked loader
// (crates/augur-cuda-sys/native/augur_qwen35_nvfp4_qpn_sm70.cu:27-28).
inline bool scale_ok(float s) { return std::isfinite(s) && s >= 0x1p-32f && s <= 24.0f; }

template <class T>
inline bool header_ok(int32_t ordinal, augur_cuda_stream_t stream, const T* args) {
    return ordinal >= 0 && stream && stream->ordinal == ordinal && args &&
           args->abi_version == AUGUR_CUDA_ABI_VERSION_V1 && args->struct_size == sizeof(T);
}

inline augur_cuda_result_v1 make_result(augur_cuda_status_t status, cudaError_t raw = cudaSuccess) {
    return {status, static_cast<int32_t>(raw)};
}
inline augur_cuda_result_v1 ok() { return make_result(AUGUR_CUDA_STATUS_OK); }
inline augur_cuda_result_v1 invalid() { return make_result(AUGUR_CUDA_STATUS_INVALID_ARGUMENT); }

// Driver-side inspection used by every preflight: the range must be device memory of
// `ordinal` and lie inside one allocation. Also gates on compute capability 10.x.
bool inspect_device_ranges(int32_t ordinal, const Range* ranges, size_t count,
                           augur_cuda_result_v1* failure);
// Plan scratch layout: two arrival-counter regions (one per member of a two-launch program)
// at fixed offsets, then partial-sum slots. Counters must read zero when a launch starts and
// every launch leaves them at zero; keeping them apart from the slots means no launch of any
// shape can ever leave slot data where another launch expects counters.
constexpr uint32_t kMaxGroups = 16384;
constexpr uint64_t kCounterRegionBytes = static_cast<uint64_t>(kMaxGroups) * 4;
constexpr uint64_t kCounterBytes = 2 * kCounterRegionBytes;

bool plan_ok(const augur_cuda_nvfp4_sm100_plan_v1* plan, int32_t ordinal, augur_cuda_stream_t stream);
Range plan_scratch_range(const augur_cuda_nvfp4_sm100_plan_v1* plan);

// Diagnostics shared by all entry points.
bool consume_injected_fault();
void count_launch(uint64_t launches = 1);
void count_allocation();
void count_free();
augur_cuda_result_v1 submitted();  // maps cudaGetLastError to SUBMISSION_FAILURE

// One-time per-device kernel attribute setup, called from plan creation (bind time).
cudaError_t gemv_configure_device();
cudaError_t gemm_configure_device();
cudaError_t gemv_tc_configure_device();
// Two-CTA clusters of the pair GEMM that the device can hold at once (0 if the query fails).
uint32_t gemm_pair_resident_clusters();

}  // namespace augur_sm100
