// Identity, stream handles, plan objects and diagnostics of the sm_100a NVFP4 library.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <new>

#include "nvfp4_internal.h"

namespace augur_sm100 {
namespace {
std::atomic<uint32_t> g_injected_faults{0};
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_allocations{0};
std::atomic<uint64_t> g_frees{0};

using cuMemGetAddressRange_fn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

// The driver library is reached through the runtime so that this library loads
// (and its host-only entry points work) on a machine without a driver.
cuMemGetAddressRange_fn address_range_entry() {
    static cuMemGetAddressRange_fn cached = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &query) !=
                cudaSuccess ||
            query != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            fn = nullptr;
        }
        return reinterpret_cast<cuMemGetAddressRange_fn>(fn);
    }();
    return cached;
}

bool device_range(Range r, int32_t ordinal) {
    if (!valid(r) || r.bytes > SIZE_MAX) return false;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, reinterpret_cast<void*>(r.address)) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (attr.type != cudaMemoryTypeDevice || attr.device != ordinal) return false;
    const auto query = address_range_entry();
    if (!query) return false;
    CUdeviceptr base = 0;
    size_t bytes = 0;
    if (query(&base, &bytes, static_cast<CUdeviceptr>(r.address)) != CUDA_SUCCESS || r.address < base) {
        return false;
    }
    const uint64_t offset = r.address - base;
    return offset <= bytes && r.bytes <= bytes - offset;
}
}  // namespace

bool inspect_device_ranges(int32_t ordinal, const Range* ranges, size_t count,
                           augur_cuda_result_v1* failure) {
    const cudaError_t set = cudaSetDevice(ordinal);
    if (set != cudaSuccess) {
        cudaGetLastError();
        *failure = make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, set);
        return false;
    }
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, ordinal) != cudaSuccess) {
        *failure = make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, cudaGetLastError());
        return false;
    }
    if (major != 10) {  // sm_100a code only runs on compute capability 10.x
        *failure = make_result(AUGUR_CUDA_STATUS_UNSUPPORTED_DEVICE);
        return false;
    }
    for (size_t i = 0; i < count; ++i) {
        if (!device_range(ranges[i], ordinal)) {
            *failure = invalid();
            return false;
        }
    }
    return true;
}

bool plan_ok(const augur_cuda_nvfp4_sm100_plan_v1* plan, int32_t ordinal, augur_cuda_stream_t stream) {
    return plan && plan->magic == kPlanMagic && plan->ordinal == ordinal && plan->owner == stream &&
           plan->scratch && plan->scratch_bytes;
}

Range plan_scratch_range(const augur_cuda_nvfp4_sm100_plan_v1* plan) {
    return {reinterpret_cast<uint64_t>(plan->status_word), plan->scratch_bytes + kPlanHeaderBytes + kPlanTrailerBytes, 256};
}

bool consume_injected_fault() {
    uint32_t pending = g_injected_faults.load();
    while (pending > 0) {
        if (g_injected_faults.compare_exchange_weak(pending, pending - 1)) return true;
    }
    return false;
}
void count_launch(uint64_t launches) { g_launches.fetch_add(launches); }
void count_allocation() { g_allocations.fetch_add(1); }
void count_free() { g_frees.fetch_add(1); }

augur_cuda_result_v1 submitted() {
    const cudaError_t e = cudaGetLastError();
    return make_result(e == cudaSuccess ? AUGUR_CUDA_STATUS_OK : AUGUR_CUDA_STATUS_SUBMISSION_FAILURE, e);
}

}  // namespace augur_sm100

using namespace augur_sm100;

extern "C" uint32_t AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_abi_version(void) {
    return AUGUR_CUDA_ABI_VERSION_V1;
}

extern "C" uint32_t AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_build_capability_v1(void) {
#if defined(AUGUR_SM100A_BUILD)
    return 100;
#else
    return 0;
#endif
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_create_v1(
    int32_t ordinal, augur_cuda_stream_t* out_stream) {
    if (ordinal < 0 || !out_stream) return invalid();
    *out_stream = nullptr;
    cudaError_t e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    cudaStream_t raw = nullptr;
    e = cudaStreamCreateWithFlags(&raw, cudaStreamNonBlocking);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    auto* handle = new (std::nothrow) augur_cuda_stream_handle{ordinal, raw, 1, 0};
    if (!handle) {
        cudaStreamDestroy(raw);
        return make_result(AUGUR_CUDA_STATUS_OUT_OF_MEMORY);
    }
    *out_stream = handle;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_adopt_v1(
    int32_t ordinal, void* raw_cuda_stream, augur_cuda_stream_t* out_stream) {
    if (ordinal < 0 || !out_stream) return invalid();
    auto* handle = new (std::nothrow)
        augur_cuda_stream_handle{ordinal, static_cast<cudaStream_t>(raw_cuda_stream), 0, 0};
    if (!handle) return make_result(AUGUR_CUDA_STATUS_OUT_OF_MEMORY);
    *out_stream = handle;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_synchronize_v1(
    augur_cuda_stream_t stream) {
    if (!stream) return invalid();
    cudaError_t e = cudaSetDevice(stream->ordinal);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    e = cudaStreamSynchronize(stream->stream);
    return e == cudaSuccess ? ok() : make_result(AUGUR_CUDA_STATUS_COMPLETION_FAILURE, e);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_stream_destroy_v1(
    augur_cuda_stream_t stream) {
    if (!stream) return invalid();
    // Plans keep a pointer to their owner for the identity check of every call: close them first.
    if (stream->plans != 0) return invalid();
    cudaError_t e = cudaSuccess;
    if (stream->owned) {
        cudaSetDevice(stream->ordinal);
        e = cudaStreamDestroy(stream->stream);
    }
    delete stream;
    return e == cudaSuccess ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_create_v1(
    int32_t ordinal, augur_cuda_stream_t stream, uint64_t scratch_len_bytes,
    augur_cuda_nvfp4_sm100_plan_v1** out_plan) {
    if (!out_plan) return invalid();
    *out_plan = nullptr;
    if (ordinal < 0 || !stream || stream->ordinal != ordinal || scratch_len_bytes == 0 ||
        scratch_len_bytes > (UINT64_C(1) << 40)) {
        return invalid();
    }
    cudaError_t e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal) != cudaSuccess) {
        return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, cudaGetLastError());
    }
    if (major != 10) return make_result(AUGUR_CUDA_STATUS_UNSUPPORTED_DEVICE);
    e = gemv_configure_device();
    if (e == cudaSuccess) e = gemm_configure_device();
    if (e == cudaSuccess) e = gemv_tc_configure_device();
    if (e != cudaSuccess) return make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    const uint64_t rounded = (scratch_len_bytes + 255) / 256 * 256;
    void* memory = nullptr;
    e = cudaMalloc(&memory, rounded + kPlanHeaderBytes + kPlanTrailerBytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return make_result(AUGUR_CUDA_STATUS_OUT_OF_MEMORY, e);
    }
    count_allocation();
    // Arrival counters and the status word must start at zero; kernels leave them at zero.
    e = cudaMemsetAsync(memory, 0, rounded + kPlanHeaderBytes + kPlanTrailerBytes, stream->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream->stream);
    auto* plan = e == cudaSuccess ? new (std::nothrow) augur_cuda_nvfp4_sm100_plan_v1{} : nullptr;
    if (!plan) {
        cudaFree(memory);
        count_free();
        return make_result(e == cudaSuccess ? AUGUR_CUDA_STATUS_OUT_OF_MEMORY : AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
    }
    plan->magic = kPlanMagic;
    plan->ordinal = ordinal;
    plan->owner = stream;
    plan->status_word = static_cast<uint32_t*>(memory);
    plan->scratch = static_cast<uint8_t*>(memory) + kPlanHeaderBytes;
    plan->scratch_bytes = rounded;
    plan->sm_count = static_cast<uint32_t>(sms);
    plan->owner_stream = stream->stream;
    ++stream->plans;
    const uint32_t resident = gemm_pair_resident_clusters();
    plan->pair_clusters = resident && resident < plan->sm_count / 2 ? resident : plan->sm_count / 2;
    *out_plan = plan;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_describe_v1(
    const augur_cuda_nvfp4_sm100_plan_v1* plan, augur_cuda_nvfp4_sm100_plan_snapshot_v1* out) {
    if (!plan || plan->magic != kPlanMagic || !out ||
        out->abi_version != AUGUR_CUDA_ABI_VERSION_V1 || out->struct_size != sizeof(*out)) {
        return invalid();
    }
    out->scratch = reinterpret_cast<uint64_t>(plan->scratch);
    out->scratch_len_bytes = plan->scratch_bytes;
    out->sm_count = plan->sm_count;
    out->reserved = 0;
    return ok();
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_destroy_v1(
    augur_cuda_nvfp4_sm100_plan_v1* plan) {
    if (!plan || plan->magic != kPlanMagic) return invalid();
    cudaSetDevice(plan->ordinal);
    cudaError_t e = cudaStreamSynchronize(plan->owner_stream);
    const cudaError_t freed = cudaFree(plan->status_word);
    count_free();
    if (e == cudaSuccess) e = freed;
    --plan->owner->plans;   // the handle is alive: it cannot be destroyed while this plan exists
    plan->magic = 0;
    delete plan;
    return e == cudaSuccess ? ok() : make_result(AUGUR_CUDA_STATUS_RUNTIME_FAILURE, e);
}

extern "C" augur_cuda_result_v1 AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_plan_device_status_v1(
    augur_cuda_nvfp4_sm100_plan_v1* plan, uint32_t* out_status) {
    if (!plan || plan->magic != kPlanMagic || !out_status) return invalid();
    cudaError_t e = cudaSetDevice(plan->ordinal);
    if (e == cudaSuccess) {
        e = cudaMemcpyAsync(out_status, plan->status_word, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                            plan->owner_stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(plan->owner_stream);
    if (e == cudaSuccess && *out_status != 0) {
        // a wait ran out: the launch left its meeting counters and row maxima (header words 16..63, trailer) half used
        e = cudaMemsetAsync(plan->status_word + 16, 0, (64 - 16) * sizeof(uint32_t), plan->owner_stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(plan->scratch + plan->scratch_bytes, 0, kPlanTrailerBytes, plan->owner_stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(plan->owner_stream);
    }
    return e == cudaSuccess ? ok() : make_result(AUGUR_CUDA_STATUS_COMPLETION_FAILURE, e);
}

extern "C" void AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_diagnostic_inject_submit_fault_v1(uint32_t count) {
    g_injected_faults.store(count);
}

extern "C" void AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_allocation_snapshot_v1(
    uint64_t* out_allocations, uint64_t* out_frees) {
    if (out_allocations) *out_allocations = g_allocations.load();
    if (out_frees) *out_frees = g_frees.load();
}

extern "C" uint64_t AUGUR_CUDA_CALL augur_cuda_nvfp4_sm100_launch_count_v1(void) {
    return g_launches.load();
}
