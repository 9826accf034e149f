// Context, status and geometry entry points of the C ABI.
#include "common.cuh"

#include <cstring>

namespace tb {

tatara_status fail(tatara_ctx* ctx, tatara_status status, const char* what) {
    if (ctx != nullptr) {
        std::snprintf(ctx->error, sizeof(ctx->error), "%s: %s", tatara_status_name(status), what);
    }
    return status;
}

tatara_status check_launch(tatara_ctx* ctx, const char* what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        std::snprintf(ctx->error, sizeof(ctx->error), "CudaError: %s: %s", what,
                      cudaGetErrorString(err));
        return TATARA_CUDA_ERROR;
    }
    ++ctx->launches;
    return TATARA_OK;
}

} // namespace tb

extern "C" {

int tatara_abi_version(void) { return 1; }

const char* tatara_status_name(tatara_status status) {
    switch (status) {
    case TATARA_OK: return "None";
    case TATARA_INVALID_BUFFER: return "InvalidBuffer";
    case TATARA_CONTEXT_OUT_OF_RANGE: return "ContextOutOfRange";
    case TATARA_STATE_SLOT_MISMATCH: return "StateSlotMismatch";
    case TATARA_INVALID_STREAM_GROUP: return "InvalidStreamGroup";
    case TATARA_INVALID_DISPATCH_EXTENT: return "InvalidDispatchExtent";
    case TATARA_INVALID_DEVICE: return "InvalidDevice";
    case TATARA_SCRATCH_TOO_SMALL: return "ScratchTooSmall";
    case TATARA_DEVICE_WAIT_TIMEOUT: return "DeviceWaitTimeout";
    case TATARA_CUDA_ERROR: return "CudaError";
    }
    return "Unknown";
}

tatara_status tatara_ctx_create(int device, tatara_ctx** out) {
    if (out == nullptr) return TATARA_INVALID_BUFFER;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        (void)cudaGetLastError();
        return TATARA_INVALID_DEVICE;
    }
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return TATARA_INVALID_DEVICE;
    if (prop.major != 10) return TATARA_INVALID_DEVICE; // sm_100a binaries only
    if (cudaSetDevice(device) != cudaSuccess) return TATARA_INVALID_DEVICE;
    auto* ctx = new tatara_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&ctx->device_status, tb::kStatusWords * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(ctx->device_status, 0, tb::kStatusWords * sizeof(uint32_t)) != cudaSuccess ||
        cudaMallocHost(&ctx->host_status, tb::kStatusWords * sizeof(uint32_t)) != cudaSuccess ||
        cudaMalloc(&ctx->lane_schedule, tb::kLaneScheduleBytes) != cudaSuccess ||
        cudaMalloc(&ctx->merge_counters, tb::kMergeCounterSlots * 2 * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(ctx->merge_counters, 0, tb::kMergeCounterSlots * 2 * sizeof(uint32_t)) != cudaSuccess) {
        (void)cudaGetLastError();
        tatara_ctx_destroy(ctx);
        return TATARA_CUDA_ERROR;
    }
    std::memset(ctx->host_status, 0, tb::kStatusWords * sizeof(uint32_t));
    *out = ctx;
    return TATARA_OK;
}

void tatara_ctx_destroy(tatara_ctx* ctx) {
    if (ctx == nullptr) return;
    if (ctx->device_status != nullptr) cudaFree(ctx->device_status);
    if (ctx->host_status != nullptr) cudaFreeHost(ctx->host_status);
    if (ctx->lane_schedule != nullptr) cudaFree(ctx->lane_schedule);
    if (ctx->merge_counters != nullptr) cudaFree(ctx->merge_counters);
    delete ctx;
}

tatara_status tatara_ctx_sync(tatara_ctx* ctx, void* stream) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemcpyAsync(ctx->host_status, ctx->device_status,
                                      tb::kStatusWords * sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) {
        std::snprintf(ctx->error, sizeof(ctx->error), "CudaError: sync: %s", cudaGetErrorString(err));
        return TATARA_CUDA_ERROR;
    }
    const uint32_t code = ctx->host_status[tb::kStatusCode];
    if (code != 0) {
        std::snprintf(ctx->error, sizeof(ctx->error), "%s: device status detail %u",
                      tatara_status_name(static_cast<tatara_status>(code)),
                      ctx->host_status[tb::kStatusDetail]);
        cudaMemsetAsync(ctx->device_status, 0, tb::kStatusWords * sizeof(uint32_t), s);
        return static_cast<tatara_status>(code);
    }
    return TATARA_OK;
}

const char* tatara_last_error_string(const tatara_ctx* ctx) {
    return ctx == nullptr ? "null context" : ctx->error;
}

uint64_t tatara_ctx_launch_count(const tatara_ctx* ctx) { return ctx == nullptr ? 0 : ctx->launches; }

tatara_status tatara_ctx_set_policy(tatara_ctx* ctx, tatara_policy policy, uint64_t value) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    switch (policy) {
    case TATARA_POLICY_DECODE_L2_PREFETCH_KEYS:
        if (value > TATARA_MAX_CONTEXT) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: prefetch rows");
        ctx->decode_l2_prefetch_keys = static_cast<uint32_t>(value);
        return TATARA_OK;
    case TATARA_POLICY_GDN_CHUNK_FORM:
        if (value > 2) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: chunk form");
        ctx->gdn_chunk_form = static_cast<uint32_t>(value);
        return TATARA_OK;
    case TATARA_POLICY_ATTN_PREFILL_FORM:
        if (value > 1) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: prefill form");
        ctx->attn_prefill_form = static_cast<uint32_t>(value);
        return TATARA_OK;
    case TATARA_POLICY_GDN_DECODE_FORM:
        if (value > 1) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: decode form");
        ctx->gdn_decode_form = static_cast<uint32_t>(value);
        return TATARA_OK;
    case TATARA_POLICY_DECODE_FUSED_MERGE:
        if (value > 1) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: fused merge");
        ctx->decode_fused_merge = static_cast<uint32_t>(value);
        return TATARA_OK;
    case TATARA_POLICY_Q4_ROW_FORM:
        if (value > 1) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: q4 row form");
        ctx->q4_row_form = static_cast<uint32_t>(value);
        return TATARA_OK;
    case TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS:
        if (value > 1) return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: early dependents");
        ctx->gdn_step_early_dependents = static_cast<uint32_t>(value);
        return TATARA_OK;
    }
    return tb::fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "set_policy: unknown policy");
}
uint64_t tatara_ctx_get_policy(const tatara_ctx* ctx, tatara_policy policy) {
    if (ctx == nullptr) return 0;
    switch (policy) {
    case TATARA_POLICY_DECODE_L2_PREFETCH_KEYS: return ctx->decode_l2_prefetch_keys;
    case TATARA_POLICY_GDN_CHUNK_FORM: return ctx->gdn_chunk_form;
    case TATARA_POLICY_ATTN_PREFILL_FORM: return ctx->attn_prefill_form;
    case TATARA_POLICY_GDN_DECODE_FORM: return ctx->gdn_decode_form;
    case TATARA_POLICY_DECODE_FUSED_MERGE: return ctx->decode_fused_merge;
    case TATARA_POLICY_Q4_ROW_FORM: return ctx->q4_row_form;
    case TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS: return ctx->gdn_step_early_dependents;
    }
    return 0;
}

uint32_t tatara_attn_partition_keys(uint32_t n_keys) {
    return n_keys == 0 ? 0 : tb::partition_keys(n_keys);
}
uint32_t tatara_attn_partitions(uint32_t n_keys) {
    return n_keys == 0 ? 0 : tb::partition_count(n_keys);
}

uint64_t tatara_attn_decode_scratch_bytes(uint32_t max_keys, uint32_t lanes) {
    // A lane has ceil(n/128) partitions up to 9472 keys and at most 74 beyond (tb::partition_keys),
    // so 74 bounds every n <= max_keys.
    (void)max_keys;
    const uint32_t worst = 74u;
    return static_cast<uint64_t>(lanes) * worst * tb::kQHeads * tb::kRecordFloats * sizeof(float);
}

} // extern "C"
