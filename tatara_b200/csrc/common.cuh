// Shared declarations of the tatara_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/tatara_b200.h"

namespace tb {

// Model geometry (reference: tools/generate_kernel_library.py:173-182, 1980-2006).
constexpr uint32_t kQHeads = 16, kKvHeads = 2, kHeadDim = 256, kHeadsPerKv = 8;
constexpr uint32_t kRopePairs = 32;
constexpr float kAttnScale = 0.0625f, kRmsEps = 1e-6f;
constexpr uint32_t kAttnProj = 9216, kAttnKOff = 8192, kAttnVOff = 8704;
constexpr uint32_t kRecordFloats = TATARA_RECORD_FLOATS;
constexpr uint32_t kGdnKeyHeads = 16, kGdnValueHeads = 32, kGdnDim = 128;
constexpr uint32_t kGdnQk = 4096, kGdnV = 4096, kGdnConv = 8192, kGdnKOff = 2048;
constexpr uint32_t kGdnProj = 12352, kGdnZOff = 8192, kGdnBOff = 12288, kGdnAOff = 12320;

constexpr uint32_t kSmCount = 148; // B200; the partition function is pinned to it

// Device-side status word slots (ctx->device_status).
enum : uint32_t { kStatusCode = 0, kStatusDetail = 1, kStatusWords = 4 };
constexpr uint32_t kMergeCounterSlots = 1024;
constexpr size_t kLaneScheduleBytes = 32768;   // holds attn_decode.cu's DecTables
// Default of TATARA_POLICY_DECODE_L2_PREFETCH_KEYS: the most K/V rows per plane that a decode CTA asks
// into L2 beyond its shared-memory ring before its dependency wait (512 bytes per row and plane); the
// kernel asks for a quarter of its item's rows up to this cap.
constexpr uint32_t kDecodeL2PrefetchKeys = 512;

} // namespace tb

struct tatara_ctx {
    int device = 0;
    int sm_count = 0;
    uint32_t* device_status = nullptr; // kStatusWords u32, zero while healthy
    uint32_t* host_status = nullptr;   // pinned mirror
    void* lane_schedule = nullptr;     // device scratch of the calls whose lane tables live in device memory
    uint64_t launches = 0;
    uint32_t decode_l2_prefetch_keys = tb::kDecodeL2PrefetchKeys;   // TATARA_POLICY_DECODE_L2_PREFETCH_KEYS
    uint32_t gdn_chunk_form = 0;                                     // TATARA_POLICY_GDN_CHUNK_FORM
    uint32_t attn_prefill_form = 0;                                  // TATARA_POLICY_ATTN_PREFILL_FORM
    uint32_t gdn_decode_form = 0;                                    // TATARA_POLICY_GDN_DECODE_FORM
    uint32_t decode_fused_merge = 0;                                 // TATARA_POLICY_DECODE_FUSED_MERGE
    uint32_t q4_row_form = 0;                                        // TATARA_POLICY_Q4_ROW_FORM
    uint32_t gdn_step_early_dependents = 0;                          // TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS
    uint32_t* merge_counters = nullptr; // kMergeCounterSlots pairs of u32 in device memory, zero between launches
    uint32_t merge_slot = 0;            // next pair (round robin: calls in flight together use different pairs)
    char error[256] = {0};
};

namespace tb {

tatara_status fail(tatara_ctx* ctx, tatara_status status, const char* what);
tatara_status check_launch(tatara_ctx* ctx, const char* what);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- split-KV partition function -------------------------------------------------------
// Keys per partition for a lane that attends `n` keys.  A pure function of n (and of the
// fixed SM count), so a lane is cut the same way alone or inside any batch.  Work items are
// (kv head, partition): 2 per partition, so 74 partitions give every SM exactly one item of a
// single lane -- one pass over its keys and ONE merge of its four warps at the end (with several
// items per CTA the key stream of an SM stalls at every merge: measured 9 us over the streaming
// time at 65 536 keys with two items per CTA).
__host__ __device__ inline uint32_t partition_keys(uint32_t n) {
    constexpr uint32_t per_wave = kSmCount / kKvHeads; // 74
    if (n <= per_wave * 128u) return 128u;   // short lanes: at least 128 keys per item
    const uint32_t keys = (n + per_wave - 1u) / per_wave;
    return (keys + 15u) & ~15u;
}
__host__ __device__ inline uint32_t partition_count(uint32_t n) {
    const uint32_t p = partition_keys(n);
    return (n + p - 1u) / p;
}

// ---- device helpers -------------------------------------------------------------------
__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16_rn(v); }
// bf16 "eager op" arithmetic of the reference kernels: f32 op, one rounding.
__device__ __forceinline__ __nv_bfloat16 bmul(__nv_bfloat16 a, __nv_bfloat16 b) {
    return f2bf(bf2f(a) * bf2f(b));
}
__device__ __forceinline__ __nv_bfloat16 badd(__nv_bfloat16 a, __nv_bfloat16 b) {
    return f2bf(bf2f(a) + bf2f(b));
}
__device__ __forceinline__ __nv_bfloat16 bsub(__nv_bfloat16 a, __nv_bfloat16 b) {
    return f2bf(bf2f(a) - bf2f(b));
}
__device__ __forceinline__ __nv_bfloat16 bdiv(__nv_bfloat16 a, __nv_bfloat16 b) {
    return f2bf(bf2f(a) / bf2f(b));
}
// Stable-branch sigmoid with per-op bf16 rounding (gdn.metal:76-79).
__device__ __forceinline__ __nv_bfloat16 sigmoid_bf16(__nv_bfloat16 x) {
    const __nv_bfloat16 one = f2bf(1.0f);
    const __nv_bfloat16 e = f2bf(expf(fabsf(bf2f(x))));
    const __nv_bfloat16 low = bdiv(one, badd(one, e));
    return bf2f(x) < 0.0f ? low : bsub(one, low);
}
__device__ __forceinline__ float sigmoid_f32(float x) {
    const float low = 1.0f / (1.0f + expf(fabsf(x)));
    return x < 0.0f ? low : 1.0f - low;
}
// decay = exp(-exp(A_log) * softplus_bf16(a + dt_bias)) (gdn.metal:133-146).
__device__ __forceinline__ float gdn_decay(__nv_bfloat16 a, __nv_bfloat16 dt_bias,
                                           __nv_bfloat16 a_log) {
    const __nv_bfloat16 zero = f2bf(0.0f);
    const __nv_bfloat16 s = badd(a, dt_bias);
    const bool pos = bf2f(s) > 0.0f;
    const __nv_bfloat16 bmax = pos ? s : zero, bmin = pos ? zero : s;
    const __nv_bfloat16 e = f2bf(expf(bf2f(bsub(bmin, bmax))));
    const float one_plus = 1.0f + bf2f(e);
    const __nv_bfloat16 l1p =
        one_plus == 1.0f ? e : f2bf(bf2f(e) * (logf(one_plus) / (one_plus - 1.0f)));
    return expf(-expf(bf2f(a_log)) * bf2f(badd(bmax, l1p)));
}
__device__ __forceinline__ float gdn_beta(__nv_bfloat16 b) { return bf2f(sigmoid_bf16(b)); }

// Adjacent-pairs sum over the 32 lanes of a warp (lane 2i + lane 2i+1 first): the order of
// the reference's pinned simd_sum tree (tools/native/fixture_suite_probe.cpp:40-60).
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

} // namespace tb
