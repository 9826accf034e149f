// q/k RMSNorm + partial RoPE + KV append (reference: attention.metal:43-198,
// prefill_attention.metal:1-92).  One CTA of 256 threads per (head, row); 18 heads per row
// (16 query + 2 key).  Memory-bound and tiny next to the attention kernels; the arithmetic
// keeps the reference's rounding points so results agree to the bf16 bit almost everywhere.
#include "common.cuh"

namespace tb {

// Lane table passed by value as a kernel parameter; N = 1 for the single-lane entry points.
template <uint32_t N>
struct RopeLanes {
    tatara_attn_lane lane[N];
};

// RoPE divisors base^(pair/32), evaluated in double and rounded once to f32.
__device__ __forceinline__ float rope_divisor(uint32_t pair) {
    return static_cast<float>(pow(1.0e7, static_cast<double>(pair) / 32.0));
}

template <uint32_t N>
__global__ void __launch_bounds__(256)
attn_qk_rope_kernel(const __nv_bfloat16* __restrict__ projection,
                    const __nv_bfloat16* __restrict__ q_weight,
                    const __nv_bfloat16* __restrict__ k_weight, __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ gate_out, __nv_bfloat16* __restrict__ keys,
                    __nv_bfloat16* __restrict__ values, uint32_t position, uint32_t capacity,
                    uint64_t projection_stride, uint64_t query_stride,
                    const __grid_constant__ RopeLanes<N> lanes, const tatara_attn_lane* lanes_device) {
    constexpr bool kBatched = N > 1;
    __shared__ float normed[kHeadDim];
    __shared__ float stage[2];
    // A kernel queued behind this one with programmatic serialization may be staged already --
    // but only when each lane appends ONE row: the decode kernel then reads, before its own
    // dependency wait, nothing but partitions that cannot hold that row.  A block of rows
    // (prefill) keeps plain stream order.
    if (kBatched || gridDim.y == 1u) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
    uint32_t pos = position + row;
    uint64_t kv_offset = 0;
    if (kBatched) {
        // the lane table of this call, or the one kept in device memory (CUDA-graph replay)
        const tatara_attn_lane l = lanes_device != nullptr ? lanes_device[row] : lanes.lane[row];
        pos = l.context;
        kv_offset = l.kv_offset;
        if (pos >= capacity) return;   // device table only: the decode setup kernel latches the status
    }
    const __nv_bfloat16* proj = projection + row * projection_stride;
    const bool is_q = head < kQHeads;
    const uint32_t local = is_q ? head : head - kQHeads;
    const uint32_t base = is_q ? head * 2u * kHeadDim : kAttnKOff + local * kHeadDim;
    const float x = bf2f(proj[base + d]);
    // 64 threads x 4 contiguous squares, one adjacent-pairs tree per warp, then s0 + s1.
    if (d < 64u) {
        float acc = 0.0f;
#pragma unroll
        for (uint32_t j = 0; j < 4u; ++j) {
            const float v = bf2f(proj[base + d * 4u + j]);
            acc += v * v;
        }
        acc = warp_sum(acc);
        if ((d & 31u) == 0u) stage[d >> 5u] = acc;
    }
    __syncthreads();
    const float inverse = 1.0f / sqrtf((stage[0] + stage[1]) / float(kHeadDim) + kRmsEps);
    const __nv_bfloat16 w = is_q ? q_weight[d] : k_weight[d];
    normed[d] = bf2f(bmul(w, f2bf(x * inverse)));
    __syncthreads();
    float rotated = normed[d];
    if (d < 2u * kRopePairs) {
        const uint32_t pair = d & 31u;
        const float theta = float(pos) / rope_divisor(pair);
        float sine, cosine;
        sincosf(theta, &sine, &cosine);
        rotated = d < 32u ? fmaf(-normed[d + 32u], sine, normed[d] * cosine)
                          : fmaf(normed[d - 32u], sine, normed[d] * cosine);
    }
    if (is_q) {
        const uint64_t at = row * query_stride + head * kHeadDim + d;
        q_out[at] = f2bf(rotated);
        gate_out[at] = proj[head * 2u * kHeadDim + kHeadDim + d];
    } else {
        const uint64_t at = kv_offset + (uint64_t(local) * capacity + pos) * kHeadDim + d;
        keys[at] = f2bf(rotated);
        values[at] = proj[kAttnVOff + local * kHeadDim + d];
    }
}

} // namespace tb

using namespace tb;

extern "C" tatara_status tatara_attn_qk_rope(tatara_ctx* ctx, void* stream, const void* projection,
                                             const void* q_weight, const void* k_weight,
                                             void* q_out, void* gate_out, void* keys, void* values,
                                             uint32_t position, uint32_t capacity, uint32_t rows) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !q_weight || !k_weight || !q_out || !gate_out || !keys || !values)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_qk_rope: null buffer");
    if (rows == 0 || rows > 65535u) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_qk_rope: rows");
    if (capacity == 0 || uint64_t(position) + rows > capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_qk_rope: position + rows > capacity");
    const RopeLanes<1> none{};
    attn_qk_rope_kernel<1><<<dim3(kQHeads + kKvHeads, rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(q_weight),
        static_cast<const __nv_bfloat16*>(k_weight), static_cast<__nv_bfloat16*>(q_out),
        static_cast<__nv_bfloat16*>(gate_out), static_cast<__nv_bfloat16*>(keys),
        static_cast<__nv_bfloat16*>(values), position, capacity, kAttnProj, kQHeads * kHeadDim, none, nullptr);
    return check_launch(ctx, "attn_qk_rope");
}

extern "C" tatara_status tatara_attn_qk_rope_batch(tatara_ctx* ctx, void* stream,
                                                   const void* projection, const void* q_weight,
                                                   const void* k_weight, void* q_out, void* gate_out,
                                                   void* keys_pool, void* values_pool,
                                                   uint32_t capacity, const tatara_attn_lane* lanes,
                                                   uint32_t n_lanes, uint32_t projection_stride,
                                                   uint32_t query_stride) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !q_weight || !k_weight || !q_out || !gate_out || !keys_pool || !values_pool || !lanes)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_qk_rope_batch: null buffer");
    if (n_lanes == 0 || n_lanes > TATARA_MAX_LANES)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_qk_rope_batch: lane count");
    if (projection_stride < kAttnProj || query_stride < kQHeads * kHeadDim)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_qk_rope_batch: stride");
    RopeLanes<TATARA_MAX_LANES> table{};
    for (uint32_t i = 0; i < n_lanes; ++i) {
        if (capacity == 0 || lanes[i].context >= capacity)
            return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_qk_rope_batch: context >= capacity");
        table.lane[i] = lanes[i];
    }
    attn_qk_rope_kernel<TATARA_MAX_LANES><<<dim3(kQHeads + kKvHeads, n_lanes), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(q_weight),
        static_cast<const __nv_bfloat16*>(k_weight), static_cast<__nv_bfloat16*>(q_out),
        static_cast<__nv_bfloat16*>(gate_out), static_cast<__nv_bfloat16*>(keys_pool),
        static_cast<__nv_bfloat16*>(values_pool), 0u, capacity, projection_stride, query_stride, table, nullptr);
    return check_launch(ctx, "attn_qk_rope_batch");
}

extern "C" tatara_status tatara_attn_qk_rope_batch_indirect(tatara_ctx* ctx, void* stream, const void* projection,
                                                            const void* q_weight, const void* k_weight, void* q_out,
                                                            void* gate_out, void* keys_pool, void* values_pool,
                                                            uint32_t capacity, const tatara_attn_lane* lanes_device,
                                                            uint32_t n_lanes, uint32_t projection_stride,
                                                            uint32_t query_stride) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !q_weight || !k_weight || !q_out || !gate_out || !keys_pool || !values_pool || !lanes_device)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_qk_rope_batch_indirect: null buffer");
    if (n_lanes == 0 || n_lanes > TATARA_MAX_LANES)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_qk_rope_batch_indirect: lane count");
    if (capacity == 0) return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_qk_rope_batch_indirect: capacity");
    if (projection_stride < kAttnProj || query_stride < kQHeads * kHeadDim)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_qk_rope_batch_indirect: stride");
    const RopeLanes<TATARA_MAX_LANES> unused{};
    attn_qk_rope_kernel<TATARA_MAX_LANES><<<dim3(kQHeads + kKvHeads, n_lanes), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(q_weight),
        static_cast<const __nv_bfloat16*>(k_weight), static_cast<__nv_bfloat16*>(q_out),
        static_cast<__nv_bfloat16*>(gate_out), static_cast<__nv_bfloat16*>(keys_pool),
        static_cast<__nv_bfloat16*>(values_pool), 0u, capacity, projection_stride, query_stride, unused, lanes_device);
    return check_launch(ctx, "attn_qk_rope_batch_indirect");
}
