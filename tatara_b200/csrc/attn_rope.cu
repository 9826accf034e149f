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

// The same operator for BLOCKS of rows (prefill), one position after another.  The decomposition above
// is 18 CTAs of 256 threads per row, each with two block barriers, and every CTA of a row evaluates
// the row's 32 RoPE angles again (a double-precision pow and a sincosf per rotated element): 70 us for 2048
// rows where the 75 MB it moves are 12 us of HBM time.  Here a WARP owns a row: lane l holds dims
// 8l .. 8l+7 of a head (16-byte accesses), the RMS is the reference's tree -- virtual thread t = dims
// 4t .. 4t+3, adjacent pairs first: threads 2l and 2l+1 meet inside the lane, then four xor levels give
// the two 32-thread sums, added last -- and the row's 32 sines and cosines are computed once, one pair
// per lane, and handed to lanes 0..7 by shuffles for all 18 heads.  Same arithmetic per element:
// bit-identical to the kernel above.
constexpr uint32_t kRopeBlockWarps = 8;

__device__ __forceinline__ void unpack_bf16x8(const uint4 raw, float out[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

__global__ void __launch_bounds__(kRopeBlockWarps * 32)
attn_qk_rope_block_kernel(const __nv_bfloat16* __restrict__ projection,
                          const __nv_bfloat16* __restrict__ q_weight,
                          const __nv_bfloat16* __restrict__ k_weight, __nv_bfloat16* __restrict__ q_out,
                          __nv_bfloat16* __restrict__ gate_out, __nv_bfloat16* __restrict__ keys,
                          __nv_bfloat16* __restrict__ values, uint32_t position, uint32_t capacity,
                          uint32_t rows) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = blockIdx.x * kRopeBlockWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint32_t pos = position + row;
    const __nv_bfloat16* proj = projection + uint64_t(row) * kAttnProj;
    // this lane's RoPE pair (pair = lane) of the row
    float sine, cosine;
    sincosf(float(pos) / rope_divisor(lane), &sine, &cosine);
    float wq[8], wk[8];
    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(q_weight + lane * 8u)), wq);
    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(k_weight + lane * 8u)), wk);
    // lanes 0..3 hold dims 0..31 (rotate with dims +32, in lane + 4), lanes 4..7 dims 32..63 (with lane - 4)
    float sin8[8], cos8[8];
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t pair = ((lane & 3u) * 8u + i) & 31u;
        sin8[i] = __shfl_sync(0xffffffffu, sine, pair);
        cos8[i] = __shfl_sync(0xffffffffu, cosine, pair);
    }
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(proj + lane * 8u));   // head 0's q dims
    for (uint32_t head = 0; head < kQHeads + kKvHeads; ++head) {
        const bool is_q = head < kQHeads;
        const uint32_t local = is_q ? head : head - kQHeads;
        // the next head's dims are requested before this head's arithmetic
        uint4 raw_next = raw;
        if (head + 1u < kQHeads + kKvHeads) {
            const uint32_t nh = head + 1u;
            const uint32_t nbase = nh < kQHeads ? nh * 2u * kHeadDim : kAttnKOff + (nh - kQHeads) * kHeadDim;
            raw_next = __ldg(reinterpret_cast<const uint4*>(proj + nbase + lane * 8u));
        }
        // the row that is copied through: the gate of a query head, the values of a key head
        const uint4 through = __ldg(reinterpret_cast<const uint4*>(
            proj + (is_q ? head * 2u * kHeadDim + kHeadDim : kAttnVOff + local * kHeadDim) + lane * 8u));
        float x[8];
        unpack_bf16x8(raw, x);
        float lo = 0.0f, hi = 0.0f;   // virtual threads 2l and 2l+1: four contiguous squares each
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) lo += x[j] * x[j];
#pragma unroll
        for (uint32_t j = 4; j < 8; ++j) hi += x[j] * x[j];
        float acc = lo + hi;          // tree level 1 (threads 2l, 2l+1)
#pragma unroll
        for (int off = 1; off < 16; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);   // levels 2 .. 5 of each 32-thread tree
        const float other = __shfl_xor_sync(0xffffffffu, acc, 16);
        const float s0 = lane < 16u ? acc : other, s1 = lane < 16u ? other : acc;
        const float inverse = 1.0f / sqrtf((s0 + s1) / float(kHeadDim) + kRmsEps);
        float normed[8];
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i)
            normed[i] = bf2f(bmul(f2bf(is_q ? wq[i] : wk[i]), f2bf(x[i] * inverse)));
        __nv_bfloat16 res[8];
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const float partner = __shfl_xor_sync(0xffffffffu, normed[i], 4);   // dim +-32 (used by lanes 0..7 only)
            float rotated = normed[i];
            if (lane < 4u) rotated = fmaf(-partner, sin8[i], normed[i] * cos8[i]);
            else if (lane < 8u) rotated = fmaf(partner, sin8[i], normed[i] * cos8[i]);
            res[i] = f2bf(rotated);
        }
        if (is_q) {
            const uint64_t at = (uint64_t(row) * kQHeads + head) * kHeadDim + lane * 8u;
            *reinterpret_cast<uint4*>(q_out + at) = *reinterpret_cast<const uint4*>(res);
            *reinterpret_cast<uint4*>(gate_out + at) = through;
        } else {
            const uint64_t at = (uint64_t(local) * capacity + pos) * kHeadDim + lane * 8u;
            *reinterpret_cast<uint4*>(keys + at) = *reinterpret_cast<const uint4*>(res);
            *reinterpret_cast<uint4*>(values + at) = through;
        }
        raw = raw_next;
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
    // blocks of rows: a warp per row, 16-byte accesses
    if (rows >= 32u && aligned(projection, 16) && aligned(q_weight, 16) && aligned(k_weight, 16) && aligned(q_out, 16) &&
        aligned(gate_out, 16) && aligned(keys, 16) && aligned(values, 16)) {
        attn_qk_rope_block_kernel<<<(rows + kRopeBlockWarps - 1u) / kRopeBlockWarps, kRopeBlockWarps * 32, 0,
                                    static_cast<cudaStream_t>(stream)>>>(
            static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(q_weight),
            static_cast<const __nv_bfloat16*>(k_weight), static_cast<__nv_bfloat16*>(q_out),
            static_cast<__nv_bfloat16*>(gate_out), static_cast<__nv_bfloat16*>(keys),
            static_cast<__nv_bfloat16*>(values), position, capacity, rows);
        return check_launch(ctx, "attn_qk_rope");
    }
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
