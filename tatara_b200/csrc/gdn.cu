// Gated DeltaNet decode-side operators (reference: gdn.metal:48-207, 231-378;
// prefill_gdn.metal:4-135, 283-320).
//
// The recurrent state is f32 [32 v-head][128 v-dim][128 k-dim] = 2 MiB per lane and layer; a
// decode step reads and rewrites all of it, so the step is HBM-bound.  Each warp owns whole
// state rows: a lane holds 4 contiguous k-dim elements (one coalesced 512-byte float4 row per
// warp), four rows are in flight per warp, and the two dot products per row are
// adjacent-pairs shuffle trees -- the reference's reduction order.
#include "tc05.cuh"

namespace tb {

// ---- conv + SiLU + q/k normalisation -----------------------------------------------------
// One activated conv channel: 4-tap causal conv (f32), bf16, SiLU with per-op bf16 rounding
// (gdn.metal:66-80).  Position `row` of a block taps the logical sequence
// [3 state rows | projection rows] at row..row+3 (prefill_gdn.metal:24-32).
// The loads of one conv channel (the four taps and its weights) and, separately, its arithmetic:
// a caller with several channels requests all of them before using any.
__device__ __forceinline__ void conv_channel_load(const __nv_bfloat16* projection, uint64_t projection_stride,
                                                  const __nv_bfloat16* conv_state,
                                                  const __nv_bfloat16* conv_weights, uint32_t row,
                                                  uint32_t channel, float taps[4], uint2& wraw) {
#pragma unroll
    for (uint32_t t = 0; t < 4; ++t) {
        const uint32_t logical = row + t;
        taps[t] = logical < 3u ? bf2f(conv_state[logical * kGdnConv + channel])
                               : bf2f(projection[uint64_t(logical - 3u) * projection_stride + channel]);
    }
    wraw = *reinterpret_cast<const uint2*>(conv_weights + uint64_t(channel) * 4u);
}
// (the four tap weights as floats: a caller that walks many rows converts them once)
__device__ __forceinline__ __nv_bfloat16 conv_channel_apply_w(const float taps[4], const float w[4]) {
    float acc = __fmul_rn(w[0], taps[0]);
    acc = __fadd_rn(acc, __fmul_rn(w[1], taps[1]));
    acc = __fadd_rn(acc, __fmul_rn(w[2], taps[2]));
    acc = __fadd_rn(acc, __fmul_rn(w[3], taps[3]));
    const __nv_bfloat16 c = f2bf(acc);
    return bmul(c, sigmoid_bf16(c));
}
__device__ __forceinline__ __nv_bfloat16 conv_channel_apply(const float taps[4], uint2 wraw) {
    const float w[4] = {__uint_as_float(wraw.x << 16), __uint_as_float(wraw.x & 0xFFFF0000u),
                        __uint_as_float(wraw.y << 16), __uint_as_float(wraw.y & 0xFFFF0000u)};
    return conv_channel_apply_w(taps, w);
}
__device__ __forceinline__ __nv_bfloat16 conv_channel(const __nv_bfloat16* projection,
                                                      uint64_t projection_stride,
                                                      const __nv_bfloat16* conv_state,
                                                      const __nv_bfloat16* conv_weights,
                                                      uint32_t row, uint32_t channel, float taps[4]) {
    uint2 wraw;
    conv_channel_load(projection, projection_stride, conv_state, conv_weights, row, channel, taps, wraw);
    return conv_channel_apply(taps, wraw);
}

// l2-normalise one 128-channel head held one channel per thread of a 128-thread group:
// 32 lanes x 4 contiguous squares, adjacent-pairs tree (gdn.metal:84-104).
__device__ __forceinline__ __nv_bfloat16 head_normalise(float* head_smem, uint32_t lane128,
                                                        float activated, bool is_query) {
    head_smem[lane128] = activated;
    __syncthreads();
    float acc = 0.0f;
    const uint32_t l = lane128 & 31u;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const float v = head_smem[l * 4u + i];
        acc += v * v;
    }
    acc = warp_sum(acc);
    const float inverse = 1.0f / sqrtf(acc / float(kGdnDim) + kRmsEps);
    const __nv_bfloat16 scale = is_query ? f2bf(1.0f / 128.0f) : f2bf(0.08838834764831845f);
    return bmul(f2bf(activated * inverse), scale);
}

// grid (96, rows) x 128 threads, exactly the reference's decomposition.  kTape: the conv tail
// (the three newest taps) is also recorded after EVERY row, conv_tape [layer][16][3][8192], so a
// rollback can restore it at any row (gdn_conv_tape_blk, prefill_gdn.metal:322-420).
template <bool kTape>
__global__ void __launch_bounds__(128)
gdn_prepare_kernel(const __nv_bfloat16* __restrict__ projection,
                   const __nv_bfloat16* __restrict__ conv_state,
                   const __nv_bfloat16* __restrict__ conv_weights, __nv_bfloat16* __restrict__ qk,
                   __nv_bfloat16* __restrict__ value, __nv_bfloat16* __restrict__ z,
                   __nv_bfloat16* __restrict__ new_conv_state, uint32_t rows,
                   __nv_bfloat16* __restrict__ conv_tape, uint32_t tape_layer) {
    __shared__ float head_smem[kGdnDim];
    const uint32_t group = blockIdx.x, row = blockIdx.y, lane = threadIdx.x;
    if (group < kGdnConv / kGdnDim) {
        const uint32_t channel = group * kGdnDim + lane;
        float taps[4];
        const __nv_bfloat16 act = conv_channel(projection, kGdnProj, conv_state, conv_weights, row, channel, taps);
        if (row + 1u == rows) {
#pragma unroll
            for (uint32_t t = 0; t < 3; ++t) new_conv_state[t * kGdnConv + channel] = f2bf(taps[t + 1u]);
        }
        if (kTape) {
#pragma unroll
            for (uint32_t t = 0; t < 3; ++t)
                conv_tape[((uint64_t(tape_layer) * 16u + row) * 3u + t) * kGdnConv + channel] = f2bf(taps[t + 1u]);
        }
        if (group < kGdnQk / kGdnDim) {
            qk[uint64_t(row) * kGdnQk + channel] =
                head_normalise(head_smem, lane, bf2f(act), group < kGdnKeyHeads);
        } else {
            value[uint64_t(row) * kGdnV + channel - kGdnQk] = act;
        }
    } else {
        const uint32_t index = (group - kGdnConv / kGdnDim) * kGdnDim + lane;
        z[uint64_t(row) * kGdnV + index] = projection[uint64_t(row) * kGdnProj + kGdnZOff + index];
    }
}

// The same operator for BLOCKS of rows (prefill).  The decomposition above launches one 128-thread CTA
// per (group, row): 196 608 CTAs for 2048 rows, each a short chain of dependent loads, a block
// barrier and a store -- 109 us for 2048 rows where the 100 MB it moves are 16 us of HBM time, more
// than the chunked scan it feeds.  Here a WARP owns one group of 128 channels (lane l: channels
// 4l .. 4l+3, the reference's own split of the l2-norm: four squares per lane, then the adjacent-pairs
// tree over the 32 lanes -- a warp reduction, no barrier) and walks a run of consecutive rows with the
// three previous taps in registers, so every projection entry is loaded once (8 bytes per lane and row,
// the loads of a run's next row issued before this row's arithmetic).  Same per-channel arithmetic
// (conv_channel_apply) and the same reduction order: bit-identical to the kernel above.
constexpr uint32_t kPrepRun = 8;          // consecutive rows per warp
constexpr uint32_t kPrepWarps = 8;        // runs per CTA

__device__ __forceinline__ void load_bf16x4_bits(const __nv_bfloat16* p, float out[4]) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xFFFF0000u);
}

__global__ void __launch_bounds__(kPrepWarps * 32)
gdn_prepare_block_kernel(const __nv_bfloat16* __restrict__ projection,
                         const __nv_bfloat16* __restrict__ conv_state,
                         const __nv_bfloat16* __restrict__ conv_weights, __nv_bfloat16* __restrict__ qk,
                         __nv_bfloat16* __restrict__ value, __nv_bfloat16* __restrict__ z,
                         __nv_bfloat16* __restrict__ new_conv_state, uint32_t rows) {
    const uint32_t group = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t r0 = (blockIdx.y * kPrepWarps + warp) * kPrepRun;
    if (r0 >= rows) return;
    const uint32_t r1 = min(rows, r0 + kPrepRun);
    if (group >= kGdnConv / kGdnDim) {   // z: a copy
        const uint32_t index = (group - kGdnConv / kGdnDim) * kGdnDim + lane * 4u;
        for (uint32_t row = r0; row < r1; ++row)
            *reinterpret_cast<uint2*>(z + uint64_t(row) * kGdnV + index) =
                __ldg(reinterpret_cast<const uint2*>(projection + uint64_t(row) * kGdnProj + kGdnZOff + index));
        return;
    }
    const uint32_t c0 = group * kGdnDim + lane * 4u;
    // the four channels' tap weights: [channel][4] bf16, 32 bytes per lane
    float wf[4][4];
    {
        const uint4 wa = __ldg(reinterpret_cast<const uint4*>(conv_weights + uint64_t(c0) * 4u));
        const uint4 wb = __ldg(reinterpret_cast<const uint4*>(conv_weights + uint64_t(c0) * 4u + 8u));
        const uint32_t raw[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            wf[i][0] = __uint_as_float(raw[2 * i] << 16); wf[i][1] = __uint_as_float(raw[2 * i] & 0xFFFF0000u);
            wf[i][2] = __uint_as_float(raw[2 * i + 1] << 16); wf[i][3] = __uint_as_float(raw[2 * i + 1] & 0xFFFF0000u);
        }
    }
    // logical sequence [3 conv-state rows | projection rows]: position `row` taps logical rows row .. row+3
    auto load_logical = [&](uint32_t logical, float out[4]) {
        if (logical < 3u) load_bf16x4_bits(conv_state + logical * kGdnConv + c0, out);
        else load_bf16x4_bits(projection + uint64_t(logical - 3u) * kGdnProj + c0, out);
    };
    float w0[4], w1[4], w2[4], cur[4], next[4];
    load_logical(r0, w0);
    load_logical(r0 + 1u, w1);
    load_logical(r0 + 2u, w2);
    load_logical(r0 + 3u, cur);
    const bool is_qk = group < kGdnQk / kGdnDim, is_query = group < kGdnKeyHeads;
    for (uint32_t row = r0; row < r1; ++row) {
        if (row + 1u < r1) load_logical(row + 4u, next);   // the next row's newest tap, ahead of this row's arithmetic
        float act[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const float taps[4] = {w0[i], w1[i], w2[i], cur[i]};
            act[i] = bf2f(conv_channel_apply_w(taps, wf[i]));
        }
        __nv_bfloat16 res[4];
        if (is_qk) {
            // head_normalise with the head's 128 channels in one warp
            float acc = 0.0f;
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) acc += act[i] * act[i];
            acc = warp_sum(acc);
            const float inverse = 1.0f / sqrtf(acc / float(kGdnDim) + kRmsEps);
            const __nv_bfloat16 scale = is_query ? f2bf(1.0f / 128.0f) : f2bf(0.08838834764831845f);
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) res[i] = bmul(f2bf(act[i] * inverse), scale);
            *reinterpret_cast<uint2*>(qk + uint64_t(row) * kGdnQk + c0) = *reinterpret_cast<const uint2*>(res);
        } else {
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) res[i] = f2bf(act[i]);
            *reinterpret_cast<uint2*>(value + uint64_t(row) * kGdnV + c0 - kGdnQk) = *reinterpret_cast<const uint2*>(res);
        }
        if (row + 1u == rows) {   // the three newest taps become the conv state
            __nv_bfloat16 t1[4], t2[4], t3[4];
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                t1[i] = f2bf(w1[i]); t2[i] = f2bf(w2[i]); t3[i] = f2bf(cur[i]);
            }
            *reinterpret_cast<uint2*>(new_conv_state + 0u * kGdnConv + c0) = *reinterpret_cast<const uint2*>(t1);
            *reinterpret_cast<uint2*>(new_conv_state + 1u * kGdnConv + c0) = *reinterpret_cast<const uint2*>(t2);
            *reinterpret_cast<uint2*>(new_conv_state + 2u * kGdnConv + c0) = *reinterpret_cast<const uint2*>(t3);
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            w0[i] = w1[i]; w1[i] = w2[i]; w2[i] = cur[i]; cur[i] = next[i];
        }
    }
}

__global__ void gdn_gates_kernel(const __nv_bfloat16* __restrict__ projection,
                                 uint64_t projection_stride, const __nv_bfloat16* __restrict__ a_log,
                                 const __nv_bfloat16* __restrict__ dt_bias, float* __restrict__ decay,
                                 float* __restrict__ beta, uint32_t rows) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * kGdnValueHeads) return;
    const uint32_t row = idx / kGdnValueHeads, head = idx % kGdnValueHeads;
    const __nv_bfloat16* proj = projection + row * projection_stride;
    decay[idx] = gdn_decay(proj[kGdnAOff + head], dt_bias[head], a_log[head]);
    beta[idx] = gdn_beta(proj[kGdnBOff + head]);
}

// ---- recurrence --------------------------------------------------------------------------
// Four state rows of one warp through one delta-rule step (gdn.metal:151-171).
// kf / qf: this lane's 4 key / query elements.  Returns the 4 row outputs (all lanes).
struct Rows4 {
    float4 s[4];
};
// Sum over the 32 lanes of FOUR values at once, each through the adjacent-pairs tree (lane i with
// i^1, then i^2, ... i^16): the same additions as four butterfly reductions, but after the first
// level a lane only carries the two rows it keeps, after the second one row, so the tree takes 6
// shuffles instead of 20.  Lane L ends with the total of row tree4_row(L); every lane of a class
// L & 3 holds the same bits the butterfly would give.
__device__ __forceinline__ uint32_t tree4_row(uint32_t lane) { return ((lane & 1u) << 1) | ((lane >> 1) & 1u); }
__device__ __forceinline__ float tree4(float r0, float r1, float r2, float r3, uint32_t lane) {
    const bool odd = (lane & 1u) != 0u, upper = (lane & 2u) != 0u;
    // level 1: even lanes keep rows 0 and 1, odd lanes rows 2 and 3
    const float a = (odd ? r2 : r0) + __shfl_xor_sync(0xffffffffu, odd ? r0 : r2, 1);
    const float b = (odd ? r3 : r1) + __shfl_xor_sync(0xffffffffu, odd ? r1 : r3, 1);
    // level 2: lanes with bit 1 clear keep the first of their two rows, the others the second
    float t = (upper ? b : a) + __shfl_xor_sync(0xffffffffu, upper ? a : b, 2);
    t += __shfl_xor_sync(0xffffffffu, t, 4);
    t += __shfl_xor_sync(0xffffffffu, t, 8);
    t += __shfl_xor_sync(0xffffffffu, t, 16);
    return t;
}
// Returns, in every lane, the output of row tree4_row(lane) of the four.
__device__ __forceinline__ float delta_rule_rows4(Rows4& r, const float kf[4], const float qf[4],
                                                  const float v[4], float decay, float beta, uint32_t lane) {
    float kv[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        r.s[j].x *= decay; r.s[j].y *= decay; r.s[j].z *= decay; r.s[j].w *= decay;
        float a = r.s[j].x * kf[0];
        a = fmaf(r.s[j].y, kf[1], a);
        a = fmaf(r.s[j].z, kf[2], a);
        kv[j] = fmaf(r.s[j].w, kf[3], a);
    }
    // every lane needs the four totals: rows 0, 2, 1, 3 sit in lanes 0, 1, 2, 3 of each group of four
    const float total = tree4(kv[0], kv[1], kv[2], kv[3], lane);
    const uint32_t quad = lane & ~3u;
    kv[0] = __shfl_sync(0xffffffffu, total, quad);
    kv[2] = __shfl_sync(0xffffffffu, total, quad | 1u);
    kv[1] = __shfl_sync(0xffffffffu, total, quad | 2u);
    kv[3] = __shfl_sync(0xffffffffu, total, quad | 3u);
    float out[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        const float delta = (v[j] - kv[j]) * beta;
        r.s[j].x = fmaf(kf[0], delta, r.s[j].x);
        r.s[j].y = fmaf(kf[1], delta, r.s[j].y);
        r.s[j].z = fmaf(kf[2], delta, r.s[j].z);
        r.s[j].w = fmaf(kf[3], delta, r.s[j].w);
        float a = r.s[j].x * qf[0];
        a = fmaf(r.s[j].y, qf[1], a);
        a = fmaf(r.s[j].z, qf[2], a);
        out[j] = fmaf(r.s[j].w, qf[3], a);
    }
    return tree4(out[0], out[1], out[2], out[3], lane);
}

// Two independent groups of four rows, level by level: the dependent chain is as long as for
// one group (the shuffle unit answers in about 25 cycles per level and a warp issues in order), the
// additions are the same.
__device__ __forceinline__ void tree4x2(const float x[4], const float y[4], uint32_t lane, float& tx, float& ty) {
    const bool odd = (lane & 1u) != 0u, upper = (lane & 2u) != 0u;
    const float xa = (odd ? x[2] : x[0]) + __shfl_xor_sync(0xffffffffu, odd ? x[0] : x[2], 1);
    const float xb = (odd ? x[3] : x[1]) + __shfl_xor_sync(0xffffffffu, odd ? x[1] : x[3], 1);
    const float ya = (odd ? y[2] : y[0]) + __shfl_xor_sync(0xffffffffu, odd ? y[0] : y[2], 1);
    const float yb = (odd ? y[3] : y[1]) + __shfl_xor_sync(0xffffffffu, odd ? y[1] : y[3], 1);
    tx = (upper ? xb : xa) + __shfl_xor_sync(0xffffffffu, upper ? xa : xb, 2);
    ty = (upper ? yb : ya) + __shfl_xor_sync(0xffffffffu, upper ? ya : yb, 2);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        const float px = __shfl_xor_sync(0xffffffffu, tx, off), py = __shfl_xor_sync(0xffffffffu, ty, off);
        tx += px;
        ty += py;
    }
}
// Eight rows (two groups of four) through one delta-rule step; returns the outputs of rows
// tree4_row(lane) of the first and of the second group.
__device__ __forceinline__ void delta_rule_rows8(Rows4& ra, Rows4& rb, const float kf[4], const float qf[4],
                                                 const float va[4], const float vb[4], float decay, float beta,
                                                 uint32_t lane, float& out_a, float& out_b) {
    float ka[4], kb[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        ra.s[j].x *= decay; ra.s[j].y *= decay; ra.s[j].z *= decay; ra.s[j].w *= decay;
        rb.s[j].x *= decay; rb.s[j].y *= decay; rb.s[j].z *= decay; rb.s[j].w *= decay;
        float a = ra.s[j].x * kf[0], b = rb.s[j].x * kf[0];
        a = fmaf(ra.s[j].y, kf[1], a); b = fmaf(rb.s[j].y, kf[1], b);
        a = fmaf(ra.s[j].z, kf[2], a); b = fmaf(rb.s[j].z, kf[2], b);
        ka[j] = fmaf(ra.s[j].w, kf[3], a); kb[j] = fmaf(rb.s[j].w, kf[3], b);
    }
    float ta, tb_;
    tree4x2(ka, kb, lane, ta, tb_);
    const uint32_t quad = lane & ~3u;
    ka[0] = __shfl_sync(0xffffffffu, ta, quad);       kb[0] = __shfl_sync(0xffffffffu, tb_, quad);
    ka[2] = __shfl_sync(0xffffffffu, ta, quad | 1u);  kb[2] = __shfl_sync(0xffffffffu, tb_, quad | 1u);
    ka[1] = __shfl_sync(0xffffffffu, ta, quad | 2u);  kb[1] = __shfl_sync(0xffffffffu, tb_, quad | 2u);
    ka[3] = __shfl_sync(0xffffffffu, ta, quad | 3u);  kb[3] = __shfl_sync(0xffffffffu, tb_, quad | 3u);
    float oa[4], ob[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        const float da = (va[j] - ka[j]) * beta, db = (vb[j] - kb[j]) * beta;
        ra.s[j].x = fmaf(kf[0], da, ra.s[j].x); rb.s[j].x = fmaf(kf[0], db, rb.s[j].x);
        ra.s[j].y = fmaf(kf[1], da, ra.s[j].y); rb.s[j].y = fmaf(kf[1], db, rb.s[j].y);
        ra.s[j].z = fmaf(kf[2], da, ra.s[j].z); rb.s[j].z = fmaf(kf[2], db, rb.s[j].z);
        ra.s[j].w = fmaf(kf[3], da, ra.s[j].w); rb.s[j].w = fmaf(kf[3], db, rb.s[j].w);
        float a = ra.s[j].x * qf[0], b = rb.s[j].x * qf[0];
        a = fmaf(ra.s[j].y, qf[1], a); b = fmaf(rb.s[j].y, qf[1], b);
        a = fmaf(ra.s[j].z, qf[2], a); b = fmaf(rb.s[j].z, qf[2], b);
        oa[j] = fmaf(ra.s[j].w, qf[3], a); ob[j] = fmaf(rb.s[j].w, qf[3], b);
    }
    tree4x2(oa, ob, lane, out_a, out_b);
}

__device__ __forceinline__ void load_bf16x4(const __nv_bfloat16* p, float out[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    out[0] = bf2f(a.x); out[1] = bf2f(a.y); out[2] = bf2f(b.x); out[3] = bf2f(b.y);
}

// Standalone recurrence step: grid (4 quarters, 32 v-heads), 256 threads = 8 warps x 4 rows.
__global__ void __launch_bounds__(256)
gdn_step_kernel(const __nv_bfloat16* __restrict__ qk, const __nv_bfloat16* __restrict__ value,
                const __nv_bfloat16* __restrict__ projection, const __nv_bfloat16* __restrict__ a_log,
                const __nv_bfloat16* __restrict__ dt_bias, const float* __restrict__ state_in,
                __nv_bfloat16* __restrict__ y, float* __restrict__ state_out) {
    const uint32_t head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t row0 = blockIdx.x * 32u + warp * 4u;
    const uint64_t base = (uint64_t(head) * kGdnDim + row0) * kGdnDim + lane * 4u;
    Rows4 r;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j)
        r.s[j] = __ldcs(reinterpret_cast<const float4*>(state_in + base + j * kGdnDim));
    const float decay = gdn_decay(projection[kGdnAOff + head], dt_bias[head], a_log[head]);
    const float beta = gdn_beta(projection[kGdnBOff + head]);
    float kf[4], qf[4], v[4];
    load_bf16x4(qk + (head >> 1) * kGdnDim + lane * 4u, qf);
    load_bf16x4(qk + kGdnKOff + (head >> 1) * kGdnDim + lane * 4u, kf);
    load_bf16x4(value + head * kGdnDim + row0, v);
    const float mine = delta_rule_rows4(r, kf, qf, v, decay, beta, lane);
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j)
        __stcs(reinterpret_cast<float4*>(state_out + base + j * kGdnDim), r.s[j]);
    if (lane < 4u) y[head * kGdnDim + row0 + tree4_row(lane)] = f2bf(mine);
}

// Weighted per-head RMSNorm of y times SiLU(z) (gdn.metal:174-207): one warp per head.
// zf: the head's z values of this lane, wraw: its four norm weights (both already loaded).
__device__ __forceinline__ void gate_norm_head_loaded(const float yv[4], const float zf[4], uint2 wraw,
                                                      __nv_bfloat16* out, uint32_t lane) {
    float acc = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) acc += yv[i] * yv[i];
    acc = warp_sum(acc);
    const float inverse = 1.0f / sqrtf(acc / float(kGdnDim) + kRmsEps);
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(&wraw);
    __nv_bfloat16 res[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const __nv_bfloat16 normed = bmul(w[i], f2bf(yv[i] * inverse));
        res[i] = f2bf((zf[i] * sigmoid_f32(zf[i])) * bf2f(normed));
    }
    *reinterpret_cast<uint2*>(out + lane * 4u) = *reinterpret_cast<const uint2*>(res);
}
__device__ __forceinline__ void gate_norm_head(const float yv[4], const __nv_bfloat16* z,
                                               const __nv_bfloat16* weight, __nv_bfloat16* out,
                                               uint32_t lane) {
    float zf[4];
    load_bf16x4(z + lane * 4u, zf);
    const uint2 wraw = *reinterpret_cast<const uint2*>(weight + lane * 4u);
    gate_norm_head_loaded(yv, zf, wraw, out, lane);
}

__global__ void __launch_bounds__(128)
gdn_gate_norm_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                     const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out) {
    const uint32_t head = blockIdx.x * 4u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    const uint64_t base = uint64_t(blockIdx.y) * kGdnV + head * kGdnDim;
    float yv[4];
    load_bf16x4(y + base + lane * 4u, yv);
    gate_norm_head(yv, z + base, weight, out + base, lane);
}

// ---- fused lane-batched decode step ------------------------------------------------------
// One CTA per (v-head, lane): conv + SiLU + l2-norm for this head's q, k and v channels,
// gates, the 128-row state update and the gated RMSNorm, with the first state rows already in
// flight while the prologue computes.  256 threads = 8 warps x 16 rows.
struct GdnLanes {
    tatara_gdn_lane lane[TATARA_MAX_LANES];
};

// Two data paths for the 64 KiB of state a CTA reads and rewrites (same arithmetic, same bits):
// kBulk = false: every lane loads its float4 of a row into registers (16 rows per warp in flight) and
// stores it back with st.global.cs.  The CTA's 512 row requests then sit in the load/store unit's
// queue ahead of everything requested later (the projection entries that arrive after the
// dependency wait).  kBulk = true: lane 0 of each warp asks the copy engine for its warp's 16 rows
// as two 4 KiB cp.async.bulk copies into shared memory, completing on two mbarriers, and sends the
// updated rows back the same way; the small requests of the prologue never queue behind them.
constexpr uint32_t kFdStateBytes = kGdnDim * kGdnDim * 4u;      // one head's state: 64 KiB
constexpr uint32_t kFdHalfBytes = 8u * kGdnDim * 4u;            // 8 rows of a warp: 4 KiB
constexpr uint32_t kFdSmem = kFdStateBytes + 16u * 8u + 16u;    // + two mbarriers per warp + the abort word

__device__ __forceinline__ void bulk_load_stream(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "{\n .reg .b64 pol;\n createpolicy.fractional.L2::evict_first.b64 pol, 1.0;\n"
        " cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], pol;\n}"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_store_stream(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile(
        "{\n .reg .b64 pol;\n createpolicy.fractional.L2::evict_first.b64 pol, 1.0;\n"
        " cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, pol;\n}"
        ::"l"(dst), "r"(src), "r"(bytes)
        : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// `projection` is NOT __restrict__: it is written by the predecessor this kernel waits for, and a
// const __restrict__ pointer lets the compiler treat its loads as invariant and move them above
// griddepcontrol.wait (seen once: garbage rows whenever the projection kernel was still running).
template <bool kBulk>
__global__ void __launch_bounds__(256)
gdn_decode_fused_kernel(const __nv_bfloat16* projection, uint64_t projection_stride,
                        const __nv_bfloat16* __restrict__ conv_weights,
                        const __nv_bfloat16* __restrict__ a_log, const __nv_bfloat16* __restrict__ dt_bias,
                        const __nv_bfloat16* __restrict__ norm_weight, __nv_bfloat16* conv_pool,
                        float* rec_pool, __nv_bfloat16* __restrict__ y_out,
                        __nv_bfloat16* __restrict__ gated, const __grid_constant__ GdnLanes lanes,
                        const tatara_gdn_lane* lanes_device, uint32_t* status, uint32_t late_half,
                        uint32_t early_dependents) {
    extern __shared__ __align__(128) uint8_t fd_smem[];   // kBulk: [128 rows][128] f32, mbarriers, abort word
    __shared__ float head_q[kGdnDim], head_k[kGdnDim];
    __shared__ float qn[kGdnDim], kn[kGdnDim], vn[kGdnDim], ys[kGdnDim];
    const uint32_t head = blockIdx.x, row_lane = blockIdx.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // the lane table of this call, or the one kept in device memory (CUDA-graph replay)
    // (both sources are read without a branch between them: the parameter table entry and the
    // pointer sit in different lines of the cold constant bank, and a branch on the pointer would
    // put the two misses one after the other -- 1100 cycles before the first request left the SM)
    tatara_gdn_lane gl = lanes.lane[row_lane];
    if (lanes_device != nullptr) gl = lanes_device[row_lane];
    const __nv_bfloat16* proj = projection + row_lane * projection_stride;
    const __nv_bfloat16* conv_in = conv_pool + gl.conv_in;
    __nv_bfloat16* conv_out = conv_pool + gl.conv_out;
    const float* state_in = rec_pool + gl.rec_in;
    float* state_out = rec_pool + gl.rec_out;

    // The layer's own conv taps and the weights are not written by the predecessor either: requested
    // here, with the state rows.  threads 0..127 -> q channel, 128..255 -> k channel; v channel on 0..127.
    const uint32_t l128 = threadIdx.x & 127u;
    const bool is_q = threadIdx.x < 128u;
    const uint32_t qk_channel = (is_q ? 0u : kGdnKOff) + (head >> 1) * kGdnDim + l128;
    const uint32_t v_channel = kGdnQk + head * kGdnDim + l128;
    float taps[4], vtaps[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const unsigned short* conv_bits = reinterpret_cast<const unsigned short*>(conv_in);
#pragma unroll
    for (uint32_t t = 0; t < 3; ++t) {
        taps[t] = __uint_as_float(uint32_t(__ldcg(conv_bits + t * kGdnConv + qk_channel)) << 16);
        if (is_q) vtaps[t] = __uint_as_float(uint32_t(__ldcg(conv_bits + t * kGdnConv + v_channel)) << 16);
    }
    const uint2 qk_w = *reinterpret_cast<const uint2*>(conv_weights + uint64_t(qk_channel) * 4u);
    const uint2 v_w = *reinterpret_cast<const uint2*>(conv_weights + uint64_t(v_channel) * 4u);
    const __nv_bfloat16 dt_raw = dt_bias[head], alog_raw = a_log[head];
    const uint2 norm_w = *reinterpret_cast<const uint2*>(norm_weight + lane * 4u);
    // Then all 16 state rows of this warp (4 batches x 4 rows, 64 KiB per CTA): the whole state read
    // overlaps the conv / norm prologue, and the few small requests above are not queued behind it.
    const uint32_t row_base = warp * 16u;
    const uint64_t sbase = (uint64_t(head) * kGdnDim + row_base) * kGdnDim + lane * 4u;
    Rows4 rows[kBulk ? 1 : 4];   // the register path keeps all 16 rows of the warp here
    float* st = reinterpret_cast<float*>(fd_smem);
    const uint32_t fd_bars = s2u(fd_smem + kFdStateBytes) + warp * 16u;   // this warp's two mbarriers
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(fd_smem + kFdStateBytes + 128u);
    if constexpr (kBulk) {
        if (threadIdx.x == 0) *abort_flag = 0u;   // read only after the prologue's __syncthreads
        if (lane == 0) {
            mbar_init(fd_bars, 1);
            mbar_init(fd_bars + 8u, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            // The first eight rows now.  With few lanes (one wave of CTAs, `late_half`) the other eight are
            // asked for after the projection entries (below): behind the whole 64 KiB of every CTA
            // those few small requests took 1.8 us to answer.  With many lanes the CTAs of a later wave
            // overlap that wait anyway, and a CTA that asks late only holds its SM longer.
            mbar_expect_tx(fd_bars, kFdHalfBytes);
            bulk_load_stream(s2u(st + row_base * kGdnDim), state_in + (uint64_t(head) * kGdnDim + row_base) * kGdnDim,
                             kFdHalfBytes, fd_bars);
            if (!late_half) {
                mbar_expect_tx(fd_bars + 8u, kFdHalfBytes);
                bulk_load_stream(s2u(st + (row_base + 8u) * kGdnDim),
                                 state_in + (uint64_t(head) * kGdnDim + row_base + 8u) * kGdnDim, kFdHalfBytes,
                                 fd_bars + 8u);
            }
        }
    } else {
#pragma unroll
        for (uint32_t batch = 0; batch < 4; ++batch)
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j)
                rows[batch].s[j] = __ldcs(reinterpret_cast<const float4*>(state_in + sbase + (batch * 4u + j) * kGdnDim));
    }
    // Launched as a programmatic dependent of its predecessor in the stream (the projection that
    // produces `projection`): what is read above is this layer's own state and weights, which that
    // predecessor does not write, so those loads are in flight while the predecessor finishes; the
    // projection row and every store wait here.  By default this kernel never signals its own
    // dependents early: a following call on the SAME state would read, before its own wait, the rows
    // written below.  A caller whose next kernels do not read this call's state or conv slots before
    // their own dependency wait (a layer walk: the out projection follows, then another layer) may say
    // so (TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS); the successor is then staged, and asks for its
    // weights, while this grid computes.
    // (`proj` is an output of the statement, so no load through it can be placed above it)
    asm volatile("griddepcontrol.wait;" : "+l"(proj) : : "memory");
    if (early_dependents) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Everything else the prologue and the epilogue read (the projection row) is requested at once:
    // one trip to L2 instead of one per dependent phase; the arithmetic keeps its order.
    taps[3] = bf2f(proj[qk_channel]);
    if (is_q) vtaps[3] = bf2f(proj[v_channel]);
    const __nv_bfloat16 a_raw = proj[kGdnAOff + head], b_raw = proj[kGdnBOff + head];
    float zf[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (warp == 0) load_bf16x4(proj + kGdnZOff + head * kGdnDim + lane * 4u, zf);
    if constexpr (kBulk) {
        if (lane == 0 && late_half) {
            mbar_expect_tx(fd_bars + 8u, kFdHalfBytes);
            bulk_load_stream(s2u(st + (row_base + 8u) * kGdnDim),
                             state_in + (uint64_t(head) * kGdnDim + row_base + 8u) * kGdnDim, kFdHalfBytes,
                             fd_bars + 8u);
        }
    }
    const __nv_bfloat16 act = conv_channel_apply(taps, qk_w);
    if ((head & 1u) == 0u) {
#pragma unroll
        for (uint32_t t = 0; t < 3; ++t) conv_out[t * kGdnConv + qk_channel] = f2bf(taps[t + 1u]);
    }
    const __nv_bfloat16 normed = head_normalise(is_q ? head_q : head_k, l128, bf2f(act), is_q);
    (is_q ? qn : kn)[l128] = bf2f(normed);
    if (is_q) {
        const __nv_bfloat16 va = conv_channel_apply(vtaps, v_w);
#pragma unroll
        for (uint32_t t = 0; t < 3; ++t) conv_out[t * kGdnConv + v_channel] = f2bf(vtaps[t + 1u]);
        vn[l128] = bf2f(va);
    }
    const float decay = gdn_decay(a_raw, dt_raw, alog_raw);
    const float beta = gdn_beta(b_raw);
    __syncthreads();

    float kf[4], qf[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        kf[i] = kn[lane * 4u + i];
        qf[i] = qn[lane * 4u + i];
    }
    bool ok = true;
#pragma unroll
    for (uint32_t half = 0; half < 2; ++half) {   // eight rows at a time: two groups of four, level by level
        const uint32_t r8 = row_base + half * 8u;
        Rows4 local[kBulk ? 2 : 1];
        if constexpr (kBulk) {
            // rows 8h .. 8h+7 of this warp have landed (bounded wait; a warp that gives up computes nothing more)
            if (ok) {
                __syncwarp();   // lane 0 initialised the barrier
                ok = mbar_wait(fd_bars + 8u * half, 0, abort_flag);
            }
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j)
                local[j >> 2].s[j & 3u] = *reinterpret_cast<const float4*>(st + (r8 + j) * kGdnDim + lane * 4u);
        }
        Rows4& ra = kBulk ? local[0] : rows[kBulk ? 0 : half * 2u];
        Rows4& rb = kBulk ? local[kBulk ? 1 : 0] : rows[kBulk ? 0 : half * 2u + 1u];
        float va[4], vb[4], out_a, out_b;
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            va[j] = vn[r8 + j];
            vb[j] = vn[r8 + 4u + j];
        }
        delta_rule_rows8(ra, rb, kf, qf, va, vb, decay, beta, lane, out_a, out_b);
        if constexpr (kBulk) {
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(st + (r8 + j) * kGdnDim + lane * 4u) = local[j >> 2].s[j & 3u];
            // eight updated rows: back to the state through the copy engine
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && ok)
                bulk_store_stream(state_out + (uint64_t(head) * kGdnDim + r8) * kGdnDim, s2u(st + r8 * kGdnDim),
                                  kFdHalfBytes);
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                __stcs(reinterpret_cast<float4*>(state_out + sbase + (half * 8u + j) * kGdnDim), ra.s[j]);
                __stcs(reinterpret_cast<float4*>(state_out + sbase + (half * 8u + 4u + j) * kGdnDim), rb.s[j]);
            }
        }
        if (lane < 4u) {
            ys[r8 + tree4_row(lane)] = bf2f(f2bf(out_a));
            ys[r8 + 4u + tree4_row(lane)] = bf2f(f2bf(out_b));
        }
    }
    __syncthreads();
    if (warp == 0) {
        const uint64_t obase = uint64_t(row_lane) * kGdnV + head * kGdnDim;
        float yv[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) yv[i] = ys[lane * 4u + i];
        if (y_out != nullptr) {
            __nv_bfloat16 yb[4];
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) yb[i] = f2bf(yv[i]);
            *reinterpret_cast<uint2*>(y_out + obase + lane * 4u) = *reinterpret_cast<const uint2*>(yb);
        }
        gate_norm_head_loaded(yv, zf, norm_w, gated + obase, lane);
    }
    if constexpr (kBulk) {
        // the copies out of this CTA's shared memory must have completed before it is released
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (threadIdx.x == 0 && *abort_flag) {
            atomicCAS(status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
            status[kStatusDetail] = blockIdx.y * kGdnValueHeads + blockIdx.x;
        }
    }
}

} // namespace tb

using namespace tb;
using bf16 = __nv_bfloat16;

extern "C" tatara_status tatara_gdn_prepare(tatara_ctx* ctx, void* stream, const void* projection,
                                            const void* conv_in, const void* conv_weights, void* qk,
                                            void* value, void* z, void* conv_out, uint32_t rows) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !conv_in || !conv_weights || !qk || !value || !z || !conv_out)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prepare: null buffer");
    if (!aligned(conv_weights, 8)) return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prepare: conv weights alignment");
    if (conv_in == conv_out) return fail(ctx, TATARA_STATE_SLOT_MISMATCH, "gdn_prepare: conv_in aliases conv_out");
    if (rows == 0 || rows > 65535u) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_prepare: rows");
    // blocks of rows: a warp per (group, run of rows), 8-byte accesses (every buffer 8-byte aligned, weights 16)
    if (rows >= 32u && aligned(projection, 8) && aligned(conv_in, 8) && aligned(conv_weights, 16) && aligned(qk, 8) &&
        aligned(value, 8) && aligned(z, 8) && aligned(conv_out, 8)) {
        const uint32_t tiles = (rows + kPrepWarps * kPrepRun - 1u) / (kPrepWarps * kPrepRun);
        gdn_prepare_block_kernel<<<dim3(96, tiles), kPrepWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const bf16*>(projection), static_cast<const bf16*>(conv_in),
            static_cast<const bf16*>(conv_weights), static_cast<bf16*>(qk), static_cast<bf16*>(value),
            static_cast<bf16*>(z), static_cast<bf16*>(conv_out), rows);
        return check_launch(ctx, "gdn_prepare");
    }
    gdn_prepare_kernel<false><<<dim3(96, rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(projection), static_cast<const bf16*>(conv_in),
        static_cast<const bf16*>(conv_weights), static_cast<bf16*>(qk), static_cast<bf16*>(value),
        static_cast<bf16*>(z), static_cast<bf16*>(conv_out), rows, nullptr, 0);
    return check_launch(ctx, "gdn_prepare");
}

extern "C" tatara_status tatara_gdn_prepare_tape(tatara_ctx* ctx, void* stream, const void* projection,
                                                 const void* conv_in, const void* conv_weights, void* qk,
                                                 void* value, void* z, void* conv_out, uint32_t rows,
                                                 void* conv_tape, uint32_t tape_layer) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !conv_in || !conv_weights || !qk || !value || !z || !conv_out || !conv_tape)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prepare_tape: null buffer");
    if (!aligned(conv_weights, 8)) return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prepare_tape: conv weights alignment");
    if (conv_in == conv_out) return fail(ctx, TATARA_STATE_SLOT_MISMATCH, "gdn_prepare_tape: conv_in aliases conv_out");
    if (rows == 0 || rows > 16u || tape_layer >= 40u)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_prepare_tape: rows above 16 or layer above 39");
    gdn_prepare_kernel<true><<<dim3(96, rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(projection), static_cast<const bf16*>(conv_in),
        static_cast<const bf16*>(conv_weights), static_cast<bf16*>(qk), static_cast<bf16*>(value),
        static_cast<bf16*>(z), static_cast<bf16*>(conv_out), rows, static_cast<bf16*>(conv_tape), tape_layer);
    return check_launch(ctx, "gdn_prepare_tape");
}

extern "C" tatara_status tatara_gdn_gates(tatara_ctx* ctx, void* stream, const void* projection,
                                          uint32_t projection_stride, const void* a_log,
                                          const void* dt_bias, void* decay, void* beta, uint32_t rows) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !a_log || !dt_bias || !decay || !beta)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_gates: null buffer");
    if (rows == 0 || projection_stride < kGdnProj)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_gates: rows / stride");
    const uint32_t total = rows * kGdnValueHeads;
    gdn_gates_kernel<<<(total + 255u) / 256u, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(projection), projection_stride, static_cast<const bf16*>(a_log),
        static_cast<const bf16*>(dt_bias), static_cast<float*>(decay), static_cast<float*>(beta), rows);
    return check_launch(ctx, "gdn_gates");
}

extern "C" tatara_status tatara_gdn_step(tatara_ctx* ctx, void* stream, const void* qk,
                                         const void* value, const void* projection, const void* a_log,
                                         const void* dt_bias, const void* state_in, void* y,
                                         void* state_out) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!qk || !value || !projection || !a_log || !dt_bias || !state_in || !y || !state_out)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_step: null buffer");
    if (!aligned(state_in, 16) || !aligned(state_out, 16) || !aligned(qk, 8) || !aligned(value, 8))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_step: misaligned buffer");
    if (state_in == state_out) return fail(ctx, TATARA_STATE_SLOT_MISMATCH, "gdn_step: state_in aliases state_out");
    gdn_step_kernel<<<dim3(4, kGdnValueHeads), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(qk), static_cast<const bf16*>(value), static_cast<const bf16*>(projection),
        static_cast<const bf16*>(a_log), static_cast<const bf16*>(dt_bias),
        static_cast<const float*>(state_in), static_cast<bf16*>(y), static_cast<float*>(state_out));
    return check_launch(ctx, "gdn_step");
}

extern "C" tatara_status tatara_gdn_gate_norm(tatara_ctx* ctx, void* stream, const void* y, const void* z,
                                              const void* weight, void* out, uint32_t rows) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!y || !z || !weight || !out) return fail(ctx, TATARA_INVALID_BUFFER, "gdn_gate_norm: null buffer");
    if (!aligned(y, 8) || !aligned(z, 8) || !aligned(weight, 8) || !aligned(out, 8))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_gate_norm: misaligned buffer");
    if (rows == 0 || rows > 65535u) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_gate_norm: rows");
    gdn_gate_norm_kernel<<<dim3(kGdnValueHeads / 4, rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(y), static_cast<const bf16*>(z), static_cast<const bf16*>(weight),
        static_cast<bf16*>(out));
    return check_launch(ctx, "gdn_gate_norm");
}

// One launch of the fused step: the form is the context's TATARA_POLICY_GDN_DECODE_FORM.
static tatara_status launch_fused_step(tatara_ctx* ctx, void* stream, const void* projection, uint32_t projection_stride,
                                       const void* conv_weights, const void* a_log, const void* dt_bias,
                                       const void* norm_weight, void* conv_pool, void* rec_pool, const GdnLanes& table,
                                       const tatara_gdn_lane* lanes_device, uint32_t n_lanes, void* y, void* gated,
                                       const char* what) {
    const bool bulk = ctx->gdn_decode_form == 0u;
    static bool configured[64] = {false};
    if (bulk && !configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(gdn_decode_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFdSmem) !=
            cudaSuccess)
            return check_launch(ctx, "gdn_decode_batch: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kGdnValueHeads, n_lanes);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = bulk ? kFdSmem : 0;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, bulk ? gdn_decode_fused_kernel<true> : gdn_decode_fused_kernel<false>,
                             static_cast<const bf16*>(projection), uint64_t(projection_stride),
                             static_cast<const bf16*>(conv_weights), static_cast<const bf16*>(a_log),
                             static_cast<const bf16*>(dt_bias), static_cast<const bf16*>(norm_weight),
                             static_cast<bf16*>(conv_pool), static_cast<float*>(rec_pool), static_cast<bf16*>(y),
                             static_cast<bf16*>(gated), table, lanes_device, ctx->device_status,
                             n_lanes * kGdnValueHeads <= 2u * uint32_t(ctx->sm_count) ? 1u : 0u,
                             ctx->gdn_step_early_dependents);
    return check_launch(ctx, what);
}

extern "C" tatara_status tatara_gdn_decode_batch(tatara_ctx* ctx, void* stream, const void* projection,
                                                 uint32_t projection_stride, const void* conv_weights,
                                                 const void* a_log, const void* dt_bias,
                                                 const void* norm_weight, void* conv_pool, void* rec_pool,
                                                 const tatara_gdn_lane* lanes, uint32_t n_lanes, void* y,
                                                 void* gated) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !conv_weights || !a_log || !dt_bias || !norm_weight || !conv_pool || !rec_pool ||
        !lanes || !gated)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_decode_batch: null buffer");
    if (!aligned(rec_pool, 16) || !aligned(conv_weights, 8) || !aligned(norm_weight, 8) ||
        !aligned(gated, 8) || !aligned(projection, 8) || (y && !aligned(y, 8)))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_decode_batch: misaligned buffer");
    if (n_lanes == 0 || n_lanes > TATARA_MAX_LANES)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "gdn_decode_batch: lane count");
    if (projection_stride < kGdnProj || (projection_stride & 3u))
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_decode_batch: projection stride");
    GdnLanes table{};
    for (uint32_t i = 0; i < n_lanes; ++i) {
        const tatara_gdn_lane& l = lanes[i];
        if (l.conv_in == l.conv_out || l.rec_in == l.rec_out)
            return fail(ctx, TATARA_STATE_SLOT_MISMATCH, "gdn_decode_batch: in slot aliases out slot");
        if ((l.rec_in & 3u) || (l.rec_out & 3u))
            return fail(ctx, TATARA_INVALID_BUFFER, "gdn_decode_batch: recurrent offset alignment");
        table.lane[i] = l;
    }
    return launch_fused_step(ctx, stream, projection, projection_stride, conv_weights, a_log, dt_bias, norm_weight,
                             conv_pool, rec_pool, table, nullptr, n_lanes, y, gated, "gdn_decode_batch");
}

extern "C" tatara_status tatara_gdn_decode_batch_indirect(tatara_ctx* ctx, void* stream, const void* projection,
                                                          uint32_t projection_stride, const void* conv_weights,
                                                          const void* a_log, const void* dt_bias,
                                                          const void* norm_weight, void* conv_pool, void* rec_pool,
                                                          const tatara_gdn_lane* lanes_device, uint32_t n_lanes,
                                                          void* y, void* gated) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!projection || !conv_weights || !a_log || !dt_bias || !norm_weight || !conv_pool || !rec_pool ||
        !lanes_device || !gated)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_decode_batch_indirect: null buffer");
    if (!aligned(rec_pool, 16) || !aligned(conv_weights, 8) || !aligned(norm_weight, 8) ||
        !aligned(gated, 8) || !aligned(projection, 8) || (y && !aligned(y, 8)) || !aligned(lanes_device, 8))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_decode_batch_indirect: misaligned buffer");
    if (n_lanes == 0 || n_lanes > TATARA_MAX_LANES)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "gdn_decode_batch_indirect: lane count");
    if (projection_stride < kGdnProj || (projection_stride & 3u))
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_decode_batch_indirect: projection stride");
    // The offsets are the caller's (written once when the table is created; tatara_lanes_advance only
    // swaps them): in != out and 16-byte alignment of the recurrent offsets are the caller's contract.
    const GdnLanes unused{};
    return launch_fused_step(ctx, stream, projection, projection_stride, conv_weights, a_log, dt_bias, norm_weight,
                             conv_pool, rec_pool, unused, lanes_device, n_lanes, y, gated, "gdn_decode_batch_indirect");
}
