// Gated DeltaNet block prefill (reference: prefill_gdn.metal:137-196,
// gdn_recurrence_gates_blk; host src/runtime/prefill_step.cpp:1958-2038).
//
// chunk == 64 runs the chunked (WY / UT transform) form on the tensor cores (gdn_chunked.cu).
// chunk == 1 selects the sequential scan: the reference's own algorithm, one warp per four
// state rows held in registers for the whole block, one state write at the end.
#include "common.cuh"

namespace tb {

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float out[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    out[0] = bf2f(a.x); out[1] = bf2f(a.y); out[2] = bf2f(b.x); out[3] = bf2f(b.y);
}

// grid (4 quarters, 32 v-heads), 256 threads = 8 warps x 4 rows.
__global__ void __launch_bounds__(256)
gdn_scan_kernel(const __nv_bfloat16* __restrict__ qk, const __nv_bfloat16* __restrict__ value,
                const float* __restrict__ decay, const float* __restrict__ beta,
                const float* __restrict__ state_in, __nv_bfloat16* __restrict__ y,
                float* __restrict__ state_out, uint32_t rows) {
    const uint32_t head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t row0 = blockIdx.x * 32u + warp * 4u;
    const uint64_t base = (uint64_t(head) * kGdnDim + row0) * kGdnDim + lane * 4u;
    float4 s[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) s[j] = *reinterpret_cast<const float4*>(state_in + base + j * kGdnDim);
    const __nv_bfloat16* qp = qk + (head >> 1) * kGdnDim + lane * 4u;
    const __nv_bfloat16* kp = qp + kGdnKOff;
    const __nv_bfloat16* vp = value + head * kGdnDim + row0;
    float kf[4], qf[4], v[4], dec, bet;
    load4(kp, kf); load4(qp, qf); load4(vp, v);
    dec = decay[head]; bet = beta[head];
    for (uint32_t step = 0; step < rows; ++step) {
        // prefetch the next step's operands while this step's reductions run
        float nk[4], nq[4], nv[4], ndec = 0.0f, nbet = 0.0f;
        if (step + 1u < rows) {
            const uint64_t n = uint64_t(step + 1u);
            load4(kp + n * kGdnQk, nk); load4(qp + n * kGdnQk, nq); load4(vp + n * kGdnV, nv);
            ndec = decay[n * kGdnValueHeads + head];
            nbet = beta[n * kGdnValueHeads + head];
        }
        float kv[4], out[4];
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            s[j].x *= dec; s[j].y *= dec; s[j].z *= dec; s[j].w *= dec;
            float a = s[j].x * kf[0];
            a = fmaf(s[j].y, kf[1], a);
            a = fmaf(s[j].z, kf[2], a);
            kv[j] = fmaf(s[j].w, kf[3], a);
        }
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) kv[j] += __shfl_xor_sync(0xffffffffu, kv[j], off);
        }
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const float delta = (v[j] - kv[j]) * bet;
            s[j].x = fmaf(kf[0], delta, s[j].x);
            s[j].y = fmaf(kf[1], delta, s[j].y);
            s[j].z = fmaf(kf[2], delta, s[j].z);
            s[j].w = fmaf(kf[3], delta, s[j].w);
            float a = s[j].x * qf[0];
            a = fmaf(s[j].y, qf[1], a);
            a = fmaf(s[j].z, qf[2], a);
            out[j] = fmaf(s[j].w, qf[3], a);
        }
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) out[j] += __shfl_xor_sync(0xffffffffu, out[j], off);
        }
        if (lane < 4u) {
            const float mine = lane == 0 ? out[0] : lane == 1 ? out[1] : lane == 2 ? out[2] : out[3];
            y[uint64_t(step) * kGdnV + head * kGdnDim + row0 + lane] = f2bf(mine);
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) { kf[i] = nk[i]; qf[i] = nq[i]; v[i] = nv[i]; }
        dec = ndec; bet = nbet;
    }
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) *reinterpret_cast<float4*>(state_out + base + j * kGdnDim) = s[j];
}

tatara_status launch_gdn_chunked(tatara_ctx* ctx, cudaStream_t stream, const __nv_bfloat16* qk,
                                 const __nv_bfloat16* value, const float* decay, const float* beta,
                                 const float* state_in, __nv_bfloat16* y, float* state_out,
                                 uint32_t rows, void* scratch, uint64_t scratch_bytes);

} // namespace tb

using namespace tb;

extern "C" tatara_status tatara_gdn_prefill(tatara_ctx* ctx, void* stream, const void* qk,
                                            const void* value, const void* decay, const void* beta,
                                            const void* state_in, void* y, void* state_out,
                                            uint32_t rows, uint32_t chunk, void* scratch,
                                            uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!qk || !value || !decay || !beta || !state_in || !y || !state_out)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill: null buffer");
    if (!aligned(state_in, 16) || !aligned(state_out, 16) || !aligned(qk, 16) || !aligned(value, 16) ||
        !aligned(y, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill: misaligned buffer");
    if (rows == 0) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_prefill: rows");
    if (chunk != 64u && chunk != 1u)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_prefill: chunk must be 64 (or 1 = sequential scan)");
    if (chunk == 64u)
        return launch_gdn_chunked(ctx, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(qk),
                                  static_cast<const __nv_bfloat16*>(value), static_cast<const float*>(decay),
                                  static_cast<const float*>(beta), static_cast<const float*>(state_in),
                                  static_cast<__nv_bfloat16*>(y), static_cast<float*>(state_out), rows, scratch,
                                  scratch_bytes);
    gdn_scan_kernel<<<dim3(4, kGdnValueHeads), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(qk), static_cast<const __nv_bfloat16*>(value),
        static_cast<const float*>(decay), static_cast<const float*>(beta),
        static_cast<const float*>(state_in), static_cast<__nv_bfloat16*>(y),
        static_cast<float*>(state_out), rows);
    return check_launch(ctx, "gdn_prefill(scan)");
}
