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

// Tape of a speculative verify band (reference geometry, tools/generate_kernel_library.py:2045-2049):
// 40 layers x 16 rows; f32 regions delta [layer][row][32][128], key [layer][row][16][128], gates
// [layer][row][32][2] = (decay, beta).
constexpr uint32_t kTapeRows = 16, kTapeLayers = 40;
constexpr uint64_t kTapeKeyOff = uint64_t(kTapeLayers) * kTapeRows * kGdnValueHeads * kGdnDim;
constexpr uint64_t kTapeGateOff = kTapeKeyOff + uint64_t(kTapeLayers) * kTapeRows * kGdnKeyHeads * kGdnDim;
constexpr uint64_t kTapeFloats = kTapeGateOff + uint64_t(kTapeLayers) * kTapeRows * kGdnValueHeads * 2u;

// grid (4 quarters, 32 v-heads), 256 threads = 8 warps x 4 rows.  kTape: also record, per row,
// delta per state row, the key row (one writer per key head) and (decay, beta) per head
// (gdn_recurrence_gates_tape_blk, prefill_gdn.metal:434-527).
template <bool kTape>
__global__ void __launch_bounds__(256)
gdn_scan_kernel(const __nv_bfloat16* __restrict__ qk, const __nv_bfloat16* __restrict__ value,
                const float* __restrict__ decay, const float* __restrict__ beta,
                const float* __restrict__ state_in, __nv_bfloat16* __restrict__ y,
                float* __restrict__ state_out, uint32_t rows, float* __restrict__ tape, uint32_t tape_layer) {
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
        if (kTape) {
            const uint64_t tape_row = uint64_t(tape_layer) * kTapeRows + step;
            if (lane < 4u) {
                const float mine = lane == 0 ? (v[0] - kv[0]) * bet : lane == 1 ? (v[1] - kv[1]) * bet
                                 : lane == 2 ? (v[2] - kv[2]) * bet : (v[3] - kv[3]) * bet;
                tape[(tape_row * kGdnValueHeads + head) * kGdnDim + row0 + lane] = mine;
            }
            if (blockIdx.x == 0 && warp == 0) {   // the block that owns state row 0 of this head
                if ((head & 1u) == 0u)
                    *reinterpret_cast<float4*>(tape + kTapeKeyOff + (tape_row * kGdnKeyHeads + (head >> 1)) * kGdnDim + lane * 4u) =
                        make_float4(kf[0], kf[1], kf[2], kf[3]);
                if (lane == 0)
                    *reinterpret_cast<float2*>(tape + kTapeGateOff + (tape_row * kGdnValueHeads + head) * 2u) = make_float2(dec, bet);
            }
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

// Replay of `steps` taped rows onto the pre-band state: the scan's own two update statements
// (decay multiply, then fma with key * delta), so the result has the bits the scan itself
// reaches after `steps` rows (gdn_tape_replay_blk, prefill_gdn.metal:529-569).
__global__ void __launch_bounds__(256)
gdn_tape_replay_kernel(const float* __restrict__ tape, const float* __restrict__ state_in,
                       float* __restrict__ state_out, uint32_t steps, uint32_t tape_layer) {
    const uint32_t head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t row0 = blockIdx.x * 32u + warp * 4u;
    const uint64_t base = (uint64_t(head) * kGdnDim + row0) * kGdnDim + lane * 4u;
    float4 s[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) s[j] = *reinterpret_cast<const float4*>(state_in + base + j * kGdnDim);
    for (uint32_t step = 0; step < steps; ++step) {
        const uint64_t tape_row = uint64_t(tape_layer) * kTapeRows + step;
        const float dec = tape[kTapeGateOff + (tape_row * kGdnValueHeads + head) * 2u];
        const float4 k = *reinterpret_cast<const float4*>(tape + kTapeKeyOff + (tape_row * kGdnKeyHeads + (head >> 1)) * kGdnDim + lane * 4u);
        const float4 d = *reinterpret_cast<const float4*>(tape + (tape_row * kGdnValueHeads + head) * kGdnDim + row0);
        const float delta[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            s[j].x *= dec; s[j].y *= dec; s[j].z *= dec; s[j].w *= dec;
            s[j].x = fmaf(k.x, delta[j], s[j].x);
            s[j].y = fmaf(k.y, delta[j], s[j].y);
            s[j].z = fmaf(k.z, delta[j], s[j].z);
            s[j].w = fmaf(k.w, delta[j], s[j].w);
        }
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
    gdn_scan_kernel<false><<<dim3(4, kGdnValueHeads), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(qk), static_cast<const __nv_bfloat16*>(value),
        static_cast<const float*>(decay), static_cast<const float*>(beta),
        static_cast<const float*>(state_in), static_cast<__nv_bfloat16*>(y),
        static_cast<float*>(state_out), rows, nullptr, 0);
    return check_launch(ctx, "gdn_prefill(scan)");
}

extern "C" uint64_t tatara_gdn_tape_bytes(void) { return kTapeFloats * sizeof(float); }
extern "C" uint64_t tatara_gdn_conv_tape_bytes(void) {
    return uint64_t(kTapeLayers) * kTapeRows * 3u * kGdnConv * 2u;
}

extern "C" tatara_status tatara_gdn_prefill_tape(tatara_ctx* ctx, void* stream, const void* qk,
                                                 const void* value, const void* decay, const void* beta,
                                                 const void* state_in, void* y, void* state_out,
                                                 uint32_t rows, void* tape, uint32_t tape_layer) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!qk || !value || !decay || !beta || !state_in || !y || !state_out || !tape)
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill_tape: null buffer");
    if (!aligned(state_in, 16) || !aligned(state_out, 16) || !aligned(qk, 16) || !aligned(value, 16) ||
        !aligned(y, 16) || !aligned(tape, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill_tape: misaligned buffer");
    if (state_in == state_out) return fail(ctx, TATARA_STATE_SLOT_MISMATCH, "gdn_prefill_tape: state_in aliases state_out");
    if (rows == 0 || rows > kTapeRows || tape_layer >= kTapeLayers)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_prefill_tape: rows above 16 or layer above 39");
    gdn_scan_kernel<true><<<dim3(4, kGdnValueHeads), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(qk), static_cast<const __nv_bfloat16*>(value),
        static_cast<const float*>(decay), static_cast<const float*>(beta),
        static_cast<const float*>(state_in), static_cast<__nv_bfloat16*>(y),
        static_cast<float*>(state_out), rows, static_cast<float*>(tape), tape_layer);
    return check_launch(ctx, "gdn_prefill_tape");
}

extern "C" tatara_status tatara_gdn_tape_replay(tatara_ctx* ctx, void* stream, const void* tape,
                                                const void* state_in, void* state_out, uint32_t steps,
                                                uint32_t tape_layer) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!tape || !state_in || !state_out) return fail(ctx, TATARA_INVALID_BUFFER, "gdn_tape_replay: null buffer");
    if (!aligned(tape, 16) || !aligned(state_in, 16) || !aligned(state_out, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_tape_replay: misaligned buffer");
    if (state_in == state_out) return fail(ctx, TATARA_STATE_SLOT_MISMATCH, "gdn_tape_replay: state_in aliases state_out");
    if (steps > kTapeRows || tape_layer >= kTapeLayers)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_tape_replay: steps above 16 or layer above 39");
    gdn_tape_replay_kernel<<<dim3(4, kGdnValueHeads), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(tape), static_cast<const float*>(state_in), static_cast<float*>(state_out), steps,
        tape_layer);
    return check_launch(ctx, "gdn_tape_replay");
}
