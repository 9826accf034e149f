// Host-side mirror of the reference runtime's attention / Gated DeltaNet layer encoders over the
// tatara_b200 C ABI (reference: include/tatara/runtime/decode_step.h:63-100, 173-187, 245-250,
// 340-385; src/runtime/decode_step.cpp:630-780, 1002-1441).  Header-only C++17; needs only
// include/tatara_b200.h and the CUDA runtime.
//
// It keeps the reference's vocabulary for this slice of the token walk:
//   DecodeStatePool   one pool per layer and state kind, equal stripes per slot; gated-delta
//                     layers interleave ping-pong parities (slot s = stripes 2s, 2s+1)
//   DecodeStateSlot   per-request state: capacity, stripe, per-layer `swapped`, status
//   DecodeStream      {state, context, stripe} of one row of a group / batch submission
//   LayerPass         the error-latching encoder (first error latches and gates later work,
//                     decode_step.cpp:106-184); ContextOutOfRange / StateSlotMismatch are
//                     returned before anything is enqueued (decode_step.cpp:812-824)
//   advance_decode_state  flips the gated-delta pairs after the token completes
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <utility>
#include <vector>

#include "../../include/tatara_b200.h"

namespace tatara::runtime {

// Same names as MetalCommandError (include/tatara/backend/metal/commands.h:232-262).
enum class CommandError : std::uint8_t {
    None,
    InvalidBuffer,
    ContextOutOfRange,
    StateSlotMismatch,
    InvalidStreamGroup,
    InvalidDispatchExtent,
    InvalidDevice,
    ScratchTooSmall,
    DeviceWaitTimeout,
    CudaError,
};
inline CommandError to_command_error(tatara_status s) noexcept { return static_cast<CommandError>(s); }
inline const char* to_string(CommandError e) noexcept { return tatara_status_name(static_cast<tatara_status>(e)); }

enum class LayerKind : std::uint8_t { GatedDelta, FullAttention };

inline constexpr std::uint32_t kQueryHeads = 16, kKeyValueHeads = 2, kHeadDimension = 256;
inline constexpr std::uint32_t kAttnProjectionRows = 9216, kAttnQueryValues = kQueryHeads * kHeadDimension;
inline constexpr std::uint32_t kGdnProjectionRows = 12352, kGdnValueValues = 4096;
inline constexpr std::uint64_t kGdnConvStateValues = 3ull * 8192ull;             // bf16
inline constexpr std::uint64_t kGdnRecurrentStateValues = 32ull * 128ull * 128ull; // f32
inline constexpr std::uint32_t kMaximumBatchRows = TATARA_MAX_LANES;
inline constexpr std::uint32_t kHidden = 2048;

// A context is a cache position, so equality with capacity is already one past the allocation
// (include/tatara/runtime/decode_geometry.h:133-135).
constexpr bool context_in_capacity(std::uint32_t context, std::uint32_t capacity) {
    return capacity != 0 && context < capacity;
}

// Zero-initialised device allocation (the reference's sealed zeroed-allocation rule,
// src/runtime/decode_step.cpp:49-57).
class DeviceBuffer {
  public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(std::uint64_t bytes) : bytes_(bytes) {
        if (bytes == 0 || cudaMalloc(&ptr_, bytes) != cudaSuccess || cudaMemset(ptr_, 0, bytes) != cudaSuccess) {
            if (ptr_ != nullptr) cudaFree(ptr_);
            ptr_ = nullptr;
            bytes_ = 0;
        }
    }
    DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(std::exchange(o.ptr_, nullptr)), bytes_(std::exchange(o.bytes_, 0)) {}
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) {
            reset();
            ptr_ = std::exchange(o.ptr_, nullptr);
            bytes_ = std::exchange(o.bytes_, 0);
        }
        return *this;
    }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { reset(); }
    explicit operator bool() const noexcept { return ptr_ != nullptr; }
    void* data() const noexcept { return ptr_; }
    std::uint64_t bytes() const noexcept { return bytes_; }

  private:
    void reset() noexcept {
        if (ptr_ != nullptr) cudaFree(ptr_);
        ptr_ = nullptr;
    }
    void* ptr_ = nullptr;
    std::uint64_t bytes_ = 0;
};

struct DecodeStatePoolLayer {
    LayerKind kind;
    DeviceBuffer first;          // attention: K pool (bf16); gated delta: conv pool (bf16)
    DeviceBuffer second;         // attention: V pool (bf16); gated delta: recurrent pool (f32)
    std::uint64_t first_stride;  // elements per stripe
    std::uint64_t second_stride;
};

struct DecodeStatePool {
    std::uint32_t stripes{0};   // slots
    std::uint32_t capacity{0};
    std::vector<DecodeStatePoolLayer> layers;
};

enum class DecodeStateSlotStatus : std::uint8_t { Ready, SnapshotPending, RestorePending, Poisoned };

struct DecodeStateSlot {
    std::uint32_t capacity{0};
    std::uint32_t stripe{0};
    std::vector<bool> swapped;  // per layer; meaningful for gated-delta layers only
    DecodeStateSlotStatus status{DecodeStateSlotStatus::Ready};
    // prefix-state transfer in flight (include/tatara/runtime/decode_step.h: active_transfer_*)
    std::uint64_t next_transfer_generation{1};
    std::uint64_t active_transfer_generation{0};
    const void* active_transfer_arena{nullptr};
    std::uint32_t active_transfer_positions{0};
    std::uint64_t active_transfer_offset_bytes{0};
    std::uint64_t active_transfer_state_bytes{0};
};

struct DecodeStream {
    DecodeStateSlot* state{nullptr};
    std::uint32_t context{0};
};

// One pool buffer per layer per state kind holding every slot's state as equal stripes
// (src/runtime/decode_step.cpp:494-536).
inline bool create_state_pool(std::uint32_t slots, std::uint32_t capacity, const std::vector<LayerKind>& schedule,
                              DecodeStatePool& pool, std::vector<DecodeStateSlot>& out_slots) {
    pool.stripes = slots;
    pool.capacity = capacity;
    pool.layers.clear();
    for (const LayerKind kind : schedule) {
        DecodeStatePoolLayer layer{kind, {}, {}, 0, 0};
        if (kind == LayerKind::FullAttention) {
            layer.first_stride = layer.second_stride = std::uint64_t{kKeyValueHeads} * capacity * kHeadDimension;
            layer.first = DeviceBuffer(layer.first_stride * slots * 2);
            layer.second = DeviceBuffer(layer.second_stride * slots * 2);
        } else {
            layer.first_stride = kGdnConvStateValues;
            layer.second_stride = kGdnRecurrentStateValues;
            layer.first = DeviceBuffer(layer.first_stride * 2 * slots * 2);   // ping-pong, bf16
            layer.second = DeviceBuffer(layer.second_stride * 2 * slots * 4); // ping-pong, f32
        }
        if (!layer.first || !layer.second) return false;
        pool.layers.push_back(std::move(layer));
    }
    // cudaMemset may return before the fill has run, and the callers' streams are non-blocking
    // (they do not order behind the default stream): the zeroes must be there before the first launch
    if (cudaDeviceSynchronize() != cudaSuccess) return false;
    out_slots.assign(slots, DecodeStateSlot{});
    for (std::uint32_t s = 0; s < slots; ++s) {
        out_slots[s].capacity = capacity;
        out_slots[s].stripe = s;
        out_slots[s].swapped.assign(schedule.size(), false);
    }
    return true;
}

struct AttentionWeights {
    const void* q_norm;  // [256] bf16
    const void* k_norm;  // [256] bf16
};
struct GatedDeltaWeights {
    const void* conv;      // [8192][4] bf16
    const void* a_log;     // [32] bf16
    const void* dt_bias;   // [32] bf16
    const void* norm;      // [128] bf16
};

// One affine-Q4 weight as the reference binds it (words, scales, biases of `rows` output rows;
// encode.quantized(...), src/runtime/decode_step.cpp:658-664, 705-708).
struct QuantizedWeight {
    const void* words{nullptr};
    const void* scales{nullptr};
    const void* biases{nullptr};
    std::uint32_t rows{0};
};
struct AttentionProjection {   // bound.attention.{query, key, value, out}
    QuantizedWeight query, key, value, out;
};
struct GatedDeltaProjection {  // bound.gated_delta.{qkv, z, b, a, out}
    QuantizedWeight qkv, z, b, a, out;
};

// Per-batch scratch slabs, one row per stream (include/tatara/runtime/decode_step.h:278-305).
struct DecodeBatchScratch {
    std::uint32_t rows{0};
    DeviceBuffer query, gate, attended;  // [rows][4096] bf16
    DeviceBuffer records;                // split-KV partial records
    DeviceBuffer gdn_y, gdn_gated;       // [rows][4096] bf16
};
inline bool create_batch_scratch(std::uint32_t rows, std::uint32_t capacity, DecodeBatchScratch& s) {
    s.rows = rows;
    const std::uint64_t slab = std::uint64_t{rows} * kAttnQueryValues * 2;
    s.query = DeviceBuffer(slab);
    s.gate = DeviceBuffer(slab);
    s.attended = DeviceBuffer(slab);
    s.records = DeviceBuffer(tatara_attn_decode_scratch_bytes(capacity, rows));
    s.gdn_y = DeviceBuffer(std::uint64_t{rows} * kGdnValueValues * 2);
    s.gdn_gated = DeviceBuffer(std::uint64_t{rows} * kGdnValueValues * 2);
    return s.query && s.gate && s.attended && s.records && s.gdn_y && s.gdn_gated;
}

// The error-latching encoder of this slice of the token walk.
class LayerPass {
  public:
    LayerPass(tatara_ctx* ctx, cudaStream_t stream) noexcept : ctx_(ctx), stream_(stream) {
        if (ctx_ == nullptr) error_ = CommandError::InvalidDevice;
    }
    CommandError error() const noexcept { return error_; }
    explicit operator bool() const noexcept { return error_ == CommandError::None; }

    // Attention layer for every stream: qk_rope (appends K/V at `context`) then decode attention.
    // projection_slab [rows][9216] bf16 in, scratch.attended [rows][4096] bf16 out.
    CommandError encode_attention(const DecodeStatePool& pool, std::uint32_t layer, const AttentionWeights& weights,
                                  const std::vector<DecodeStream>& streams, const void* projection_slab,
                                  DecodeBatchScratch& scratch) {
        if (error_ != CommandError::None) return error_;
        if (CommandError e = check_group(pool, layer, LayerKind::FullAttention, streams, scratch); e != CommandError::None)
            return latch(e);
        const DecodeStatePoolLayer& pl = pool.layers[layer];
        std::vector<tatara_attn_lane> table(streams.size());
        for (std::size_t r = 0; r < streams.size(); ++r)
            table[r] = tatara_attn_lane{std::uint64_t{streams[r].state->stripe} * pl.first_stride, streams[r].context, 0};
        const auto rows = static_cast<std::uint32_t>(streams.size());
        tatara_status st = tatara_attn_qk_rope_batch(ctx_, stream_, projection_slab, weights.q_norm, weights.k_norm,
                                                     scratch.query.data(), scratch.gate.data(), pl.first.data(),
                                                     pl.second.data(), pool.capacity, table.data(), rows,
                                                     kAttnProjectionRows, kAttnQueryValues);
        if (st != TATARA_OK) return latch(to_command_error(st));
        st = tatara_attn_decode_batch(ctx_, stream_, scratch.query.data(), scratch.gate.data(), pl.first.data(),
                                      pl.second.data(), table.data(), rows, pool.capacity, kAttnQueryValues,
                                      scratch.attended.data(), scratch.records.data(), scratch.records.bytes());
        return st == TATARA_OK ? CommandError::None : latch(to_command_error(st));
    }

    // Gated-delta layer for every stream: conv + recurrence + gate-norm in one launch.
    // projection_slab [rows][12352] bf16 in, scratch.gdn_gated [rows][4096] bf16 out.
    CommandError encode_gated_delta(const DecodeStatePool& pool, std::uint32_t layer, const GatedDeltaWeights& weights,
                                    const std::vector<DecodeStream>& streams, const void* projection_slab,
                                    DecodeBatchScratch& scratch) {
        if (error_ != CommandError::None) return error_;
        if (CommandError e = check_group(pool, layer, LayerKind::GatedDelta, streams, scratch); e != CommandError::None)
            return latch(e);
        const DecodeStatePoolLayer& pl = pool.layers[layer];
        std::vector<tatara_gdn_lane> table(streams.size());
        for (std::size_t r = 0; r < streams.size(); ++r) {
            const DecodeStateSlot& slot = *streams[r].state;
            const std::uint64_t in = 2ull * slot.stripe + (slot.swapped[layer] ? 1u : 0u);
            const std::uint64_t out = 2ull * slot.stripe + (slot.swapped[layer] ? 0u : 1u);
            table[r] = tatara_gdn_lane{in * pl.first_stride, out * pl.first_stride, in * pl.second_stride,
                                       out * pl.second_stride};
        }
        const tatara_status st = tatara_gdn_decode_batch(
            ctx_, stream_, projection_slab, kGdnProjectionRows, weights.conv, weights.a_log, weights.dt_bias,
            weights.norm, pl.first.data(), pl.second.data(), table.data(), static_cast<std::uint32_t>(streams.size()),
            scratch.gdn_y.data(), scratch.gdn_gated.data());
        return st == TATARA_OK ? CommandError::None : latch(to_command_error(st));
    }

    // attn_project: normed [rows][2048] bf16 -> projection_slab [rows][9216] bf16, each row with the
    // reference's exact per-row sequence (decode_step.cpp:705-711).
    CommandError encode_attention_project(const AttentionProjection& w, const void* normed, std::uint32_t rows,
                                          void* projection_slab) {
        const tatara_q4_matrix m[3] = {as_matrix(w.query), as_matrix(w.key), as_matrix(w.value)};
        return project(m, 3, kHidden, normed, kHidden, rows, projection_slab, kAttnProjectionRows);
    }
    // gdn_project: normed -> projection_slab [rows][12352] bf16 (decode_step.cpp:657-664).
    CommandError encode_gated_delta_project(const GatedDeltaProjection& w, const void* normed, std::uint32_t rows,
                                            void* projection_slab) {
        const tatara_q4_matrix m[4] = {as_matrix(w.qkv), as_matrix(w.z), as_matrix(w.b), as_matrix(w.a)};
        return project(m, 4, kHidden, normed, kHidden, rows, projection_slab, kGdnProjectionRows);
    }
    // out_projection: attended / gated [rows][4096] bf16 -> branch [rows][branch_stride] bf16
    // (decode_step.cpp:698-702, 732-736).
    CommandError encode_out_projection(const QuantizedWeight& out, const void* input, std::uint32_t rows, void* branch,
                                       std::uint64_t branch_stride) {
        const tatara_q4_matrix m[1] = {as_matrix(out)};
        return project(m, 1, kAttnQueryValues, input, kAttnQueryValues, rows, branch, branch_stride);
    }

    // commit() + wait_until_completed(): returns the latched host error or a device-side one.
    CommandError commit_and_wait() {
        if (error_ != CommandError::None) return error_;
        const tatara_status st = tatara_ctx_sync(ctx_, stream_);
        return st == TATARA_OK ? CommandError::None : latch(to_command_error(st));
    }

  private:
    static tatara_q4_matrix as_matrix(const QuantizedWeight& w) noexcept {
        return tatara_q4_matrix{w.words, w.scales, w.biases, w.rows, 0};
    }
    CommandError project(const tatara_q4_matrix* m, std::uint32_t n, std::uint32_t k, const void* input,
                         std::uint64_t input_stride, std::uint32_t rows, void* out, std::uint64_t out_stride) {
        if (error_ != CommandError::None) return error_;
        if (rows == 0 || rows > kMaximumBatchRows) return latch(CommandError::InvalidStreamGroup);
        const tatara_status st = tatara_q4_project(ctx_, stream_, input, input_stride, rows, m, n, k, out, out_stride);
        return st == TATARA_OK ? CommandError::None : latch(to_command_error(st));
    }
    CommandError latch(CommandError e) noexcept {
        if (error_ == CommandError::None) error_ = e;
        return e;
    }
    static CommandError check_group(const DecodeStatePool& pool, std::uint32_t layer, LayerKind kind,
                                    const std::vector<DecodeStream>& streams, const DecodeBatchScratch& scratch) {
        if (streams.empty() || streams.size() > kMaximumBatchRows || streams.size() > scratch.rows)
            return CommandError::InvalidStreamGroup;
        if (layer >= pool.layers.size() || pool.layers[layer].kind != kind) return CommandError::StateSlotMismatch;
        for (std::size_t r = 0; r < streams.size(); ++r) {
            const DecodeStateSlot* slot = streams[r].state;
            if (slot == nullptr || slot->status != DecodeStateSlotStatus::Ready || slot->capacity != pool.capacity ||
                slot->stripe >= pool.stripes || slot->swapped.size() != pool.layers.size())
                return CommandError::StateSlotMismatch;
            for (std::size_t o = 0; o < r; ++o)  // states must be pairwise distinct
                if (streams[o].state == slot) return CommandError::InvalidStreamGroup;
            if (!context_in_capacity(streams[r].context, slot->capacity)) return CommandError::ContextOutOfRange;
        }
        return CommandError::None;
    }

    tatara_ctx* ctx_;
    cudaStream_t stream_;
    CommandError error_{CommandError::None};
};

// Swaps the gated-delta conv and recurrent pairs after a token completes
// (src/runtime/decode_step.cpp:1432-1441).
inline void advance_decode_state(const DecodeStatePool& pool, const std::vector<DecodeStream>& streams) {
    for (const DecodeStream& s : streams)
        for (std::size_t l = 0; l < pool.layers.size(); ++l)
            if (pool.layers[l].kind == LayerKind::GatedDelta) s.state->swapped[l] = !s.state->swapped[l];
}

} // namespace tatara::runtime
