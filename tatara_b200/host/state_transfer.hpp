// Host-side state formats either side of the layer kernels, over the tatara_b200 C ABI:
//
//   * the canonical prefix-state payload (reference: include/tatara/runtime/prefix_state_transfer.h,
//     src/runtime/prefix_state_transfer.cpp:296-470; prefill_geometry.h:205-246): one live
//     conv + recurrent plane per gated-delta layer, family-major and schedule-ordered, followed
//     by the packed K then V prefix positions of every KV head of every attention layer.
//     Snapshot copies slot -> arena from whichever ping-pong half is live; restore installs the
//     gated-delta bytes into the canonical input half and resets the phase.  The segment list
//     is executed as ONE tatara_state_copy launch instead of one blit per segment.
//   * the `Q36BRS01` state record (reference: tools/native/decode_harness.cpp:339-461): magic,
//     u32 positions, then per layer in schedule order the live gated-delta planes or the packed
//     K heads followed by the packed V heads.
//
// Header-only C++17 beside hybrid_layers.hpp; same vocabulary and error enums as the reference.
#pragma once

#include <cstddef>
#include <limits>

#include "hybrid_layers.hpp"

namespace tatara::runtime {

inline constexpr std::uint32_t kPrefixStateLayoutSchemaVersion = 1;
inline constexpr std::uint64_t kBf16Bytes = 2;

enum class PrefixStateLayoutError : std::uint8_t {
    None, InvalidSchedule, InvalidGeometry, PositionOutOfRange, FamilyCountMismatch, TotalMismatch, Overflow,
    SegmentOutOfRange,
};
enum class PrefixStateSegmentKind : std::uint8_t { GatedDeltaConvolution, GatedDeltaRecurrent, AttentionKey, AttentionValue };
enum class PrefixStateBufferPlane : std::uint8_t { First, FirstOutput, Second, SecondOutput, Arena };
enum class PrefixStateTransferDirection : std::uint8_t { Snapshot, Restore };
enum class PrefixStateTransferError : std::uint8_t {
    None, InvalidLayout, InvalidStateSlot, StateSlotNotReady, InvalidArena, ArenaOutOfRange, GenerationExhausted,
    PhaseEvidenceTooSmall, CommandEncodingFailed, StaleTicket, AlreadyCompleted, PoisonedStateSlot,
};

struct PrefixStateLayoutSpec {
    const LayerKind* schedule{nullptr};
    std::size_t layers{0};
    std::uint32_t capacity{0};
    std::uint32_t positions{0};
    std::uint32_t key_value_heads{0};
    std::uint32_t head_dimension{0};
    std::uint32_t expected_gated_delta_layers{0};
    std::uint32_t expected_attention_layers{0};
    std::uint64_t gated_delta_convolution_bytes{0};
    std::uint64_t gated_delta_recurrent_bytes{0};
    std::uint64_t expected_total_bytes{0};
};
struct PrefixStateLayout {
    PrefixStateLayoutSpec specification;
    std::uint32_t gated_delta_layers{0};
    std::uint32_t attention_layers{0};
    std::uint32_t segment_count{0};
    std::uint64_t attention_segment_bytes{0};
    std::uint64_t attention_slot_head_stride_bytes{0};
    std::uint64_t gated_delta_bytes{0};
    std::uint64_t attention_bytes{0};
    std::uint64_t total_bytes{0};
};
struct PrefixStateLayoutResult {
    PrefixStateLayoutError error{PrefixStateLayoutError::InvalidGeometry};
    PrefixStateLayout layout;
    explicit operator bool() const noexcept { return error == PrefixStateLayoutError::None; }
};
struct PrefixStateSegment {
    PrefixStateSegmentKind kind{PrefixStateSegmentKind::GatedDeltaConvolution};
    std::uint32_t layer_index{0};
    std::uint32_t head_index{0};
    std::uint64_t slot_offset_bytes{0};
    std::uint64_t snapshot_offset_bytes{0};
    std::uint64_t length_bytes{0};
};
struct PrefixStateSegmentResult {
    PrefixStateLayoutError error{PrefixStateLayoutError::SegmentOutOfRange};
    PrefixStateSegment segment;
    explicit operator bool() const noexcept { return error == PrefixStateLayoutError::None; }
};
struct PrefixStateCopyRoute {
    PrefixStateBufferPlane source{PrefixStateBufferPlane::First};
    PrefixStateBufferPlane destination{PrefixStateBufferPlane::Arena};
};

namespace state_transfer_detail {
inline bool add(std::uint64_t a, std::uint64_t b, std::uint64_t& out) noexcept {
    if (b > std::numeric_limits<std::uint64_t>::max() - a) return false;
    out = a + b;
    return true;
}
inline bool mul(std::uint64_t a, std::uint64_t b, std::uint64_t& out) noexcept {
    if (a != 0 && b > std::numeric_limits<std::uint64_t>::max() / a) return false;
    out = a * b;
    return true;
}
inline bool known(LayerKind k) noexcept { return k == LayerKind::GatedDelta || k == LayerKind::FullAttention; }
// index in the schedule of the `ordinal`-th layer of one family
inline std::uint32_t family_layer(const PrefixStateLayoutSpec& spec, bool gated, std::uint32_t ordinal) noexcept {
    std::uint32_t seen = 0;
    for (std::size_t l = 0; l < spec.layers; ++l)
        if ((spec.schedule[l] == LayerKind::GatedDelta) == gated && seen++ == ordinal) return static_cast<std::uint32_t>(l);
    return std::numeric_limits<std::uint32_t>::max();
}
} // namespace state_transfer_detail

// Sizes and counts of the canonical payload; every product is overflow-checked and the total
// must equal the caller's own figure (src/runtime/prefix_state_transfer.cpp:296-362).
inline PrefixStateLayoutResult make_prefix_state_layout(const PrefixStateLayoutSpec& spec) noexcept {
    using namespace state_transfer_detail;
    if (spec.schedule == nullptr || spec.layers == 0 || spec.layers > std::numeric_limits<std::uint32_t>::max())
        return {PrefixStateLayoutError::InvalidSchedule, {}};
    if (spec.capacity == 0 || spec.key_value_heads == 0 || spec.head_dimension == 0 ||
        spec.expected_gated_delta_layers == 0 || spec.expected_attention_layers == 0 ||
        spec.gated_delta_convolution_bytes == 0 || spec.gated_delta_recurrent_bytes == 0 || spec.expected_total_bytes == 0)
        return {PrefixStateLayoutError::InvalidGeometry, {}};
    if (spec.positions == 0 || spec.positions > spec.capacity) return {PrefixStateLayoutError::PositionOutOfRange, {}};
    PrefixStateLayout layout;
    layout.specification = spec;
    for (std::size_t l = 0; l < spec.layers; ++l) {
        if (!known(spec.schedule[l])) return {PrefixStateLayoutError::InvalidSchedule, {}};
        ++(spec.schedule[l] == LayerKind::GatedDelta ? layout.gated_delta_layers : layout.attention_layers);
    }
    if (layout.gated_delta_layers != spec.expected_gated_delta_layers ||
        layout.attention_layers != spec.expected_attention_layers)
        return {PrefixStateLayoutError::FamilyCountMismatch, {}};
    std::uint64_t per_gated = 0, attention_segments = 0, segments = 0;
    if (!add(spec.gated_delta_convolution_bytes, spec.gated_delta_recurrent_bytes, per_gated) ||
        !mul(spec.positions, spec.head_dimension, layout.attention_segment_bytes) ||
        !mul(layout.attention_segment_bytes, kBf16Bytes, layout.attention_segment_bytes) ||
        !mul(spec.capacity, spec.head_dimension, layout.attention_slot_head_stride_bytes) ||
        !mul(layout.attention_slot_head_stride_bytes, kBf16Bytes, layout.attention_slot_head_stride_bytes) ||
        !mul(layout.gated_delta_layers, per_gated, layout.gated_delta_bytes) ||
        !mul(layout.attention_layers, 2ull * spec.key_value_heads, attention_segments) ||
        !mul(attention_segments, layout.attention_segment_bytes, layout.attention_bytes) ||
        !add(layout.gated_delta_bytes, layout.attention_bytes, layout.total_bytes) ||
        !add(2ull * layout.gated_delta_layers, attention_segments, segments) ||
        segments > std::numeric_limits<std::uint32_t>::max())
        return {PrefixStateLayoutError::Overflow, {}};
    if (layout.total_bytes != spec.expected_total_bytes) return {PrefixStateLayoutError::TotalMismatch, {}};
    layout.segment_count = static_cast<std::uint32_t>(segments);
    return {PrefixStateLayoutError::None, layout};
}

// Segment `index` of the payload: gated-delta segments first (conv, recurrent per layer), then
// per attention layer the K heads and the V heads (src/runtime/prefix_state_transfer.cpp:375-434).
inline PrefixStateSegmentResult prefix_state_segment(const PrefixStateLayout& layout, std::uint32_t index) noexcept {
    using namespace state_transfer_detail;
    if (index >= layout.segment_count) return {PrefixStateLayoutError::SegmentOutOfRange, {}};
    const PrefixStateLayoutSpec& spec = layout.specification;
    const std::uint32_t gated_segments = 2u * layout.gated_delta_layers;
    PrefixStateSegment seg;
    if (index < gated_segments) {
        const std::uint32_t ordinal = index / 2u;
        const bool recurrent = (index & 1u) != 0;
        seg.layer_index = family_layer(spec, true, ordinal);
        if (seg.layer_index == std::numeric_limits<std::uint32_t>::max()) return {PrefixStateLayoutError::FamilyCountMismatch, {}};
        seg.kind = recurrent ? PrefixStateSegmentKind::GatedDeltaRecurrent : PrefixStateSegmentKind::GatedDeltaConvolution;
        seg.snapshot_offset_bytes = std::uint64_t{ordinal} * (spec.gated_delta_convolution_bytes + spec.gated_delta_recurrent_bytes) +
                                    (recurrent ? spec.gated_delta_convolution_bytes : 0);
        seg.length_bytes = recurrent ? spec.gated_delta_recurrent_bytes : spec.gated_delta_convolution_bytes;
        return {PrefixStateLayoutError::None, seg};
    }
    const std::uint32_t relative = index - gated_segments, per_layer = 2u * spec.key_value_heads;
    const std::uint32_t within = relative % per_layer;
    const bool value = within >= spec.key_value_heads;
    seg.layer_index = family_layer(spec, false, relative / per_layer);
    if (seg.layer_index == std::numeric_limits<std::uint32_t>::max()) return {PrefixStateLayoutError::FamilyCountMismatch, {}};
    seg.kind = value ? PrefixStateSegmentKind::AttentionValue : PrefixStateSegmentKind::AttentionKey;
    seg.head_index = value ? within - spec.key_value_heads : within;
    seg.slot_offset_bytes = std::uint64_t{seg.head_index} * layout.attention_slot_head_stride_bytes;
    seg.snapshot_offset_bytes = layout.gated_delta_bytes + std::uint64_t{relative} * layout.attention_segment_bytes;
    seg.length_bytes = layout.attention_segment_bytes;
    return {PrefixStateLayoutError::None, seg};
}

// Which slot plane a segment is read from (snapshot: the live ping-pong half) or written to
// (restore: always the canonical input half) (src/runtime/prefix_state_transfer.cpp:436-468).
inline PrefixStateCopyRoute prefix_state_copy_route(const PrefixStateSegment& segment, PrefixStateTransferDirection direction,
                                                    bool gated_delta_swapped) noexcept {
    PrefixStateBufferPlane live = PrefixStateBufferPlane::First, canonical = PrefixStateBufferPlane::First;
    switch (segment.kind) {
    case PrefixStateSegmentKind::GatedDeltaConvolution:
        live = gated_delta_swapped ? PrefixStateBufferPlane::FirstOutput : PrefixStateBufferPlane::First;
        break;
    case PrefixStateSegmentKind::GatedDeltaRecurrent:
        live = gated_delta_swapped ? PrefixStateBufferPlane::SecondOutput : PrefixStateBufferPlane::Second;
        canonical = PrefixStateBufferPlane::Second;
        break;
    case PrefixStateSegmentKind::AttentionKey:
        break;
    case PrefixStateSegmentKind::AttentionValue:
        live = canonical = PrefixStateBufferPlane::Second;
        break;
    }
    if (direction == PrefixStateTransferDirection::Snapshot) return {live, PrefixStateBufferPlane::Arena};
    return {PrefixStateBufferPlane::Arena, canonical};
}

inline PrefixStateTransferError validate_prefix_state_arena_extent(const PrefixStateLayout& layout, std::uint64_t arena_offset_bytes,
                                                                   std::uint64_t arena_capacity_bytes) noexcept {
    if (layout.total_bytes == 0) return PrefixStateTransferError::InvalidLayout;
    if (arena_offset_bytes > arena_capacity_bytes || layout.total_bytes > arena_capacity_bytes - arena_offset_bytes)
        return PrefixStateTransferError::ArenaOutOfRange;
    return PrefixStateTransferError::None;
}

// One bit per layer: the ping-pong phase each gated-delta layer was snapshotted in.
inline std::size_t prefix_state_phase_evidence_bytes(std::size_t layers) noexcept { return (layers + 7) / 8; }

// The layout of a pool of this library's geometry at `positions` prefix positions.
inline PrefixStateLayoutResult make_prefix_state_layout(const DecodeStatePool& pool, const std::vector<LayerKind>& schedule,
                                                        std::uint32_t positions) noexcept {
    using namespace state_transfer_detail;
    if (pool.capacity == 0 || schedule.size() != pool.layers.size()) return {PrefixStateLayoutError::InvalidGeometry, {}};
    PrefixStateLayoutSpec spec;
    spec.schedule = schedule.data();
    spec.layers = schedule.size();
    spec.capacity = pool.capacity;
    spec.positions = positions;
    spec.key_value_heads = kKeyValueHeads;
    spec.head_dimension = kHeadDimension;
    for (const LayerKind k : schedule) ++(k == LayerKind::GatedDelta ? spec.expected_gated_delta_layers : spec.expected_attention_layers);
    spec.gated_delta_convolution_bytes = kGdnConvStateValues * 2;
    spec.gated_delta_recurrent_bytes = kGdnRecurrentStateValues * 4;
    std::uint64_t per_position = 2ull * kKeyValueHeads * kHeadDimension * kBf16Bytes, attention = 0, gated = 0;
    if (!mul(per_position, positions, attention) || !mul(attention, spec.expected_attention_layers, attention) ||
        !mul(spec.gated_delta_convolution_bytes + spec.gated_delta_recurrent_bytes, spec.expected_gated_delta_layers, gated) ||
        !add(attention, gated, spec.expected_total_bytes))
        return {PrefixStateLayoutError::Overflow, {}};
    return make_prefix_state_layout(spec);
}

struct PrefixStateTransferTicket {
    PrefixStateTransferDirection direction{PrefixStateTransferDirection::Snapshot};
    const DecodeStatePool* owner{nullptr};
    DecodeStateSlot* state_owner{nullptr};
    const void* arena_owner{nullptr};
    std::uint32_t positions{0};
    std::uint64_t arena_offset_bytes{0};
    std::uint64_t state_bytes{0};
    std::uint64_t generation{0};
    bool pending{false};
};
struct PrefixStateTransferResult {
    PrefixStateTransferError error{PrefixStateTransferError::InvalidLayout};
    PrefixStateLayoutError layout_error{PrefixStateLayoutError::None};
    CommandError command_error{CommandError::None};
    std::uint32_t segment_count{0};
    std::uint64_t state_bytes{0};
    PrefixStateTransferTicket ticket;
    explicit operator bool() const noexcept { return error == PrefixStateTransferError::None && ticket.pending; }
};

namespace state_transfer_detail {
// Device address of (layer, plane) of one slot in a pooled allocation: gated-delta stripes are
// interleaved ping-pong pairs (2s, 2s+1), attention stripes are one per slot.
inline std::byte* plane_address(const DecodeStatePool& pool, const DecodeStateSlot& slot, std::uint32_t layer,
                                PrefixStateBufferPlane plane) noexcept {
    const DecodeStatePoolLayer& pl = pool.layers[layer];
    const bool second = plane == PrefixStateBufferPlane::Second || plane == PrefixStateBufferPlane::SecondOutput;
    const bool output = plane == PrefixStateBufferPlane::FirstOutput || plane == PrefixStateBufferPlane::SecondOutput;
    auto* base = static_cast<std::byte*>(second ? pl.second.data() : pl.first.data());
    if (pl.kind == LayerKind::FullAttention) {
        if (output) return nullptr;
        return base + std::uint64_t{slot.stripe} * pl.first_stride * kBf16Bytes;
    }
    const std::uint64_t stripe = 2ull * slot.stripe + (output ? 1u : 0u);
    return second ? base + stripe * pl.second_stride * 4 : base + stripe * pl.first_stride * kBf16Bytes;
}
inline bool slot_fits_pool(const DecodeStatePool& pool, const DecodeStateSlot& slot) noexcept {
    return slot.capacity == pool.capacity && slot.stripe < pool.stripes && slot.swapped.size() == pool.layers.size();
}
inline void clear_active_transfer(DecodeStateSlot& slot) noexcept {
    slot.active_transfer_generation = 0;
    slot.active_transfer_arena = nullptr;
    slot.active_transfer_positions = 0;
    slot.active_transfer_offset_bytes = 0;
    slot.active_transfer_state_bytes = 0;
}

inline PrefixStateTransferResult encode_transfer(PrefixStateTransferDirection direction, tatara_ctx* ctx, cudaStream_t stream,
                                                 const DecodeStatePool& pool, const std::vector<LayerKind>& schedule,
                                                 DecodeStateSlot& slot, DeviceBuffer& arena, std::uint64_t arena_offset_bytes,
                                                 std::uint32_t positions, std::byte* phase_evidence, std::size_t phase_capacity) {
    PrefixStateTransferResult result;
    const auto failure = [&](PrefixStateTransferError e, PrefixStateLayoutError le = PrefixStateLayoutError::None,
                             CommandError ce = CommandError::None) {
        result.error = e;
        result.layout_error = le;
        result.command_error = ce;
        return result;
    };
    if (slot.status == DecodeStateSlotStatus::Poisoned) return failure(PrefixStateTransferError::PoisonedStateSlot);
    if (!slot_fits_pool(pool, slot)) return failure(PrefixStateTransferError::InvalidStateSlot);
    if (slot.status != DecodeStateSlotStatus::Ready) return failure(PrefixStateTransferError::StateSlotNotReady);
    if (!arena) return failure(PrefixStateTransferError::InvalidArena);
    const std::size_t phase_bytes =
        direction == PrefixStateTransferDirection::Snapshot ? prefix_state_phase_evidence_bytes(schedule.size()) : 0;
    if (phase_bytes > phase_capacity) return failure(PrefixStateTransferError::PhaseEvidenceTooSmall);
    const PrefixStateLayoutResult planned = make_prefix_state_layout(pool, schedule, positions);
    if (!planned) return failure(PrefixStateTransferError::InvalidLayout, planned.error);
    const PrefixStateLayout& layout = planned.layout;
    if (validate_prefix_state_arena_extent(layout, arena_offset_bytes, arena.bytes()) != PrefixStateTransferError::None)
        return failure(PrefixStateTransferError::ArenaOutOfRange);
    if (arena_offset_bytes % 16u != 0) return failure(PrefixStateTransferError::ArenaOutOfRange);
    if (slot.next_transfer_generation == 0) return failure(PrefixStateTransferError::GenerationExhausted);
    if (ctx == nullptr) return failure(PrefixStateTransferError::CommandEncodingFailed, PrefixStateLayoutError::None, CommandError::InvalidDevice);

    // The whole plan is resolved to addresses before the one launch that executes it.
    std::vector<tatara_copy_segment> copies(layout.segment_count);
    for (std::uint32_t i = 0; i < layout.segment_count; ++i) {
        const PrefixStateSegmentResult selected = prefix_state_segment(layout, i);
        if (!selected || selected.segment.layer_index >= pool.layers.size())
            return failure(PrefixStateTransferError::InvalidLayout, selected.error);
        const PrefixStateSegment& seg = selected.segment;
        const PrefixStateCopyRoute route = prefix_state_copy_route(seg, direction, slot.swapped[seg.layer_index]);
        const PrefixStateBufferPlane slot_plane = direction == PrefixStateTransferDirection::Snapshot ? route.source : route.destination;
        std::byte* in_slot = plane_address(pool, slot, seg.layer_index, slot_plane);
        if (in_slot == nullptr) return failure(PrefixStateTransferError::InvalidStateSlot);
        std::byte* in_arena = static_cast<std::byte*>(arena.data()) + arena_offset_bytes + seg.snapshot_offset_bytes;
        in_slot += seg.slot_offset_bytes;
        copies[i] = direction == PrefixStateTransferDirection::Snapshot ? tatara_copy_segment{in_slot, in_arena, seg.length_bytes}
                                                                        : tatara_copy_segment{in_arena, in_slot, seg.length_bytes};
    }
    const tatara_status st = tatara_state_copy(ctx, stream, copies.data(), layout.segment_count);
    if (st != TATARA_OK) {
        slot.status = DecodeStateSlotStatus::Poisoned;
        clear_active_transfer(slot);
        return failure(PrefixStateTransferError::CommandEncodingFailed, PrefixStateLayoutError::None, to_command_error(st));
    }
    if (direction == PrefixStateTransferDirection::Snapshot) {
        for (std::size_t b = 0; b < phase_bytes; ++b) phase_evidence[b] = std::byte{0};
        for (std::size_t l = 0; l < schedule.size(); ++l)
            if (schedule[l] == LayerKind::GatedDelta && slot.swapped[l])
                phase_evidence[l / 8] |= std::byte(1u << (l % 8));
    }
    const std::uint64_t generation = slot.next_transfer_generation;
    slot.next_transfer_generation = generation == std::numeric_limits<std::uint64_t>::max() ? 0 : generation + 1;
    slot.active_transfer_generation = generation;
    slot.active_transfer_arena = arena.data();
    slot.active_transfer_positions = positions;
    slot.active_transfer_offset_bytes = arena_offset_bytes;
    slot.active_transfer_state_bytes = layout.total_bytes;
    slot.status = direction == PrefixStateTransferDirection::Snapshot ? DecodeStateSlotStatus::SnapshotPending
                                                                      : DecodeStateSlotStatus::RestorePending;
    result.error = PrefixStateTransferError::None;
    result.segment_count = layout.segment_count;
    result.state_bytes = layout.total_bytes;
    result.ticket = PrefixStateTransferTicket{direction, &pool, &slot, arena.data(), positions, arena_offset_bytes,
                                              layout.total_bytes, generation, true};
    return result;
}
inline bool ticket_matches(const PrefixStateTransferTicket& t, const DecodeStatePool& pool, const DecodeStateSlot& slot,
                           const DeviceBuffer& arena) noexcept {
    const DecodeStateSlotStatus expected = t.direction == PrefixStateTransferDirection::Snapshot
                                               ? DecodeStateSlotStatus::SnapshotPending
                                               : DecodeStateSlotStatus::RestorePending;
    return t.owner == &pool && t.state_owner == &slot && t.arena_owner == arena.data() && t.generation != 0 &&
           slot_fits_pool(pool, slot) && slot.active_transfer_generation == t.generation &&
           slot.active_transfer_arena == arena.data() && slot.active_transfer_positions == t.positions &&
           slot.active_transfer_offset_bytes == t.arena_offset_bytes && slot.active_transfer_state_bytes == t.state_bytes &&
           slot.status == expected;
}
} // namespace state_transfer_detail

// Enqueues slot -> arena copies of the first `positions` prefix positions; the slot is
// SnapshotPending until complete_prefix_state_transfer.  `phase_evidence` receives one bit per
// layer (the live ping-pong half of each gated-delta layer at snapshot time).
inline PrefixStateTransferResult encode_prefix_state_snapshot(tatara_ctx* ctx, cudaStream_t stream, const DecodeStatePool& pool,
                                                              const std::vector<LayerKind>& schedule, DecodeStateSlot& slot,
                                                              DeviceBuffer& arena, std::uint64_t arena_offset_bytes,
                                                              std::uint32_t positions, std::byte* phase_evidence,
                                                              std::size_t phase_capacity) {
    return state_transfer_detail::encode_transfer(PrefixStateTransferDirection::Snapshot, ctx, stream, pool, schedule, slot, arena,
                                                  arena_offset_bytes, positions, phase_evidence, phase_capacity);
}
// Enqueues arena -> slot copies into the canonical input halves; completion resets the phases.
inline PrefixStateTransferResult encode_prefix_state_restore(tatara_ctx* ctx, cudaStream_t stream, const DecodeStatePool& pool,
                                                             const std::vector<LayerKind>& schedule, DecodeStateSlot& slot,
                                                             DeviceBuffer& arena, std::uint64_t arena_offset_bytes,
                                                             std::uint32_t positions) {
    return state_transfer_detail::encode_transfer(PrefixStateTransferDirection::Restore, ctx, stream, pool, schedule, slot, arena,
                                                  arena_offset_bytes, positions, nullptr, 0);
}
// After the stream work has completed: the slot becomes Ready again; a restore leaves every
// gated-delta layer in the canonical phase.
inline PrefixStateTransferError complete_prefix_state_transfer(PrefixStateTransferTicket& ticket, const DecodeStatePool& pool,
                                                               DecodeStateSlot& slot, const DeviceBuffer& arena) noexcept {
    if (!ticket.pending) return PrefixStateTransferError::AlreadyCompleted;
    if (!state_transfer_detail::ticket_matches(ticket, pool, slot, arena)) return PrefixStateTransferError::StaleTicket;
    if (ticket.direction == PrefixStateTransferDirection::Restore)
        for (std::size_t l = 0; l < slot.swapped.size(); ++l) slot.swapped[l] = false;
    slot.status = DecodeStateSlotStatus::Ready;
    state_transfer_detail::clear_active_transfer(slot);
    ticket.pending = false;
    return PrefixStateTransferError::None;
}
// A transfer whose stream work failed: a snapshot leaves the slot usable, a restore poisons it.
inline PrefixStateTransferError abort_prefix_state_transfer(PrefixStateTransferTicket& ticket, const DecodeStatePool& pool,
                                                            DecodeStateSlot& slot, const DeviceBuffer& arena) noexcept {
    if (!ticket.pending) return PrefixStateTransferError::AlreadyCompleted;
    if (!state_transfer_detail::ticket_matches(ticket, pool, slot, arena)) return PrefixStateTransferError::StaleTicket;
    slot.status = ticket.direction == PrefixStateTransferDirection::Snapshot ? DecodeStateSlotStatus::Ready
                                                                             : DecodeStateSlotStatus::Poisoned;
    state_transfer_detail::clear_active_transfer(slot);
    ticket.pending = false;
    return PrefixStateTransferError::None;
}

// ---- `Q36BRS01` state record (tools/native/decode_harness.cpp:339-461) ---------------------
inline constexpr char kStateRecordMagic[8] = {'Q', '3', '6', 'B', 'R', 'S', '0', '1'};
enum class StateRecordError : std::uint8_t { None, MagicMismatch, PositionOutOfRange, Truncated, UnconsumedBytes, InvalidStateSlot, CopyFailed };

inline std::uint64_t state_record_bytes(const std::vector<LayerKind>& schedule, std::uint32_t positions) noexcept {
    std::uint64_t total = 12;
    for (const LayerKind k : schedule)
        total += k == LayerKind::GatedDelta ? kGdnConvStateValues * 2 + kGdnRecurrentStateValues * 4
                                            : 2ull * kKeyValueHeads * positions * kHeadDimension * kBf16Bytes;
    return total;
}

// Serialises the live state of one slot (synchronous device-to-host copies).
inline StateRecordError write_state_record(const DecodeStatePool& pool, const std::vector<LayerKind>& schedule,
                                           const DecodeStateSlot& slot, std::uint32_t positions, std::vector<std::byte>& record) {
    using namespace state_transfer_detail;
    if (!slot_fits_pool(pool, slot) || schedule.size() != pool.layers.size()) return StateRecordError::InvalidStateSlot;
    if (positions == 0 || positions > pool.capacity) return StateRecordError::PositionOutOfRange;
    record.assign(state_record_bytes(schedule, positions), std::byte{0});
    std::memcpy(record.data(), kStateRecordMagic, 8);
    std::memcpy(record.data() + 8, &positions, 4);
    std::size_t cursor = 12;
    const auto pull = [&](const std::byte* device, std::uint64_t bytes) {
        const bool ok = cudaMemcpy(record.data() + cursor, device, bytes, cudaMemcpyDeviceToHost) == cudaSuccess;
        cursor += bytes;
        return ok;
    };
    const std::uint64_t head_bytes = std::uint64_t{positions} * kHeadDimension * kBf16Bytes;
    const std::uint64_t head_stride = std::uint64_t{pool.capacity} * kHeadDimension * kBf16Bytes;
    for (std::uint32_t l = 0; l < schedule.size(); ++l) {
        if (schedule[l] == LayerKind::GatedDelta) {
            const bool out = slot.swapped[l];
            if (!pull(plane_address(pool, slot, l, out ? PrefixStateBufferPlane::FirstOutput : PrefixStateBufferPlane::First),
                      kGdnConvStateValues * 2) ||
                !pull(plane_address(pool, slot, l, out ? PrefixStateBufferPlane::SecondOutput : PrefixStateBufferPlane::Second),
                      kGdnRecurrentStateValues * 4))
                return StateRecordError::CopyFailed;
        } else {
            for (const PrefixStateBufferPlane plane : {PrefixStateBufferPlane::First, PrefixStateBufferPlane::Second})
                for (std::uint32_t head = 0; head < kKeyValueHeads; ++head)
                    if (!pull(plane_address(pool, slot, l, plane) + head * head_stride, head_bytes)) return StateRecordError::CopyFailed;
        }
    }
    return StateRecordError::None;
}

// Installs a record into a slot: gated-delta planes into the canonical input halves (phase
// reset), K/V prefixes into positions [0, count).  The record is validated in full (magic,
// position count, exact length) before the first byte is copied.
inline StateRecordError load_state_record(const std::byte* record, std::size_t record_bytes, const DecodeStatePool& pool,
                                          const std::vector<LayerKind>& schedule, DecodeStateSlot& slot, std::uint32_t* positions_out) {
    using namespace state_transfer_detail;
    if (record == nullptr || record_bytes < 12 || std::memcmp(record, kStateRecordMagic, 8) != 0) return StateRecordError::MagicMismatch;
    std::uint32_t count = 0;
    std::memcpy(&count, record + 8, 4);
    if (count == 0 || count > pool.capacity) return StateRecordError::PositionOutOfRange;
    if (!slot_fits_pool(pool, slot) || schedule.size() != pool.layers.size()) return StateRecordError::InvalidStateSlot;
    const std::uint64_t need = state_record_bytes(schedule, count);
    if (record_bytes < need) return StateRecordError::Truncated;
    if (record_bytes > need) return StateRecordError::UnconsumedBytes;
    std::size_t cursor = 12;
    const auto push = [&](std::byte* device, std::uint64_t bytes) {
        const bool ok = cudaMemcpy(device, record + cursor, bytes, cudaMemcpyHostToDevice) == cudaSuccess;
        cursor += bytes;
        return ok;
    };
    const std::uint64_t head_bytes = std::uint64_t{count} * kHeadDimension * kBf16Bytes;
    const std::uint64_t head_stride = std::uint64_t{pool.capacity} * kHeadDimension * kBf16Bytes;
    for (std::uint32_t l = 0; l < schedule.size(); ++l) {
        if (schedule[l] == LayerKind::GatedDelta) {
            if (!push(plane_address(pool, slot, l, PrefixStateBufferPlane::First), kGdnConvStateValues * 2) ||
                !push(plane_address(pool, slot, l, PrefixStateBufferPlane::Second), kGdnRecurrentStateValues * 4))
                return StateRecordError::CopyFailed;
            slot.swapped[l] = false;
        } else {
            for (const PrefixStateBufferPlane plane : {PrefixStateBufferPlane::First, PrefixStateBufferPlane::Second})
                for (std::uint32_t head = 0; head < kKeyValueHeads; ++head)
                    if (!push(plane_address(pool, slot, l, plane) + head * head_stride, head_bytes)) return StateRecordError::CopyFailed;
        }
    }
    if (positions_out != nullptr) *positions_out = count;
    return StateRecordError::None;
}

// ---- speculative-decode rollback (src/engine/speculative_decode.cpp:517-596) -----------------
// After a verify band of at most 16 rows was run with the tape kernels and only `committed` rows
// were accepted: the caller has put the pre-band gated-delta state back into the slot's live
// halves; this replays `committed` taped rows from each live recurrent plane into its partner
// and installs the conv tail recorded after row committed-1 into the partner conv plane (all conv
// tails in one tatara_state_copy launch).  When the stream has completed, advance_decode_state
// flips the halves, exactly as after a decode token.
inline CommandError encode_gdn_tape_rollback(tatara_ctx* ctx, cudaStream_t stream, const DecodeStatePool& pool,
                                             const std::vector<LayerKind>& schedule, const DecodeStateSlot& slot,
                                             const void* tape, const void* conv_tape, std::uint32_t committed) {
    using namespace state_transfer_detail;
    if (ctx == nullptr) return CommandError::InvalidDevice;
    if (tape == nullptr || conv_tape == nullptr) return CommandError::InvalidBuffer;
    if (committed == 0 || committed > 16u || schedule.size() > 40u) return CommandError::InvalidDispatchExtent;
    if (!slot_fits_pool(pool, slot) || schedule.size() != pool.layers.size() || slot.status != DecodeStateSlotStatus::Ready)
        return CommandError::StateSlotMismatch;
    const std::uint64_t conv_row_bytes = kGdnConvStateValues * 2;
    std::vector<tatara_copy_segment> tails;
    for (std::uint32_t l = 0; l < schedule.size(); ++l) {
        if (schedule[l] != LayerKind::GatedDelta) continue;
        const bool swapped = slot.swapped[l];
        const std::byte* rec_in = plane_address(pool, slot, l, swapped ? PrefixStateBufferPlane::SecondOutput : PrefixStateBufferPlane::Second);
        std::byte* rec_out = plane_address(pool, slot, l, swapped ? PrefixStateBufferPlane::Second : PrefixStateBufferPlane::SecondOutput);
        const tatara_status st = tatara_gdn_tape_replay(ctx, stream, tape, rec_in, rec_out, committed, l);
        if (st != TATARA_OK) return to_command_error(st);
        std::byte* conv_out = plane_address(pool, slot, l, swapped ? PrefixStateBufferPlane::First : PrefixStateBufferPlane::FirstOutput);
        tails.push_back(tatara_copy_segment{static_cast<const std::byte*>(conv_tape) + (std::uint64_t{l} * 16u + (committed - 1u)) * conv_row_bytes,
                                            conv_out, conv_row_bytes});
    }
    if (tails.empty()) return CommandError::None;
    const tatara_status st = tatara_state_copy(ctx, stream, tails.data(), static_cast<std::uint32_t>(tails.size()));
    return st == TATARA_OK ? CommandError::None : to_command_error(st);
}

} // namespace tatara::runtime
