// Native test of the C++ host layer (tatara_b200/host/hybrid_layers.hpp) over the C ABI, in the
// style of the reference's tests (tests/native/*_test.cpp: plain main(), a distinct non-zero exit
// code per failed check).  Host-only checks always run; the device checks run when a B200 is
// present: a two-layer slice (gated delta + full attention), three lanes at different contexts,
// three decode tokens batched, compared with the CPU oracle and, bit for bit, with solo runs.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <utility>
#include <vector>

#include "../../tatara_b200/host/state_transfer.hpp"

using namespace tatara::runtime;
using u16 = std::uint16_t;

extern "C" {  // oracle/tatara_oracle.cpp (test infrastructure)
void orc_attn_qk_rope(const u16*, const u16*, const u16*, u16*, u16*, u16*, u16*, std::uint32_t, std::uint32_t, std::uint32_t);
void orc_attn_decode(const u16*, const u16*, const u16*, const u16*, std::uint32_t, std::uint32_t, u16*, int);
void orc_gdn_prepare(const u16*, const u16*, const u16*, u16*, u16*, u16*, u16*, std::uint32_t);
void orc_gdn_gates(const u16*, std::uint32_t, const u16*, const u16*, float*, float*, std::uint32_t);
void orc_gdn_scan(const u16*, const u16*, const float*, const float*, const float*, u16*, float*, std::uint32_t, int);
void orc_gdn_gate_norm(const u16*, const u16*, const u16*, u16*, std::uint32_t);
void orc_q4_project(const u16*, std::uint32_t, std::uint32_t, const std::uint32_t*, const u16*, const u16*, std::uint32_t,
                    std::uint32_t, u16*, std::uint32_t, int, int);
}

namespace {

u16 to_bf16(float v) {
    std::uint32_t b;
    std::memcpy(&b, &v, 4);
    return static_cast<u16>((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
float from_bf16(u16 h) {
    const std::uint32_t b = static_cast<std::uint32_t>(h) << 16;
    float v;
    std::memcpy(&v, &b, 4);
    return v;
}
struct Rng {
    std::uint64_t s;
    std::uint64_t next() { s ^= s >> 12; s ^= s << 25; s ^= s >> 27; return s * 0x2545F4914F6CDD1Dull; }
    float uniform() { return static_cast<float>(next() >> 40) / 16777216.0f; }
    float normal() { float a = 0; for (int i = 0; i < 12; ++i) a += uniform(); return a - 6.0f; }
    void fill(std::vector<u16>& v, float scale = 1.0f, float shift = 0.0f) { for (auto& x : v) x = to_bf16(shift + scale * normal()); }
};
template <class T>
bool upload(void* dst, const std::vector<T>& src) { return cudaMemcpy(dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice) == cudaSuccess; }
bool close_enough(const std::vector<u16>& got, const u16* want, std::size_t n, float max_abs) {
    double dot = 0, na = 0, nb = 0;
    float worst = 0;
    for (std::size_t i = 0; i < n; ++i) {
        const float a = from_bf16(got[i]), b = from_bf16(want[i]);
        if (!std::isfinite(a)) return false;
        worst = std::fmax(worst, std::fabs(a - b));
        dot += double(a) * b; na += double(a) * a; nb += double(b) * b;
    }
    const double cosine = (na == 0 && nb == 0) ? 1.0 : dot / std::sqrt(na * nb);
    return worst <= max_abs && cosine >= 0.9999;
}

int host_only_checks() {
    if (context_in_capacity(0, 0) || !context_in_capacity(7, 8) || context_in_capacity(8, 8)) return 10;
    if (std::strcmp(to_string(CommandError::ContextOutOfRange), "ContextOutOfRange") != 0) return 11;
    if (std::strcmp(to_string(CommandError::StateSlotMismatch), "StateSlotMismatch") != 0) return 12;
    if (std::strcmp(to_string(CommandError::None), "None") != 0) return 13;
    LayerPass pass(nullptr, nullptr);
    if (pass.error() != CommandError::InvalidDevice) return 14;
    DecodeStatePool pool;
    DecodeBatchScratch scratch;
    if (pass.encode_attention(pool, 0, AttentionWeights{}, {}, nullptr, scratch) != CommandError::InvalidDevice) return 15;
    if (pass.encode_gated_delta(pool, 0, GatedDeltaWeights{}, {}, nullptr, scratch) != CommandError::InvalidDevice) return 16;
    if (tatara_attn_partition_keys(1) != 128 || tatara_attn_partitions(9472) != 74) return 17;
    if (tatara_attn_decode_scratch_bytes(4097, 2) != 2 * tatara_attn_decode_scratch_bytes(4097, 1)) return 18;
    return 0;
}

int device_checks(tatara_ctx* ctx) {
    constexpr std::uint32_t kSlots = 3, kCapacity = 512, kTokens = 3;
    const std::vector<LayerKind> schedule{LayerKind::GatedDelta, LayerKind::FullAttention};
    const std::uint32_t start_context[kSlots] = {5, 200, 300};
    Rng rng{0x51A7E5ull};

    // weights
    std::vector<u16> qn(256), kn(256), conv_w(8192 * 4), a_log(32), dt_bias(32), gnorm(128);
    rng.fill(qn, 0.1f, 1.0f); rng.fill(kn, 0.1f, 1.0f); rng.fill(conv_w, 0.5f); rng.fill(dt_bias, 0.5f); rng.fill(gnorm, 0.1f, 1.0f);
    for (auto& x : a_log) x = to_bf16(std::log(1.0f + 15.0f * rng.uniform()));
    DeviceBuffer d_qn(512), d_kn(512), d_conv(8192 * 8), d_alog(64), d_dt(64), d_gn(256);
    if (!upload(d_qn.data(), qn) || !upload(d_kn.data(), kn) || !upload(d_conv.data(), conv_w) ||
        !upload(d_alog.data(), a_log) || !upload(d_dt.data(), dt_bias) || !upload(d_gn.data(), gnorm)) return 20;
    const AttentionWeights aw{d_qn.data(), d_kn.data()};
    const GatedDeltaWeights gw{d_conv.data(), d_alog.data(), d_dt.data(), d_gn.data()};

    // two identical pools: one driven batched, one driven lane by lane
    DecodeStatePool pool[2];
    std::vector<DecodeStateSlot> slots[2];
    DecodeBatchScratch scratch[2];
    for (int p = 0; p < 2; ++p)
        if (!create_state_pool(kSlots, kCapacity, schedule, pool[p], slots[p]) ||
            !create_batch_scratch(kSlots, kCapacity, scratch[p])) return 21;

    // host mirrors for the oracle
    struct HostLane {
        std::vector<u16> keys, values, conv;
        std::vector<float> state;
    };
    std::vector<HostLane> host(kSlots);
    for (std::uint32_t s = 0; s < kSlots; ++s) {
        HostLane& h = host[s];
        h.keys.assign(2 * kCapacity * 256, 0); h.values.assign(2 * kCapacity * 256, 0);
        h.conv.resize(3 * 8192); rng.fill(h.conv);
        h.state.resize(32 * 128 * 128);
        for (auto& x : h.state) x = 0.02f * rng.normal();
        // history: fill positions 0..context-1 through the library, mirror with the oracle
        std::vector<u16> hist(std::size_t{start_context[s]} * 9216); rng.fill(hist);
        DeviceBuffer d_hist(hist.size() * 2), d_q(std::size_t{start_context[s]} * 4096 * 2), d_g(std::size_t{start_context[s]} * 4096 * 2);
        if (!upload(d_hist.data(), hist)) return 22;
        std::vector<u16> oq(std::size_t{start_context[s]} * 4096), og(oq.size());
        orc_attn_qk_rope(hist.data(), qn.data(), kn.data(), oq.data(), og.data(), h.keys.data(), h.values.data(), 0, kCapacity, start_context[s]);
        for (int p = 0; p < 2; ++p) {
            const DecodeStatePoolLayer& al = pool[p].layers[1];
            u16* k = static_cast<u16*>(al.first.data()) + s * al.first_stride;
            u16* v = static_cast<u16*>(al.second.data()) + s * al.second_stride;
            if (tatara_attn_qk_rope(ctx, nullptr, d_hist.data(), d_qn.data(), d_kn.data(), d_q.data(), d_g.data(), k, v, 0,
                                    kCapacity, start_context[s]) != TATARA_OK) return 23;
            const DecodeStatePoolLayer& gl = pool[p].layers[0];
            if (!upload(static_cast<u16*>(gl.first.data()) + 2 * s * gl.first_stride, h.conv) ||
                !upload(static_cast<float*>(gl.second.data()) + 2 * s * gl.second_stride, h.state)) return 24;
        }
    }
    if (tatara_ctx_sync(ctx, nullptr) != TATARA_OK) return 25;

    DeviceBuffer d_gproj(kSlots * 12352 * 2), d_aproj(kSlots * 9216 * 2);
    std::vector<u16> batched_attn(kSlots * 4096), batched_gdn(kSlots * 4096), solo(4096);
    for (std::uint32_t token = 0; token < kTokens; ++token) {
        std::vector<u16> gproj(kSlots * 12352), aproj(kSlots * 9216);
        rng.fill(gproj); rng.fill(aproj);
        if (!upload(d_gproj.data(), gproj) || !upload(d_aproj.data(), aproj)) return 30;
        std::vector<DecodeStream> streams;
        for (std::uint32_t s = 0; s < kSlots; ++s) streams.push_back(DecodeStream{&slots[0][s], start_context[s] + token});
        LayerPass pass(ctx, nullptr);
        if (pass.encode_gated_delta(pool[0], 0, gw, streams, d_gproj.data(), scratch[0]) != CommandError::None) return 31;
        if (pass.encode_attention(pool[0], 1, aw, streams, d_aproj.data(), scratch[0]) != CommandError::None) return 32;
        if (pass.commit_and_wait() != CommandError::None) return 33;
        cudaMemcpy(batched_gdn.data(), scratch[0].gdn_gated.data(), batched_gdn.size() * 2, cudaMemcpyDeviceToHost);
        cudaMemcpy(batched_attn.data(), scratch[0].attended.data(), batched_attn.size() * 2, cudaMemcpyDeviceToHost);
        advance_decode_state(pool[0], streams);

        for (std::uint32_t s = 0; s < kSlots; ++s) {
            // oracle for this lane and token
            HostLane& h = host[s];
            const std::uint32_t context = start_context[s] + token;
            std::vector<u16> qk(4096), v(4096), z(4096), conv_out(3 * 8192), y(4096), gated(4096);
            std::vector<float> decay(32), beta(32), state_out(h.state.size());
            orc_gdn_prepare(&gproj[s * 12352], h.conv.data(), conv_w.data(), qk.data(), v.data(), z.data(), conv_out.data(), 1);
            orc_gdn_gates(&gproj[s * 12352], 12352, a_log.data(), dt_bias.data(), decay.data(), beta.data(), 1);
            orc_gdn_scan(qk.data(), v.data(), decay.data(), beta.data(), h.state.data(), y.data(), state_out.data(), 1, 4);
            orc_gdn_gate_norm(y.data(), z.data(), gnorm.data(), gated.data(), 1);
            h.conv = conv_out; h.state = state_out;
            std::vector<u16> oq(4096), og(4096), want(4096);
            orc_attn_qk_rope(&aproj[s * 9216], qn.data(), kn.data(), oq.data(), og.data(), h.keys.data(), h.values.data(), context, kCapacity, 1);
            orc_attn_decode(oq.data(), og.data(), h.keys.data(), h.values.data(), context, kCapacity, want.data(), 4);
            const std::vector<u16> got_attn(batched_attn.begin() + s * 4096, batched_attn.begin() + (s + 1) * 4096);
            const std::vector<u16> got_gdn(batched_gdn.begin() + s * 4096, batched_gdn.begin() + (s + 1) * 4096);
            if (!close_enough(got_attn, want.data(), 4096, 2e-2f)) return 40 + int(s);
            if (!close_enough(got_gdn, gated.data(), 4096, 4e-2f)) return 50 + int(s);

            // the same lane alone on the second pool: bit-identical (lossless concurrency)
            DeviceBuffer d_g1(12352 * 2), d_a1(9216 * 2);
            cudaMemcpy(d_g1.data(), &gproj[s * 12352], 12352 * 2, cudaMemcpyHostToDevice);
            cudaMemcpy(d_a1.data(), &aproj[s * 9216], 9216 * 2, cudaMemcpyHostToDevice);
            const std::vector<DecodeStream> one{DecodeStream{&slots[1][s], context}};
            LayerPass solo_pass(ctx, nullptr);
            if (solo_pass.encode_gated_delta(pool[1], 0, gw, one, d_g1.data(), scratch[1]) != CommandError::None) return 60;
            if (solo_pass.encode_attention(pool[1], 1, aw, one, d_a1.data(), scratch[1]) != CommandError::None) return 61;
            if (solo_pass.commit_and_wait() != CommandError::None) return 62;
            cudaMemcpy(solo.data(), scratch[1].attended.data(), 4096 * 2, cudaMemcpyDeviceToHost);
            if (std::memcmp(solo.data(), got_attn.data(), 4096 * 2) != 0) return 70 + int(s);
            cudaMemcpy(solo.data(), scratch[1].gdn_gated.data(), 4096 * 2, cudaMemcpyDeviceToHost);
            if (std::memcmp(solo.data(), got_gdn.data(), 4096 * 2) != 0) return 80 + int(s);
            advance_decode_state(pool[1], one);
        }
    }

    // error behaviour: out-of-range context is refused before anything is enqueued, latches, and
    // gates the rest of the pass
    {
        const std::uint64_t before = tatara_ctx_launch_count(ctx);
        std::vector<DecodeStream> streams{DecodeStream{&slots[0][0], kCapacity}};
        LayerPass pass(ctx, nullptr);
        if (pass.encode_attention(pool[0], 1, aw, streams, d_aproj.data(), scratch[0]) != CommandError::ContextOutOfRange) return 90;
        streams[0].context = 1;
        if (pass.encode_attention(pool[0], 1, aw, streams, d_aproj.data(), scratch[0]) != CommandError::ContextOutOfRange) return 91;
        if (pass.commit_and_wait() != CommandError::ContextOutOfRange) return 92;
        if (tatara_ctx_launch_count(ctx) != before) return 93;
        LayerPass wrong(ctx, nullptr);
        if (wrong.encode_attention(pool[0], 0, aw, streams, d_aproj.data(), scratch[0]) != CommandError::StateSlotMismatch) return 94;
        LayerPass dup(ctx, nullptr);
        std::vector<DecodeStream> twice{DecodeStream{&slots[0][0], 1}, DecodeStream{&slots[0][0], 2}};
        if (dup.encode_gated_delta(pool[0], 0, gw, twice, d_gproj.data(), scratch[0]) != CommandError::InvalidStreamGroup) return 95;
        slots[0][1].status = DecodeStateSlotStatus::Poisoned;
        LayerPass poisoned(ctx, nullptr);
        std::vector<DecodeStream> bad{DecodeStream{&slots[0][1], 1}};
        if (poisoned.encode_gated_delta(pool[0], 0, gw, bad, d_gproj.data(), scratch[0]) != CommandError::StateSlotMismatch) return 96;
    }
    return 0;
}

} // namespace

// Projection encoders: gdn_project geometry (four matrices, 12352 columns) for two rows, bit for bit
// against the oracle's fused chain, and the latched error for an empty row group.
int projection_checks(tatara_ctx* ctx) {
    Rng rng{0xC0FFEEull};
    constexpr std::uint32_t k = kHidden, rows = 2;
    const std::uint32_t sizes[4] = {8192, 4096, 32, 32};
    std::vector<std::vector<std::uint32_t>> words(4);
    std::vector<std::vector<u16>> scales(4), biases(4);
    std::vector<DeviceBuffer> dw, ds, db;
    QuantizedWeight q[4];
    for (int m = 0; m < 4; ++m) {
        words[m].resize(std::size_t{sizes[m]} * k / 8);
        for (auto& w : words[m]) w = static_cast<std::uint32_t>(rng.next());
        scales[m].resize(std::size_t{sizes[m]} * k / 64);
        biases[m].resize(scales[m].size());
        for (std::size_t i = 0; i < scales[m].size(); ++i) {
            const float sc = 0.0025f * (1.0f + 0.2f * (2.0f * rng.uniform() - 1.0f));
            scales[m][i] = to_bf16(sc);
            biases[m][i] = to_bf16(-7.5f * sc * (1.0f + 0.1f * rng.normal()));
        }
        dw.emplace_back(words[m].size() * 4); ds.emplace_back(scales[m].size() * 2); db.emplace_back(biases[m].size() * 2);
        if (!upload(dw.back().data(), words[m]) || !upload(ds.back().data(), scales[m]) || !upload(db.back().data(), biases[m])) return 60;
        q[m] = QuantizedWeight{dw.back().data(), ds.back().data(), db.back().data(), sizes[m]};
    }
    std::vector<u16> x(rows * k); rng.fill(x);
    DeviceBuffer dx(x.size() * 2), dout(std::size_t{rows} * kGdnProjectionRows * 2);
    if (!upload(dx.data(), x)) return 61;
    LayerPass pass(ctx, nullptr);
    const GatedDeltaProjection gp{q[0], q[1], q[2], q[3], QuantizedWeight{}};
    if (pass.encode_gated_delta_project(gp, dx.data(), rows, dout.data()) != CommandError::None) return 62;
    if (pass.commit_and_wait() != CommandError::None) return 63;
    std::vector<u16> got(std::size_t{rows} * kGdnProjectionRows), want(got.size());
    if (cudaMemcpy(got.data(), dout.data(), got.size() * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return 64;
    std::uint32_t col = 0;
    for (int m = 0; m < 4; ++m) {
        orc_q4_project(x.data(), k, rows, words[m].data(), scales[m].data(), biases[m].data(), sizes[m], k,
                       want.data() + col, kGdnProjectionRows, 1, 4);
        col += sizes[m];
    }
    if (std::memcmp(got.data(), want.data(), got.size() * 2) != 0) return 65;
    LayerPass bad(ctx, nullptr);
    if (bad.encode_gated_delta_project(gp, dx.data(), 0, dout.data()) != CommandError::InvalidStreamGroup) return 66;
    if (bad.encode_out_projection(q[1], dx.data(), 1, dout.data(), kHidden) != CommandError::InvalidStreamGroup) return 67;  // latched
    return 0;
}

// Canonical prefix-state layout: the reference's frozen figures (tests/native/prefix_state_transfer_test.cpp:
// 223-231, 236-262, 376-432) restated as checks on this planner.
int layout_checks() {
    std::vector<LayerKind> model(40);
    for (std::size_t l = 0; l < model.size(); ++l) model[l] = (l % 4 == 3) ? LayerKind::FullAttention : LayerKind::GatedDelta;
    const std::pair<std::uint32_t, std::uint64_t> frozen[4] = {
        {4096, 148275200ull}, {49408, 1076264960ull}, {50000, 1088389120ull}, {65536, 1406566400ull}};
    for (const auto& [positions, bytes] : frozen) {
        PrefixStateLayoutSpec spec{model.data(), model.size(), 65536, positions, 2, 256, 30, 10, 49152, 2097152, bytes};
        const PrefixStateLayoutResult r = make_prefix_state_layout(spec);
        if (!r || r.layout.segment_count != 100 || r.layout.total_bytes != bytes) return 70;
    }
    PrefixStateLayoutSpec spec{model.data(), model.size(), 16384, 4096, 2, 256, 30, 10, 49152, 2097152, 148275200ull};
    const PrefixStateLayoutResult planned = make_prefix_state_layout(spec);
    if (!planned || planned.layout.gated_delta_layers != 30 || planned.layout.attention_layers != 10) return 71;
    if (planned.layout.attention_segment_bytes != 2097152 || planned.layout.attention_slot_head_stride_bytes != 8388608) return 72;
    if (prefix_state_phase_evidence_bytes(model.size()) != 5) return 73;
    // segments tile the payload exactly, family-major, each family in schedule order
    std::uint64_t next = 0;
    std::uint32_t gated = 0, attention = 0;
    for (std::uint32_t i = 0; i < planned.layout.segment_count; ++i) {
        const PrefixStateSegmentResult s = prefix_state_segment(planned.layout, i);
        if (!s || s.segment.snapshot_offset_bytes != next) return 74;
        next += s.segment.length_bytes;
        const bool g = s.segment.kind == PrefixStateSegmentKind::GatedDeltaConvolution || s.segment.kind == PrefixStateSegmentKind::GatedDeltaRecurrent;
        if ((model[s.segment.layer_index] == LayerKind::GatedDelta) != g) return 75;
        ++(g ? gated : attention);
    }
    if (next != planned.layout.total_bytes || gated != 60 || attention != 40) return 76;
    const PrefixStateSegment a0 = prefix_state_segment(planned.layout, 60).segment, a1 = prefix_state_segment(planned.layout, 61).segment,
                             v0 = prefix_state_segment(planned.layout, 62).segment;
    if (a0.layer_index != 3 || a0.kind != PrefixStateSegmentKind::AttentionKey || a0.head_index != 0 || a0.slot_offset_bytes != 0) return 77;
    if (a1.kind != PrefixStateSegmentKind::AttentionKey || a1.head_index != 1 || a1.slot_offset_bytes != 8388608) return 78;
    if (v0.kind != PrefixStateSegmentKind::AttentionValue || v0.head_index != 0) return 79;
    if (validate_prefix_state_arena_extent(planned.layout, 64, planned.layout.total_bytes + 64) != PrefixStateTransferError::None) return 80;
    if (validate_prefix_state_arena_extent(planned.layout, 64, planned.layout.total_bytes + 63) != PrefixStateTransferError::ArenaOutOfRange) return 81;
    // copy routes: snapshot reads the live half, restore writes the canonical input half
    const PrefixStateSegment conv = prefix_state_segment(planned.layout, 0).segment, rec = prefix_state_segment(planned.layout, 1).segment;
    if (prefix_state_copy_route(conv, PrefixStateTransferDirection::Snapshot, false).source != PrefixStateBufferPlane::First ||
        prefix_state_copy_route(conv, PrefixStateTransferDirection::Snapshot, true).source != PrefixStateBufferPlane::FirstOutput ||
        prefix_state_copy_route(rec, PrefixStateTransferDirection::Snapshot, true).source != PrefixStateBufferPlane::SecondOutput) return 82;
    const PrefixStateCopyRoute rc = prefix_state_copy_route(conv, PrefixStateTransferDirection::Restore, true);
    if (rc.source != PrefixStateBufferPlane::Arena || rc.destination != PrefixStateBufferPlane::First ||
        prefix_state_copy_route(rec, PrefixStateTransferDirection::Restore, true).destination != PrefixStateBufferPlane::Second) return 83;
    // a small mixed schedule and the typed failures
    const LayerKind mixed[4] = {LayerKind::FullAttention, LayerKind::GatedDelta, LayerKind::FullAttention, LayerKind::GatedDelta};
    const PrefixStateLayoutSpec small{mixed, 4, 19, 7, 4, 8, 2, 2, 24, 40, 1920};
    const PrefixStateLayoutResult synthetic = make_prefix_state_layout(small);
    if (!synthetic || synthetic.layout.segment_count != 20 || synthetic.layout.total_bytes != 1920) return 84;
    if (prefix_state_segment(synthetic.layout, 0).segment.layer_index != 1 || prefix_state_segment(synthetic.layout, 4).segment.layer_index != 0) return 85;
    PrefixStateLayoutSpec bad = small;
    bad.positions = 0;
    if (make_prefix_state_layout(bad).error != PrefixStateLayoutError::PositionOutOfRange) return 86;
    bad.positions = 20;
    if (make_prefix_state_layout(bad).error != PrefixStateLayoutError::PositionOutOfRange) return 87;
    bad = small; bad.expected_attention_layers = 3;
    if (make_prefix_state_layout(bad).error != PrefixStateLayoutError::FamilyCountMismatch) return 88;
    bad = small; ++bad.expected_total_bytes;
    if (make_prefix_state_layout(bad).error != PrefixStateLayoutError::TotalMismatch) return 89;
    bad = small; bad.gated_delta_convolution_bytes = ~0ull;
    if (make_prefix_state_layout(bad).error != PrefixStateLayoutError::Overflow) return 90;
    const LayerKind unknown[2] = {LayerKind::GatedDelta, static_cast<LayerKind>(255)};
    bad = small; bad.schedule = unknown; bad.layers = 2; bad.expected_gated_delta_layers = 1; bad.expected_attention_layers = 1;
    if (make_prefix_state_layout(bad).error != PrefixStateLayoutError::InvalidSchedule) return 91;
    if (prefix_state_segment(synthetic.layout, 20).error != PrefixStateLayoutError::SegmentOutOfRange) return 92;
    // state record framing
    const std::vector<LayerKind> two{LayerKind::GatedDelta, LayerKind::FullAttention};
    if (state_record_bytes(two, 5) != 12 + 49152 + 2097152 + 2 * 2 * 5 * 512) return 93;
    DecodeStatePool none;
    DecodeStateSlot slot;
    const std::byte junk[16] = {};
    if (load_state_record(junk, sizeof(junk), none, two, slot, nullptr) != StateRecordError::MagicMismatch) return 94;
    return 0;
}

// Snapshot -> scribble -> restore through one launch each, from a swapped phase; and the state
// record written from one slot and loaded into another.
int transfer_checks(tatara_ctx* ctx) {
    constexpr std::uint32_t kCapacity = 96, kPositions = 40;
    const std::vector<LayerKind> schedule{LayerKind::GatedDelta, LayerKind::FullAttention, LayerKind::GatedDelta};
    DecodeStatePool pool;
    std::vector<DecodeStateSlot> slots;
    if (!create_state_pool(2, kCapacity, schedule, pool, slots)) return 100;
    Rng rng{0xABCDull};
    // fill every pool buffer with noise
    for (auto& pl : pool.layers)
        for (DeviceBuffer* b : {&pl.first, &pl.second}) {
            std::vector<std::uint32_t> noise(b->bytes() / 4);
            for (auto& w : noise) w = static_cast<std::uint32_t>(rng.next());
            if (!upload(b->data(), noise)) return 101;
        }
    DecodeStateSlot& slot = slots[1];
    slot.swapped[0] = true;   // layer 0 live in the output half, layer 2 in the input half
    const PrefixStateLayoutResult planned = make_prefix_state_layout(pool, schedule, kPositions);
    if (!planned || planned.layout.segment_count != 8) return 102;
    DeviceBuffer arena(planned.layout.total_bytes + 256);
    std::byte evidence[1] = {};
    PrefixStateTransferResult snap = encode_prefix_state_snapshot(ctx, nullptr, pool, schedule, slot, arena, 256, kPositions, evidence, 1);
    if (!snap || snap.segment_count != 8 || snap.state_bytes != planned.layout.total_bytes) return 103;
    if (slot.status != DecodeStateSlotStatus::SnapshotPending || evidence[0] != std::byte{1}) return 104;
    // a pending slot refuses layer work and a second transfer
    {
        LayerPass pass(ctx, nullptr);
        DecodeBatchScratch scratch;
        if (!create_batch_scratch(1, kCapacity, scratch)) return 105;
        if (pass.encode_gated_delta(pool, 0, GatedDeltaWeights{}, {DecodeStream{&slot, 0}}, arena.data(), scratch) != CommandError::StateSlotMismatch) return 106;
        if (encode_prefix_state_restore(ctx, nullptr, pool, schedule, slot, arena, 256, kPositions).error != PrefixStateTransferError::StateSlotNotReady) return 107;
    }
    if (tatara_ctx_sync(ctx, nullptr) != TATARA_OK) return 108;
    PrefixStateTransferTicket stale = snap.ticket;
    if (complete_prefix_state_transfer(snap.ticket, pool, slot, arena) != PrefixStateTransferError::None) return 109;
    if (complete_prefix_state_transfer(snap.ticket, pool, slot, arena) != PrefixStateTransferError::AlreadyCompleted) return 110;
    if (complete_prefix_state_transfer(stale, pool, slot, arena) != PrefixStateTransferError::StaleTicket) return 111;
    if (slot.status != DecodeStateSlotStatus::Ready || slot.active_transfer_generation != 0) return 112;

    // expected payload, assembled on the host from the pool contents
    std::vector<std::byte> want(planned.layout.total_bytes), got(planned.layout.total_bytes);
    for (std::uint32_t i = 0; i < planned.layout.segment_count; ++i) {
        const PrefixStateSegment seg = prefix_state_segment(planned.layout, i).segment;
        const PrefixStateCopyRoute route = prefix_state_copy_route(seg, PrefixStateTransferDirection::Snapshot, slot.swapped[seg.layer_index]);
        const std::byte* src = state_transfer_detail::plane_address(pool, slot, seg.layer_index, route.source) + seg.slot_offset_bytes;
        if (cudaMemcpy(want.data() + seg.snapshot_offset_bytes, src, seg.length_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return 113;
    }
    if (cudaMemcpy(got.data(), static_cast<std::byte*>(arena.data()) + 256, got.size(), cudaMemcpyDeviceToHost) != cudaSuccess) return 114;
    if (got != want) return 115;

    // restore into the other slot: canonical halves, phases reset, positions beyond the prefix untouched
    DecodeStateSlot& other = slots[0];
    other.swapped[2] = true;
    std::vector<std::byte> tail_before(16);
    const std::byte* tail = state_transfer_detail::plane_address(pool, other, 1, PrefixStateBufferPlane::First) + kPositions * 512;
    if (cudaMemcpy(tail_before.data(), tail, 16, cudaMemcpyDeviceToHost) != cudaSuccess) return 116;
    PrefixStateTransferResult rest = encode_prefix_state_restore(ctx, nullptr, pool, schedule, other, arena, 256, kPositions);
    if (!rest || other.status != DecodeStateSlotStatus::RestorePending) return 117;
    if (tatara_ctx_sync(ctx, nullptr) != TATARA_OK) return 118;
    if (complete_prefix_state_transfer(rest.ticket, pool, other, arena) != PrefixStateTransferError::None) return 119;
    if (other.swapped[0] || other.swapped[2] || other.status != DecodeStateSlotStatus::Ready) return 120;
    for (std::uint32_t i = 0; i < planned.layout.segment_count; ++i) {
        const PrefixStateSegment seg = prefix_state_segment(planned.layout, i).segment;
        const PrefixStateCopyRoute route = prefix_state_copy_route(seg, PrefixStateTransferDirection::Restore, false);
        const std::byte* dst = state_transfer_detail::plane_address(pool, other, seg.layer_index, route.destination) + seg.slot_offset_bytes;
        if (cudaMemcpy(got.data() + seg.snapshot_offset_bytes, dst, seg.length_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return 121;
    }
    if (got != want) return 122;
    std::vector<std::byte> tail_after(16);
    if (cudaMemcpy(tail_after.data(), tail, 16, cudaMemcpyDeviceToHost) != cudaSuccess || tail_after != tail_before) return 123;

    // the state record: slot 1 (layer 0 swapped) -> bytes -> slot 0; both then serialise identically
    std::vector<std::byte> record, again;
    if (write_state_record(pool, schedule, slot, kPositions, record) != StateRecordError::None) return 124;
    if (record.size() != state_record_bytes(schedule, kPositions) || std::memcmp(record.data(), "Q36BRS01", 8) != 0) return 125;
    std::uint32_t count = 0;
    other.swapped[0] = true;
    if (load_state_record(record.data(), record.size(), pool, schedule, other, &count) != StateRecordError::None || count != kPositions) return 126;
    if (other.swapped[0]) return 127;
    if (write_state_record(pool, schedule, other, kPositions, again) != StateRecordError::None || again != record) return 128;
    if (load_state_record(record.data(), record.size() - 1, pool, schedule, other, nullptr) != StateRecordError::Truncated) return 129;
    record.push_back(std::byte{0});
    if (load_state_record(record.data(), record.size(), pool, schedule, other, nullptr) != StateRecordError::UnconsumedBytes) return 130;
    const std::uint32_t too_many = kCapacity + 1;
    std::memcpy(record.data() + 8, &too_many, 4);
    if (load_state_record(record.data(), record.size(), pool, schedule, other, nullptr) != StateRecordError::PositionOutOfRange) return 131;
    // arena bounds and poisoned slots are typed
    if (encode_prefix_state_snapshot(ctx, nullptr, pool, schedule, slot, arena, 512, kPositions, evidence, 1).error != PrefixStateTransferError::ArenaOutOfRange) return 132;
    if (encode_prefix_state_snapshot(ctx, nullptr, pool, schedule, slot, arena, 256, kPositions, evidence, 0).error != PrefixStateTransferError::PhaseEvidenceTooSmall) return 133;
    slot.status = DecodeStateSlotStatus::Poisoned;
    if (encode_prefix_state_snapshot(ctx, nullptr, pool, schedule, slot, arena, 256, kPositions, evidence, 1).error != PrefixStateTransferError::PoisonedStateSlot) return 134;
    return 0;
}

// Rollback of a verify band: a 6-row band is taped on one gated-delta layer, 4 rows are committed;
// the rolled-back slot must hold the bits of a straight 4-row run.
int rollback_checks(tatara_ctx* ctx) {
    constexpr std::uint32_t kBand = 6, kCommitted = 4;
    const std::vector<LayerKind> schedule{LayerKind::FullAttention, LayerKind::GatedDelta};
    DecodeStatePool pool;
    std::vector<DecodeStateSlot> slots;
    if (!create_state_pool(1, 64, schedule, pool, slots)) return 140;
    DecodeStateSlot& slot = slots[0];
    Rng rng{0x7A9Eull};
    std::vector<u16> proj(kBand * 12352), conv_w(8192 * 4), conv(3 * 8192), a_log(32), dt_bias(32);
    rng.fill(proj); rng.fill(conv_w, 0.5f); rng.fill(conv); rng.fill(dt_bias, 0.5f);
    for (auto& x : a_log) x = to_bf16(std::log(1.0f + 15.0f * rng.uniform()));
    std::vector<float> state(32 * 128 * 128);
    for (auto& x : state) x = 0.02f * rng.normal();
    using state_transfer_detail::plane_address;
    std::byte* conv_live = plane_address(pool, slot, 1, PrefixStateBufferPlane::First);
    std::byte* rec_live = plane_address(pool, slot, 1, PrefixStateBufferPlane::Second);
    std::byte* conv_other = plane_address(pool, slot, 1, PrefixStateBufferPlane::FirstOutput);
    std::byte* rec_other = plane_address(pool, slot, 1, PrefixStateBufferPlane::SecondOutput);
    if (!upload(conv_live, conv) || !upload(rec_live, state)) return 141;
    DeviceBuffer d_proj(proj.size() * 2), d_w(conv_w.size() * 2), d_alog(64), d_dt(64), qk(kBand * 4096 * 2), v(kBand * 4096 * 2),
        z(kBand * 4096 * 2), y(kBand * 4096 * 2), decay(kBand * 32 * 4), beta(kBand * 32 * 4), tape(tatara_gdn_tape_bytes()),
        conv_tape(tatara_gdn_conv_tape_bytes()), scratch_conv(3 * 8192 * 2), scratch_state(state.size() * 4);
    if (!upload(d_proj.data(), proj) || !upload(d_w.data(), conv_w) || !upload(d_alog.data(), a_log) || !upload(d_dt.data(), dt_bias)) return 142;
    // the verify band, taped, writing into scratch planes (the slot keeps the pre-band state)
    if (tatara_gdn_prepare_tape(ctx, nullptr, d_proj.data(), conv_live, d_w.data(), qk.data(), v.data(), z.data(), scratch_conv.data(), kBand,
                                conv_tape.data(), 1) != TATARA_OK) return 143;
    if (tatara_gdn_gates(ctx, nullptr, d_proj.data(), 12352, d_alog.data(), d_dt.data(), decay.data(), beta.data(), kBand) != TATARA_OK) return 144;
    if (tatara_gdn_prefill_tape(ctx, nullptr, qk.data(), v.data(), decay.data(), beta.data(), rec_live, y.data(), scratch_state.data(), kBand,
                                tape.data(), 1) != TATARA_OK) return 145;
    if (encode_gdn_tape_rollback(ctx, nullptr, pool, schedule, slot, tape.data(), conv_tape.data(), 0) != CommandError::InvalidDispatchExtent) return 146;
    if (encode_gdn_tape_rollback(ctx, nullptr, pool, schedule, slot, tape.data(), conv_tape.data(), kCommitted) != CommandError::None) return 147;
    // the straight run of the committed rows
    DeviceBuffer want_conv(3 * 8192 * 2), want_state(state.size() * 4);
    if (tatara_gdn_prepare(ctx, nullptr, d_proj.data(), conv_live, d_w.data(), qk.data(), v.data(), z.data(), want_conv.data(), kCommitted) != TATARA_OK) return 148;
    if (tatara_gdn_prefill(ctx, nullptr, qk.data(), v.data(), decay.data(), beta.data(), rec_live, y.data(), want_state.data(), kCommitted, 1,
                           nullptr, 0) != TATARA_OK) return 149;
    if (tatara_ctx_sync(ctx, nullptr) != TATARA_OK) return 150;
    std::vector<std::byte> a(state.size() * 4), b(a.size()), c(3 * 8192 * 2), d(c.size());
    if (cudaMemcpy(a.data(), rec_other, a.size(), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(b.data(), want_state.data(), b.size(), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(c.data(), conv_other, c.size(), cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(d.data(), want_conv.data(), d.size(), cudaMemcpyDeviceToHost) != cudaSuccess) return 151;
    if (a != b) return 152;
    if (c != d) return 153;
    advance_decode_state(pool, {DecodeStream{&slot, 0}});
    return slot.swapped[1] ? 0 : 154;
}

int main() {
    if (const int rc = host_only_checks(); rc != 0) { std::printf("host check failed: %d\n", rc); return rc; }
    if (const int rc = layout_checks(); rc != 0) { std::printf("layout check failed: %d\n", rc); return rc; }
    tatara_ctx* ctx = nullptr;
    const tatara_status st = tatara_ctx_create(0, &ctx);
    if (st == TATARA_INVALID_DEVICE) { std::printf("host checks passed; no B200 present, device checks skipped\n"); return 0; }
    if (st != TATARA_OK) return 2;
    int rc = device_checks(ctx);
    if (rc == 0) rc = projection_checks(ctx);
    if (rc == 0) rc = transfer_checks(ctx);
    if (rc == 0) rc = rollback_checks(ctx);
    tatara_ctx_destroy(ctx);
    if (rc != 0) { std::printf("device check failed: %d\n", rc); return rc; }
    std::printf("host and device checks passed\n");
    return 0;
}
