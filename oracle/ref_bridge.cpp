// Bridge onto the reference's own CPU model of its kernels
// (tests/native/kernel_reference.{h,cpp}, compiled unmodified from the reference
// tree by oracle/Makefile into oracle/_ref/).  TEST INFRASTRUCTURE ONLY.
//
// The reference model takes transcendental values (rsqrt, cos/sin, exp, sigmoid)
// as inputs that its probes query from the Metal device.  No such device exists
// here, so this bridge supplies them from float libm -- the reference's own
// `FloatLibm` / `ReciprocalOfSqrt` candidates -- and drives the pinned variants
// (fused multiply-add chains, adjacent-pairs 32-lane tree;
// tools/native/fixture_suite_probe.cpp:40-60).  It exports plain-C functions so
// that tests can compare the restated oracle against the reference bit for bit
// and so that tests/golden/make_golden.py can write the golden vectors.

#include "kernel_reference.h"

#include <cmath>
#include <cstdint>
#include <span>
#include <vector>

using namespace tatara::testing;
using u16 = std::uint16_t;
using u32 = std::uint32_t;

namespace {
constexpr AttnGeometry kAttn{.query_heads = 16, .kv_heads = 2, .head_dimension = 256};
constexpr GdnGeometry kGdn{.key_heads = 16, .value_heads = 32, .head_dimension = 128};
constexpr auto kTree = SimdTreeShape::AdjacentPairs;
constexpr auto kLibm = TranscendentalModel::FloatLibm;

float rope_divisor(u32 pair) {
    return static_cast<float>(std::pow(1.0e7, static_cast<double>(pair) / 32.0));
}
} // namespace

extern "C" {

u16 ref_bf16_from_f32(float v) { return bf16_from_f32(v); }
u16 ref_bf16_mul(u16 a, u16 b) { return bfloat_multiply_candidate(a, b); }

void ref_xorshift_banded(std::uint64_t seed, u16* out, u32 count) {
    Xorshift64Star generator(seed);
    for (u32 i = 0; i < count; ++i) out[i] = generator.next_banded_bf16();
}

// One position of attn_qk_rope (projection[9216]); q_out/gate_out [16][256].
void ref_attn_qk_rope(const u16* projection, const u16* q_weight, const u16* k_weight,
                      u16* q_out, u16* gate_out, u16* keys, u16* values, u32 position,
                      u32 capacity) {
    const std::span<const u16> proj(projection, 9216);
    std::vector<float> inverses(18), cosines(32), sines(32);
    for (u32 head = 0; head < 18; ++head) {
        const u32 base = head < 16 ? head * 512 : 8192 + (head - 16) * 256;
        inverses[head] =
            rsqrt_candidate(attn_rms_argument(proj, base, 256, 1e-6f), RsqrtOrder::ReciprocalOfSqrt);
    }
    for (u32 pair = 0; pair < 32; ++pair) {
        const float theta = static_cast<float>(position) / rope_divisor(pair);
        cosines[pair] = std::cos(theta);
        sines[pair] = std::sin(theta);
    }
    const std::size_t cache = std::size_t{2} * capacity * 256;
    attn_qk_rope_reference(proj, {q_weight, 256}, {k_weight, 256}, position, capacity, kAttn,
                           inverses, cosines, sines, ChainOrder::Fused, {q_out, 4096},
                           {gate_out, 4096}, {keys, cache}, {values, cache});
}

// Single-kernel decode family for all 16 heads.
void ref_attn_decode(const u16* q, const u16* gate, const u16* keys, const u16* values,
                     u32 context, u32 capacity, u16* out) {
    const std::size_t cache = std::size_t{2} * capacity * 256;
    for (u32 head = 0; head < 16; ++head) {
        std::vector<float> arguments;
        attention_decode_arguments({q, 4096}, {keys, cache}, head, context, capacity, kAttn,
                                   arguments);
        for (float& a : arguments) a = std::exp(a);
        attention_decode_reference({q, 4096}, {gate, 4096}, {keys, cache}, {values, cache}, head,
                                   context, capacity, kAttn, arguments, ChainOrder::Fused,
                                   {out, 4096});
    }
}

// Partitioned family: scores -> values -> combine with 256-key partitions.
// records [16][nparts][258] receives the partial records.
void ref_attn_split(const u16* q, const u16* gate, const u16* keys, const u16* values,
                    u32 context, u32 capacity, float* records, u16* out) {
    const std::size_t cache = std::size_t{2} * capacity * 256;
    const u32 part = 256;
    const u32 nparts = (context + 1 + part - 1) / part;
    for (u32 head = 0; head < 16; ++head) {
        float* head_records = records + std::size_t{head} * nparts * 258;
        for (u32 p = 0; p < nparts; ++p) {
            std::vector<float> arguments;
            attention_scores_gqa4_arguments({q, 4096}, {keys, cache}, head, context, capacity, part,
                                            p, kAttn, arguments);
            for (float& a : arguments) a = std::exp(a);
            std::vector<float> weights(258);
            attention_scores_gqa4_reference({q, 4096}, {keys, cache}, head, context, capacity, part,
                                            p, kAttn, arguments, weights);
            attention_values_gqa8_reference(weights, {values, cache}, head >> 3, context, capacity,
                                            part, p, kAttn, ChainOrder::Fused,
                                            {head_records + std::size_t{p} * 258, 258});
        }
        std::vector<float> arguments, gate_exps(256);
        attention_combine_arguments({head_records, std::size_t{nparts} * 258}, nparts, arguments);
        for (float& a : arguments) a = std::exp(a);
        for (u32 d = 0; d < 256; ++d) gate_exps[d] = std::exp(-f32_from_bf16(gate[head * 256 + d]));
        attention_combine_reference({head_records, std::size_t{nparts} * 258}, {gate, 4096}, head,
                                    nparts, kAttn, arguments, gate_exps, ChainOrder::Fused,
                                    {out + head * 256, 256});
    }
}

// One position of gdn_prepare.
void ref_gdn_prepare(const u16* projection, const u16* conv_state, const u16* conv_weights,
                     u16* qk, u16* value, u16* z, u16* new_conv_state) {
    std::vector<u16> convolved(8192), activated(8192);
    gdn_conv_forward({projection, 12352}, {conv_state, 3 * 8192}, {conv_weights, 8192 * 4}, 8192,
                     convolved, {new_conv_state, 3 * 8192});
    for (u32 ch = 0; ch < 8192; ++ch)
        activated[ch] =
            bfloat_multiply_candidate(convolved[ch], bf16_sigmoid_candidate(convolved[ch], kLibm));
    std::vector<float> inverses(32);
    for (u32 head = 0; head < 32; ++head)
        inverses[head] = rsqrt_candidate(gdn_head_rsqrt_argument(activated, head, 128, 1e-6f, kTree),
                                         RsqrtOrder::ReciprocalOfSqrt);
    gdn_qk_normalize(activated, inverses, kGdn, bf16_from_f32(1.0f / 128.0f),
                     bf16_from_f32(0.08838834764831845f), {qk, 4096});
    for (u32 i = 0; i < 4096; ++i) {
        value[i] = activated[4096 + i];
        z[i] = projection[8192 + i];
    }
}

void ref_gdn_gates(const u16* projection, const u16* a_log, const u16* dt_bias, float* decay,
                   float* beta) {
    for (u32 head = 0; head < 32; ++head) {
        const u16 shifted = bfloat_add_candidate(projection[12320 + head], dt_bias[head]);
        decay[head] = gdn_decay_candidate(shifted, a_log[head], kLibm);
        beta[head] = f32_from_bf16(bf16_sigmoid_candidate(projection[12288 + head], kLibm));
    }
}

void ref_gdn_step(const u16* qk, const u16* value, const float* decay, const float* beta,
                  const float* state_in, u16* y, float* state_out) {
    const std::size_t state = std::size_t{32} * 128 * 128;
    gdn_recurrence_reference({qk, 4096}, {value, 4096}, {decay, 32}, {beta, 32}, {state_in, state},
                             kGdn, kTree, ChainOrder::Fused, {y, 4096}, {state_out, state});
}

void ref_gdn_gate_norm(const u16* y, const u16* z, const u16* weight, u16* out) {
    std::vector<float> inverses(32), sigmoids(4096);
    for (u32 head = 0; head < 32; ++head)
        inverses[head] = rsqrt_candidate(gdn_head_rsqrt_argument({y, 4096}, head, 128, 1e-6f, kTree),
                                         RsqrtOrder::ReciprocalOfSqrt);
    for (u32 i = 0; i < 4096; ++i) sigmoids[i] = f32_sigmoid_candidate(f32_from_bf16(z[i]), kLibm);
    gdn_gate_norm_reference({y, 4096}, {z, 4096}, {weight, 128}, inverses, sigmoids, 32, 128,
                            {out, 4096});
}

// q4_dot_reference with the adjacent-pairs tree; `fused` picks the chain order.
float ref_q4_dot(const u16* x, const u32* words, const u16* scales, const u16* biases, u32 k,
                 int fused) {
    return q4_dot_reference({x, k}, {words, k / 8}, {scales, k / 64}, {biases, k / 64}, k, kTree,
                            fused ? ChainOrder::Fused : ChainOrder::Separate);
}

} // extern "C"
