// CPU oracle for the attention + Gated DeltaNet hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the
// test-suite, the smoke entry and the benchmark's cpu_baseline / reference arm
// are the only callers.  Nothing in the product library links or calls it.
//
// It is a scalar fp32 restatement (bf16 storage, f32 arithmetic) of the
// reference engine's kernels, following the reference's own CPU model of those
// kernels operation by operation so that the two can be compared bit for bit:
//   * tests/native/kernel_reference.cpp (bf16 RNE, flush-to-zero, adjacent-pairs
//     32-lane tree, fused multiply-add chains, float libm transcendentals)
//   * src/backend/metal/kernels/{attention,prefill_attention,gdn,prefill_gdn}.metal
// Each function cites the lines it follows.  Parity pin: tests compare every
// function here against the reference's CPU model compiled from its own
// sources (oracle/_ref, built by oracle/Makefile) and against the committed
// golden vectors generated from it (tests/golden).
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fPIC -shared (see oracle/Makefile).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

namespace {

using u16 = std::uint16_t;
using u32 = std::uint32_t;
using u64 = std::uint64_t;

// Model geometry (tools/generate_kernel_library.py:173-182, 1980-2006).
constexpr u32 kQHeads = 16, kKvHeads = 2, kD = 256, kHeadsPerKv = 8;
constexpr u32 kRopePairs = 32;
constexpr float kScale = 0.0625f, kEps = 1e-6f;
constexpr u32 kAttnProj = 9216, kAttnKOff = 8192, kAttnVOff = 8704;
constexpr u32 kRecord = 258;
constexpr u32 kGdnKeyHeads = 16, kGdnValueHeads = 32, kGd = 128;
constexpr u32 kGdnQk = 4096, kGdnV = 4096, kGdnConv = 8192;
constexpr u32 kGdnProj = 12352, kGdnZOff = 8192, kGdnBOff = 12288, kGdnAOff = 12320;
constexpr float kInf = std::numeric_limits<float>::infinity();

inline u32 f2u(float f) { u32 u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(u32 u) { float f; std::memcpy(&f, &u, 4); return f; }

// kernel_reference.cpp:77-88 — round to nearest even, Inf/NaN pass through.
inline u16 bf16r(float v) {
    const u32 b = f2u(v);
    if ((b & 0x7F800000u) == 0x7F800000u) return static_cast<u16>(b >> 16);
    return static_cast<u16>((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
inline float bf(u16 b) { return u2f(static_cast<u32>(b) << 16); }
// kernel_reference.cpp:90-103 — the device flushes subnormals to signed zero.
inline u16 ftzb(u16 b) { return (b & 0x7F80u) == 0 ? static_cast<u16>(b & 0x8000u) : b; }
inline float ftz(float v) {
    const u32 b = f2u(v);
    return (b & 0x7F800000u) == 0 ? u2f(b & 0x80000000u) : v;
}
// bf16 "eager op" arithmetic: f32 op on flushed inputs, one rounding, flushed
// (kernel_reference.cpp:148-152, 299-317).
inline u16 bmul(u16 a, u16 b) { return ftzb(bf16r(ftz(bf(ftzb(a)) * bf(ftzb(b))))); }
inline u16 badd(u16 a, u16 b) { return ftzb(bf16r(ftz(bf(ftzb(a)) + bf(ftzb(b))))); }
inline u16 bsub(u16 a, u16 b) { return ftzb(bf16r(ftz(bf(ftzb(a)) - bf(ftzb(b))))); }
inline u16 bdiv(u16 a, u16 b) { return ftzb(bf16r(ftz(bf(ftzb(a)) / bf(ftzb(b))))); }

// Adjacent-pairs reduction over a power-of-two lane vector
// (kernel_reference.cpp:24-35; the pinned simd_sum shape).
float pairs_sum(float* v, u32 n) {
    while (n > 1) {
        for (u32 i = 0; i < n / 2; ++i) v[i] = v[2 * i] + v[2 * i + 1];
        n /= 2;
    }
    return v[0];
}
// 256-slot halving tree used for tile sums (kernel_reference.cpp:601-610).
float halving_sum_256(const float* slots) {
    float red[256];
    std::memcpy(red, slots, sizeof(red));
    for (u32 off = 128; off; off >>= 1)
        for (u32 i = 0; i < off; ++i) red[i] += red[i + off];
    return red[0];
}

// Stable-branch sigmoid with per-op bf16 rounding (gdn.metal:76-79, 147-150;
// kernel_reference.cpp:335-346).
u16 sigmoid_bf16(u16 in) {
    const float x = bf(ftzb(in));
    const u16 e = ftzb(bf16r(ftz(std::exp(std::fabs(x)))));
    const u16 one = 0x3F80;
    const u16 low = bdiv(one, badd(one, e));
    return x < 0.0f ? low : bsub(one, low);
}
// f32 stable-branch sigmoid (gdn.metal:203-205; kernel_reference.cpp:348-353).
float sigmoid_f32(float x) {
    const float low = ftz(1.0f / (1.0f + ftz(std::exp(std::fabs(x)))));
    return x < 0.0f ? low : 1.0f - low;
}
// decay = exp(-exp(A_log) * softplus_bf16(a + dt_bias)) (gdn.metal:133-146;
// kernel_reference.cpp:355-375).  `shifted` is the bf16 sum a + dt_bias.
float gdn_decay(u16 shifted, u16 a_log) {
    const u16 s = ftzb(shifted);
    const bool pos = bf(s) > 0.0f;
    const u16 bmax = pos ? s : u16{0};
    const u16 bmin = pos ? u16{0} : s;
    const u16 diff = bsub(bmin, bmax);
    const u16 e = ftzb(bf16r(ftz(std::exp(bf(diff)))));
    const float one_plus = 1.0f + bf(e);
    u16 l1p = e;
    if (one_plus != 1.0f)
        l1p = ftzb(bf16r(ftz(bf(e) * (std::log(one_plus) / (one_plus - 1.0f)))));
    const u16 sp = badd(bmax, l1p);
    return std::exp(-std::exp(bf(ftzb(a_log))) * bf(sp));
}

void parallel_for(u32 n, int threads, const std::function<void(u32)>& body) {
    if (threads <= 1 || n <= 1) {
        for (u32 i = 0; i < n; ++i) body(i);
        return;
    }
    const u32 t = std::min<u32>(static_cast<u32>(threads), n);
    std::vector<std::thread> pool;
    for (u32 w = 0; w < t; ++w)
        pool.emplace_back([&, w] { for (u32 i = w; i < n; i += t) body(i); });
    for (auto& th : pool) th.join();
}

// RoPE divisor pow(base, pair/32) evaluated in double and rounded once to f32
// (attention.metal:96-97 writes it as an f32 pow; the reference's CPU model
// takes cos/sin as device-queried inputs, kernel_reference.h:151-160).
inline float rope_divisor(u32 pair) {
    return static_cast<float>(std::pow(1.0e7, static_cast<double>(pair) / 32.0));
}

// 32-lane strided dot + adjacent-pairs tree (kernel_reference.cpp:587-599).
float strided_dot(const u16* q, const u16* k) {
    float lanes[32];
    for (u32 l = 0; l < 32; ++l) {
        float dot = 0.0f;
        for (u32 d = l; d < kD; d += 32) dot += bf(q[d]) * bf(k[d]);
        lanes[l] = dot;
    }
    return pairs_sum(lanes, 32);
}

// Online softmax over keys [begin, end) of one kv head in 256-key tiles:
// acc[256] (unnormalised numerator), running max, running denominator.
// Follows attention_decode (attention.metal:223-271) and attention_partial_blk
// (prefill_attention.metal:129-195); CPU model kernel_reference.cpp:741-775.
void online_softmax(const u16* q, const u16* keys, const u16* values, u32 begin, u32 end,
                    float* acc, float& run_max, float& denom) {
    run_max = -kInf;
    denom = 0.0f;
    for (u32 d = 0; d < kD; ++d) acc[d] = 0.0f;
    float scores[256], probs[256];
    for (u32 tile = begin; tile < end; tile += 256) {
        const u32 count = std::min(end - tile, 256u);
        float tile_max = -kInf;
        for (u32 t = 0; t < count; ++t) {
            scores[t] = ftz(strided_dot(q, keys + static_cast<u64>(tile + t) * kD) * kScale);
            tile_max = std::max(tile_max, scores[t]);
        }
        const float new_max = std::max(run_max, tile_max);
        const float rescale = run_max == -kInf ? 0.0f : std::exp(run_max - new_max);
        for (u32 t = 0; t < 256; ++t) probs[t] = t < count ? std::exp(scores[t] - new_max) : 0.0f;
        const float tile_sum = halving_sum_256(probs);
        for (u32 d = 0; d < kD; ++d) {
            float a = ftz(acc[d] * rescale);
            for (u32 t = 0; t < count; ++t)
                a = std::fma(probs[t], bf(values[static_cast<u64>(tile + t) * kD + d]), a);
            acc[d] = a;
        }
        denom = ftz(ftz(denom * rescale) + tile_sum);
        run_max = new_max;
    }
}

// out = bf16((acc/denom) * sigmoid(gate)) (attention.metal:272-275;
// kernel_reference.cpp:776-783).
inline u16 gated_output(float acc, float denom, u16 gate) {
    const float value = ftz(acc / denom);
    const float g = bf(gate);
    const float sig = ftz(1.0f / (1.0f + ftz(std::exp(-g))));
    return ftzb(bf16r(ftz(value * sig)));
}

// Affine Q4, group 64, one output row (q4_dot.metal:9-42; CPU model
// kernel_reference.cpp:388-442).  Lane l of 32 owns 16 consecutive inputs of every
// 512-column block; nibbles are taken in place with masks and the inputs are
// pre-divided by the nibble's place value; per block the lane adds
// scale*quant + sum*bias; the 32 lane results go through the adjacent-pairs tree.
// `fused` selects the reference model's ChainOrder::Fused (fma chains) or
// ChainOrder::Separate (each product and sum rounded).
float q4_dot(const u16* x, const u16* packed, const u16* scales, const u16* biases, u32 k_size,
             bool fused) {
    float lanes[32];
    for (u32 lane = 0; lane < 32; ++lane) {
        float result = 0.0f;
        for (u32 k = 0; k < k_size; k += 512) {
            const u32 x0 = k + lane * 16;
            float xv[16];
            float sum = 0.0f;
            for (u32 i = 0; i < 16; i += 4) {
                const float a0 = bf(x[x0 + i]), a1 = bf(x[x0 + i + 1]);
                const float a2 = bf(x[x0 + i + 2]), a3 = bf(x[x0 + i + 3]);
                sum = ftz(sum + ftz(ftz(a0 + a1) + a2 + a3));
                xv[i] = a0;
                xv[i + 1] = a1 / 16.0f;
                xv[i + 2] = a2 / 256.0f;
                xv[i + 3] = a3 / 4096.0f;
            }
            float quant = 0.0f;
            const u32 word0 = (k >> 2) + lane * 4;
            for (u32 i = 0; i < 4; ++i) {
                const u16 word = packed[word0 + i];
                const float w0 = static_cast<float>(word & 0x000Fu), w1 = static_cast<float>(word & 0x00F0u);
                const float w2 = static_cast<float>(word & 0x0F00u), w3 = static_cast<float>(word & 0xF000u);
                if (fused) {
                    quant = std::fma(xv[i * 4 + 3], w3,
                                     std::fma(xv[i * 4 + 2], w2,
                                              std::fma(xv[i * 4 + 1], w1, std::fma(xv[i * 4], w0, quant))));
                } else {
                    const float t0 = xv[i * 4] * w0, t1 = xv[i * 4 + 1] * w1;
                    const float t2 = xv[i * 4 + 2] * w2, t3 = xv[i * 4 + 3] * w3;
                    quant = quant + (((t0 + t1) + t2) + t3);
                }
            }
            const u32 group = (k >> 6) + (lane >> 2);
            const float scale = bf(scales[group]), bias = bf(biases[group]);
            if (fused) result = std::fma(sum, bias, std::fma(scale, quant, result));
            else result = result + (scale * quant + sum * bias);
        }
        lanes[lane] = result;
    }
    return pairs_sum(lanes, 32);
}

// bf16(q*scale + bias) of one weight, the staging step of the reference's tensor-unit
// projection policy (native_dense_qgemm.metal, "weight_tile[...] = bfloat(float(quantized) *
// affine_scale + affine_bias)"); nibble j of a 32-bit word is column 8*word + j.
inline u16 q4_weight_bf16(const u32* words, const u16* scales, const u16* biases, u32 k) {
    const u32 q = (words[k >> 3] >> (4u * (k & 7u))) & 15u;
    return bf16r(std::fma(static_cast<float>(q), bf(scales[k >> 6]), bf(biases[k >> 6])));
}

} // namespace

extern "C" {

int orc_abi_version() { return 1; }
int orc_hardware_threads() {
    const unsigned n = std::thread::hardware_concurrency();
    return n == 0 ? 1 : static_cast<int>(n);
}

u16 orc_bf16_from_f32(float v) { return bf16r(v); }
float orc_f32_from_bf16(u16 b) { return bf(b); }
u16 orc_bf16_mul(u16 a, u16 b) { return bmul(a, b); }
float orc_rope_divisor(u32 pair) { return rope_divisor(pair); }

// q/k RMSNorm + partial RoPE + KV append for `rows` consecutive positions
// starting at `position`.  attention.metal:43-113, prefill_attention.metal:1-92;
// CPU model kernel_reference.cpp:616-689.
//   projection [rows][9216] = per head h: q(256) | gate(256), then k(2x256), v(2x256)
//   q_out, gate_out [rows][16][256]; keys/values [kv][capacity][256] at position+row.
void orc_attn_qk_rope(const u16* projection, const u16* q_weight, const u16* k_weight,
                      u16* q_out, u16* gate_out, u16* keys, u16* values, u32 position,
                      u32 capacity, u32 rows) {
    float divisor[kRopePairs];
    for (u32 p = 0; p < kRopePairs; ++p) divisor[p] = rope_divisor(p);
    for (u32 row = 0; row < rows; ++row) {
        const u16* proj = projection + static_cast<u64>(row) * kAttnProj;
        const u32 pos = position + row;
        float cosv[kRopePairs], sinv[kRopePairs];
        for (u32 p = 0; p < kRopePairs; ++p) {
            const float theta = static_cast<float>(pos) / divisor[p];
            cosv[p] = std::cos(theta);
            sinv[p] = std::sin(theta);
        }
        for (u32 head = 0; head < kQHeads + kKvHeads; ++head) {
            const bool is_q = head < kQHeads;
            const u32 local = is_q ? head : head - kQHeads;
            const u32 base = is_q ? head * 2 * kD : kAttnKOff + local * kD;
            // 64 threads x 4 contiguous squares, two 32-lane trees, then the
            // 32-slot stage tree (attention.metal:64-86).
            float stage[32] = {0};
            float lanes[32];
            for (u32 t = 0; t < 64; ++t) {
                float a = 0.0f;
                for (u32 j = 0; j < 4; ++j) {
                    const float v = bf(proj[base + t * 4 + j]);
                    a += v * v;
                }
                lanes[t % 32] = a;
                if (t % 32 == 31) stage[t / 32] = pairs_sum(lanes, 32);
            }
            const float inv = 1.0f / std::sqrt(pairs_sum(stage, 32) / static_cast<float>(kD) + kEps);
            float normed[kD];
            for (u32 d = 0; d < kD; ++d) {
                const u16 scaled = ftzb(bf16r(ftz(bf(proj[base + d]) * inv)));
                normed[d] = bf(bmul(is_q ? q_weight[d] : k_weight[d], scaled));
            }
            for (u32 d = 0; d < kD; ++d) {
                float r = normed[d];
                if (d < 2 * kRopePairs) {
                    const u32 p = d & 31u;
                    r = d < 32 ? std::fma(-normed[d + 32], sinv[p], normed[d] * cosv[p])
                               : std::fma(normed[d - 32], sinv[p], normed[d] * cosv[p]);
                    r = ftz(r);
                }
                const u16 stored = ftzb(bf16r(r));
                if (is_q) {
                    q_out[(static_cast<u64>(row) * kQHeads + head) * kD + d] = stored;
                    gate_out[(static_cast<u64>(row) * kQHeads + head) * kD + d] =
                        proj[head * 2 * kD + kD + d];
                } else {
                    const u64 at = (static_cast<u64>(local) * capacity + pos) * kD + d;
                    keys[at] = stored;
                    values[at] = proj[kAttnVOff + local * kD + d];
                }
            }
        }
    }
}

// One decode step: head h attends keys 0..context inclusive.
// attention.metal:200-276; CPU model kernel_reference.cpp:725-784.
void orc_attn_decode(const u16* q, const u16* gate, const u16* keys, const u16* values,
                     u32 context, u32 capacity, u16* out, int threads) {
    parallel_for(kQHeads, threads, [&](u32 h) {
        const u32 kv = h / kHeadsPerKv;
        float acc[kD], m, l;
        online_softmax(q + h * kD, keys + static_cast<u64>(kv) * capacity * kD,
                       values + static_cast<u64>(kv) * capacity * kD, 0, context + 1, acc, m, l);
        for (u32 d = 0; d < kD; ++d) out[h * kD + d] = gated_output(acc[d], l, gate[h * kD + d]);
    });
}

// Partial records over keys [key_begin, key_end): records[h][258] =
// [numerator(256) | max | sum].  prefill_attention.metal:97-205; equals the
// scores/values record pair kernel_reference.cpp:813-873 for ranges <= 256 keys.
void orc_attn_partial(const u16* q, const u16* keys, const u16* values, u32 key_begin,
                      u32 key_end, u32 capacity, float* records, u32 record_stride_heads,
                      int threads) {
    parallel_for(kQHeads, threads, [&](u32 h) {
        const u32 kv = h / kHeadsPerKv;
        float* rec = records + static_cast<u64>(h) * record_stride_heads;
        online_softmax(q + h * kD, keys + static_cast<u64>(kv) * capacity * kD,
                       values + static_cast<u64>(kv) * capacity * kD, key_begin, key_end, rec,
                       rec[256], rec[257]);
    });
}

// Log-sum-exp merge of records[h][p][258], then gate.  attention.metal:1086-1108,
// prefill_attention.metal:207-254 (empty partition => weight 0);
// CPU model kernel_reference.cpp:875-918.
void orc_attn_combine(const float* records, u32 nparts, const u16* gate, u16* out) {
    for (u32 h = 0; h < kQHeads; ++h) {
        const float* base = records + static_cast<u64>(h) * nparts * kRecord;
        float gmax = -kInf;
        for (u32 p = 0; p < nparts; ++p) gmax = std::max(gmax, base[p * kRecord + 256]);
        float acc[kD] = {0};
        float denom = 0.0f;
        for (u32 p = 0; p < nparts; ++p) {
            const float lm = base[p * kRecord + 256];
            const float w = lm == -kInf ? 0.0f : std::exp(lm - gmax);
            for (u32 d = 0; d < kD; ++d) acc[d] = std::fma(w, base[p * kRecord + d], acc[d]);
            denom = std::fma(w, base[p * kRecord + 257], denom);
        }
        for (u32 d = 0; d < kD; ++d) out[h * kD + d] = gated_output(acc[d], denom, gate[h * kD + d]);
    }
}

// Causal block prefill: row r (absolute position context_base + r) attends keys
// 0..position inclusive of the lane cache.  One partition per row is the
// reference's numerical control (prefill_attention.metal:97-254).
//   query, gate, out [rows][16][256]; row_list (optional) selects rows to compute.
void orc_attn_prefill(const u16* query, const u16* gate, const u16* keys, const u16* values,
                      u32 context_base, u32 rows, u32 capacity, const u32* row_list, u32 n_list,
                      u16* out, int threads) {
    const u32 n = row_list ? n_list : rows;
    parallel_for(n * kQHeads, threads, [&](u32 item) {
        const u32 r = row_list ? row_list[item / kQHeads] : item / kQHeads;
        const u32 h = item % kQHeads;
        const u32 kv = h / kHeadsPerKv;
        const u64 at = (static_cast<u64>(r) * kQHeads + h) * kD;
        float acc[kD], m, l;
        online_softmax(query + at, keys + static_cast<u64>(kv) * capacity * kD,
                       values + static_cast<u64>(kv) * capacity * kD, 0, context_base + r + 1, acc,
                       m, l);
        for (u32 d = 0; d < kD; ++d) out[at + d] = gated_output(acc[d], l, gate[at + d]);
    });
}

// Width-4 causal conv + SiLU + q/k normalisation over `rows` positions.
// gdn.metal:48-112, prefill_gdn.metal:4-88; CPU pieces kernel_reference.cpp:377-386,
// 445-496.  projection [rows][12352]; conv_state [3][8192] oldest first;
// conv_weights [8192][4]; qk/value/z [rows][4096]; new_conv_state [3][8192].
void orc_gdn_prepare(const u16* projection, const u16* conv_state, const u16* conv_weights,
                     u16* qk, u16* value, u16* z, u16* new_conv_state, u32 rows) {
    std::vector<u16> activated(kGdnConv);
    for (u32 row = 0; row < rows; ++row) {
        const u16* proj = projection + static_cast<u64>(row) * kGdnProj;
        for (u32 ch = 0; ch < kGdnConv; ++ch) {
            float taps[4];
            for (u32 t = 0; t < 4; ++t) {
                const u32 logical = row + t; // sequence = 3 state rows then projection rows
                taps[t] = logical < 3 ? bf(conv_state[logical * kGdnConv + ch])
                                      : bf(projection[static_cast<u64>(logical - 3) * kGdnProj + ch]);
            }
            float acc = 0.0f;
            for (u32 t = 0; t < 4; ++t)
                acc = ftz(acc + ftz(bf(ftzb(conv_weights[ch * 4 + t])) * taps[t]));
            const u16 c = ftzb(bf16r(acc));
            activated[ch] = bmul(c, sigmoid_bf16(c));
            if (row + 1 == rows)
                for (u32 t = 0; t < 3; ++t) new_conv_state[t * kGdnConv + ch] = bf16r(taps[t + 1]);
        }
        for (u32 head = 0; head < 2 * kGdnKeyHeads; ++head) {
            float lanes[32];
            for (u32 l = 0; l < 32; ++l) {
                float s = 0.0f;
                for (u32 i = 0; i < 4; ++i) {
                    const float v = bf(activated[head * kGd + l * 4 + i]);
                    s += v * v;
                }
                lanes[l] = s;
            }
            const float inv = 1.0f / std::sqrt(pairs_sum(lanes, 32) / static_cast<float>(kGd) + kEps);
            // q heads scale 1/128, k heads bf16(1/sqrt(128)) (gdn.metal:102-104).
            const u16 scale = head < kGdnKeyHeads ? u16{0x3C00} : u16{0x3DB5};
            for (u32 i = 0; i < kGd; ++i) {
                const u32 idx = head * kGd + i;
                const u16 normed = ftzb(bf16r(ftz(bf(activated[idx]) * inv)));
                qk[static_cast<u64>(row) * kGdnQk + idx] = bmul(normed, scale);
            }
        }
        for (u32 i = 0; i < kGdnV; ++i) {
            value[static_cast<u64>(row) * kGdnV + i] = activated[kGdnQk + i];
            z[static_cast<u64>(row) * kGdnV + i] = proj[kGdnZOff + i];
        }
    }
}

// Per (row, v-head) decay and beta planes [rows][32] f32.
// prefill_gdn.metal:94-135, gdn.metal:133-150; kernel_reference.cpp:335-375.
void orc_gdn_gates(const u16* projection, u32 projection_stride, const u16* a_log,
                   const u16* dt_bias, float* decay, float* beta, u32 rows) {
    for (u32 row = 0; row < rows; ++row) {
        const u16* proj = projection + static_cast<u64>(row) * projection_stride;
        for (u32 h = 0; h < kGdnValueHeads; ++h) {
            const u16 shifted = badd(proj[kGdnAOff + h], dt_bias[h]);
            decay[row * kGdnValueHeads + h] = gdn_decay(shifted, a_log[h]);
            beta[row * kGdnValueHeads + h] = bf(sigmoid_bf16(proj[kGdnBOff + h]));
        }
    }
}

// Sequential delta-rule scan over `rows` steps (rows = 1 is the decode step).
// gdn.metal:151-171, prefill_gdn.metal:158-195; kernel_reference.cpp:498-563.
//   qk [rows][4096] (q at 0, k at 2048); value, y [rows][4096];
//   decay, beta [rows][32]; state [32][128 vdim][128 kdim] f32.
void orc_gdn_scan(const u16* qk, const u16* value, const float* decay, const float* beta,
                  const float* state_in, u16* y, float* state_out, u32 rows, int threads) {
    parallel_for(kGdnValueHeads * kGd, threads, [&](u32 item) {
        const u32 vh = item / kGd, vd = item % kGd;
        const u32 qbase = (vh >> 1) * kGd, kbase = kGdnQk / 2 + qbase;
        const u64 sbase = static_cast<u64>(item) * kGd;
        float state[kGd];
        for (u32 e = 0; e < kGd; ++e) state[e] = state_in[sbase + e];
        for (u32 step = 0; step < rows; ++step) {
            const u16* qkr = qk + static_cast<u64>(step) * kGdnQk;
            const float dec = decay[step * kGdnValueHeads + vh];
            const float bet = beta[step * kGdnValueHeads + vh];
            float lanes[32];
            for (u32 l = 0; l < 32; ++l) {
                float kvp = 0.0f;
                for (u32 i = 0; i < 4; ++i) {
                    const u32 e = l * 4 + i;
                    state[e] = ftz(state[e] * dec);
                    kvp = std::fma(state[e], bf(qkr[kbase + e]), kvp);
                }
                lanes[l] = kvp;
            }
            const float kv = pairs_sum(lanes, 32);
            const float v = bf(value[static_cast<u64>(step) * kGdnV + vh * kGd + vd]);
            const float delta = ftz(ftz(v - kv) * bet);
            for (u32 l = 0; l < 32; ++l) {
                float o = 0.0f;
                for (u32 i = 0; i < 4; ++i) {
                    const u32 e = l * 4 + i;
                    state[e] = std::fma(bf(qkr[kbase + e]), delta, state[e]);
                    o = std::fma(state[e], bf(qkr[qbase + e]), o);
                }
                lanes[l] = o;
            }
            y[static_cast<u64>(step) * kGdnV + vh * kGd + vd] = ftzb(bf16r(pairs_sum(lanes, 32)));
        }
        for (u32 e = 0; e < kGd; ++e) state_out[sbase + e] = state[e];
    });
}

// Weighted per-head RMSNorm of y times SiLU(z).  gdn.metal:174-207,
// prefill_gdn.metal:283-320; kernel_reference.cpp:565-583.
void orc_gdn_gate_norm(const u16* y, const u16* z, const u16* weight, u16* out, u32 rows) {
    for (u64 row = 0; row < rows; ++row)
        for (u32 h = 0; h < kGdnValueHeads; ++h) {
            const u64 base = row * kGdnV + h * kGd;
            float lanes[32];
            for (u32 l = 0; l < 32; ++l) {
                float s = 0.0f;
                for (u32 i = 0; i < 4; ++i) {
                    const float v = bf(y[base + l * 4 + i]);
                    s += v * v;
                }
                lanes[l] = s;
            }
            const float inv = 1.0f / std::sqrt(pairs_sum(lanes, 32) / static_cast<float>(kGd) + kEps);
            for (u32 i = 0; i < kGd; ++i) {
                const u16 normed = ftzb(bf16r(ftz(bf(y[base + i]) * inv)));
                const u16 weighted = bmul(weight[i], normed);
                const float g = bf(z[base + i]);
                out[base + i] = ftzb(bf16r(ftz(ftz(g * sigmoid_f32(g)) * bf(weighted))));
            }
        }
}

// ---- affine-Q4 projections on either side of the layers -------------------------------
// One matrix of `n` output rows: words [n][k/8] u32, scales/biases [n][k/64] bf16.

float orc_q4_dot(const u16* x, const u32* words, const u16* scales, const u16* biases, u32 k,
                 int fused) {
    return q4_dot(x, reinterpret_cast<const u16*>(words), scales, biases, k, fused != 0);
}

// Exact-row policy: out[r*out_stride + col] = bf16(q4_dot(x[r], row col)) for every input row r
// (attn_project attention.metal:1-41, gdn_project gdn.metal:1-46, gdn_outproj gdn.metal:209-226 and
// their row-batched / block forms, which keep each row's sequence: q4_dot.metal:44-104,
// prefill_dense.metal:1-49).
void orc_q4_project(const u16* x, u32 x_stride, u32 rows, const u32* words, const u16* scales,
                    const u16* biases, u32 n, u32 k, u16* out, u32 out_stride, int fused,
                    int threads) {
    parallel_for(n, threads, [&](u32 col) {
        const u16* packed = reinterpret_cast<const u16*>(words + static_cast<u64>(col) * (k / 8));
        const u16* sc = scales + static_cast<u64>(col) * (k / 64);
        const u16* bi = biases + static_cast<u64>(col) * (k / 64);
        for (u32 r = 0; r < rows; ++r)
            out[static_cast<u64>(r) * out_stride + col] =
                bf16r(q4_dot(x + static_cast<u64>(r) * x_stride, packed, sc, bi, k, fused != 0));
    });
}

// Dequantised bf16 weights [n][k] of the tensor-unit policy.
void orc_q4_dequantize(const u32* words, const u16* scales, const u16* biases, u32 n, u32 k,
                       u16* weights) {
    for (u32 col = 0; col < n; ++col)
        for (u32 i = 0; i < k; ++i)
            weights[static_cast<u64>(col) * k + i] =
                q4_weight_bf16(words + static_cast<u64>(col) * (k / 8), scales + static_cast<u64>(col) * (k / 64),
                               biases + static_cast<u64>(col) * (k / 64), i);
}

// Tensor-unit policy: out = bf16(sum_k x[r][k] * w_bf16[col][k]), f32 accumulation in k order
// (native_dense_qgemm.metal: bf16 operands, float accumulators, bf16 store).  The accumulation
// order of a matrix unit is not specified, so this is a tolerance oracle, not a bit oracle.
void orc_project_dense(const u16* x, u32 x_stride, u32 rows, const u16* weights, u32 n, u32 k,
                       u16* out, u32 out_stride, int threads) {
    parallel_for(n, threads, [&](u32 col) {
        const u16* w = weights + static_cast<u64>(col) * k;
        for (u32 r = 0; r < rows; ++r) {
            const u16* xr = x + static_cast<u64>(r) * x_stride;
            float acc = 0.0f;
            for (u32 i = 0; i < k; ++i) acc = std::fma(bf(xr[i]), bf(w[i]), acc);
            out[static_cast<u64>(r) * out_stride + col] = bf16r(acc);
        }
    });
}

// ---- speculative-decode support: the GDN tape of a verify band and its replay ----------
// Tape geometry of the reference (tools/generate_kernel_library.py:2045-2049): 40 layers x 16
// rows; f32 regions  delta [layer][row][32 v-heads][128]  at 0,  key [layer][row][16 k-heads][128]
// at 40*16*32*128,  gates [layer][row][32][2] = (decay, beta)  after the key region.
constexpr u32 kTapeRows = 16, kTapeLayers = 40;
constexpr u64 kTapeKeyOff = static_cast<u64>(kTapeLayers) * kTapeRows * 32 * 128;
constexpr u64 kTapeGateOff = kTapeKeyOff + static_cast<u64>(kTapeLayers) * kTapeRows * 16 * 128;

u64 orc_gdn_tape_floats() { return kTapeGateOff + static_cast<u64>(kTapeLayers) * kTapeRows * 32 * 2; }

// The sequential scan that also records, per row: delta per (v-head, v-dim), the key row of each
// k-head as f32, and (decay, beta) per v-head (gdn_recurrence_gates_tape_blk,
// prefill_gdn.metal:434-527).  rows <= 16.
void orc_gdn_scan_tape(const u16* qk, const u16* value, const float* decay, const float* beta,
                       const float* state_in, u16* y, float* state_out, u32 rows, float* tape,
                       u32 tape_layer, int threads) {
    parallel_for(kGdnValueHeads * kGd, threads, [&](u32 item) {
        const u32 vh = item / kGd, vd = item % kGd;
        const u32 qbase = (vh >> 1) * kGd, kbase = kGdnQk / 2 + qbase;
        const u64 sbase = static_cast<u64>(item) * kGd;
        float state[kGd];
        for (u32 e = 0; e < kGd; ++e) state[e] = state_in[sbase + e];
        for (u32 step = 0; step < rows; ++step) {
            const u16* qkr = qk + static_cast<u64>(step) * kGdnQk;
            const float dec = decay[step * kGdnValueHeads + vh];
            const float bet = beta[step * kGdnValueHeads + vh];
            float lanes[32];
            for (u32 l = 0; l < 32; ++l) {
                float kvp = 0.0f;
                for (u32 i = 0; i < 4; ++i) {
                    const u32 e = l * 4 + i;
                    state[e] = ftz(state[e] * dec);
                    kvp = std::fma(state[e], bf(qkr[kbase + e]), kvp);
                }
                lanes[l] = kvp;
            }
            const float kv = pairs_sum(lanes, 32);
            const float v = bf(value[static_cast<u64>(step) * kGdnV + vh * kGd + vd]);
            const float delta = ftz(ftz(v - kv) * bet);
            const u64 tape_row = static_cast<u64>(tape_layer) * kTapeRows + step;
            tape[(tape_row * kGdnValueHeads + vh) * kGd + vd] = delta;
            if (vd == 0) {
                if ((vh & 1u) == 0)
                    for (u32 e = 0; e < kGd; ++e)
                        tape[kTapeKeyOff + (tape_row * kGdnKeyHeads + (vh >> 1)) * kGd + e] = bf(qkr[kbase + e]);
                tape[kTapeGateOff + (tape_row * kGdnValueHeads + vh) * 2] = dec;
                tape[kTapeGateOff + (tape_row * kGdnValueHeads + vh) * 2 + 1] = bet;
            }
            for (u32 l = 0; l < 32; ++l) {
                float o = 0.0f;
                for (u32 i = 0; i < 4; ++i) {
                    const u32 e = l * 4 + i;
                    state[e] = std::fma(bf(qkr[kbase + e]), delta, state[e]);
                    o = std::fma(state[e], bf(qkr[qbase + e]), o);
                }
                lanes[l] = o;
            }
            y[static_cast<u64>(step) * kGdnV + vh * kGd + vd] = ftzb(bf16r(pairs_sum(lanes, 32)));
        }
        for (u32 e = 0; e < kGd; ++e) state_out[sbase + e] = state[e];
    });
}

// Rebuilds the state after `steps` committed rows from the pre-band state and the tape, with the
// scan's own two update statements (gdn_tape_replay_blk, prefill_gdn.metal:529-569).
void orc_gdn_tape_replay(const float* tape, const float* state_in, float* state_out, u32 steps,
                         u32 tape_layer, int threads) {
    parallel_for(kGdnValueHeads * kGd, threads, [&](u32 item) {
        const u32 vh = item / kGd, vd = item % kGd;
        const u64 sbase = static_cast<u64>(item) * kGd;
        float state[kGd];
        for (u32 e = 0; e < kGd; ++e) state[e] = state_in[sbase + e];
        for (u32 step = 0; step < steps; ++step) {
            const u64 tape_row = static_cast<u64>(tape_layer) * kTapeRows + step;
            const float dec = tape[kTapeGateOff + (tape_row * kGdnValueHeads + vh) * 2];
            const float delta = tape[(tape_row * kGdnValueHeads + vh) * kGd + vd];
            const float* key = tape + kTapeKeyOff + (tape_row * kGdnKeyHeads + (vh >> 1)) * kGd;
            for (u32 e = 0; e < kGd; ++e) {
                state[e] = ftz(state[e] * dec);
                state[e] = std::fma(key[e], delta, state[e]);
            }
        }
        for (u32 e = 0; e < kGd; ++e) state_out[sbase + e] = state[e];
    });
}

// gdn_conv_tape_blk (prefill_gdn.metal:322-420): gdn_prepare that also records the conv tail
// (the three newest taps) after EVERY row: conv_tape [layer][16 rows][3][8192] bf16.
void orc_gdn_conv_tape(const u16* projection, const u16* conv_state, u32 rows, u16* conv_tape,
                       u32 tape_layer) {
    for (u32 row = 0; row < rows; ++row)
        for (u32 ch = 0; ch < kGdnConv; ++ch)
            for (u32 t = 0; t < 3; ++t) {
                const u32 logical = row + t + 1;
                const u16 tap = logical < 3 ? conv_state[logical * kGdnConv + ch]
                                            : projection[static_cast<u64>(logical - 3) * kGdnProj + ch];
                conv_tape[((static_cast<u64>(tape_layer) * kTapeRows + row) * 3 + t) * kGdnConv + ch] = tap;
            }
}

} // extern "C"
