// Times the wave loop (wave_loop.hpp) on a model-shaped stack: `layers` layers in the 3 gated-delta :
// 1 full-attention pattern of Qwen3.6-35B-A3B, `lanes` streams in one lane group, every stream
// joined through the owner (prompt blocks with the tensor-unit policy) to `context` positions and
// then decoded for `tokens` waves.  Beside it, the same waves walked eagerly through LayerPass with
// host tables (the reference's way: re-encode every token, src/runtime/decode_step.cpp:1002-1426).
// Prints one JSON line.  Weights and prompts are seeded synthetic data.
//
//   bench_wave_loop [--lanes 8] [--context 16384] [--tokens 64] [--layers 40] [--unit 2048]
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "tatara_b200/host/wave_loop.hpp"

using namespace tatara::runtime;
using namespace tatara::engine;
using u16 = std::uint16_t;
using Clock = std::chrono::steady_clock;

namespace {

u16 to_bf16(float v) {
    std::uint32_t b;
    std::memcpy(&b, &v, 4);
    return static_cast<u16>((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
struct Rng {
    std::uint64_t s;
    std::uint64_t next() { s ^= s >> 12; s ^= s << 25; s ^= s >> 27; return s * 0x2545F4914F6CDD1Dull; }
    float uniform() { return static_cast<float>(next() >> 40) / 16777216.0f; }
    float normal() { float a = 0; for (int i = 0; i < 12; ++i) a += uniform(); return a - 6.0f; }
};

struct Store {
    std::vector<DeviceBuffer> buffers;
    std::uint64_t bytes{0};
    const void* put(const void* host, std::size_t n) {
        buffers.emplace_back(n);
        bytes += n;
        if (!buffers.back() || cudaMemcpy(buffers.back().data(), host, n, cudaMemcpyHostToDevice) != cudaSuccess) std::exit(3);
        return buffers.back().data();
    }
    void* room(std::size_t n) {
        buffers.emplace_back(n);
        if (!buffers.back()) std::exit(3);
        return buffers.back().data();
    }
    QuantizedWeight q4(Rng& rng, std::uint32_t rows, std::uint32_t k, float gain) {
        std::vector<std::uint32_t> words(std::size_t{rows} * k / 8);
        for (auto& w : words) w = static_cast<std::uint32_t>(rng.next());
        std::vector<u16> scales(std::size_t{rows} * k / 64), biases(scales.size());
        for (std::size_t i = 0; i < scales.size(); ++i) {
            const float sc = gain * (1.0f + 0.2f * (2.0f * rng.uniform() - 1.0f));
            scales[i] = to_bf16(sc);
            biases[i] = to_bf16(-7.5f * sc * (1.0f + 0.1f * rng.normal()));
        }
        return QuantizedWeight{put(words.data(), words.size() * 4), put(scales.data(), scales.size() * 2),
                               put(biases.data(), biases.size() * 2), rows};
    }
    const void* vec(Rng& rng, std::size_t n, float scale, float shift) {
        std::vector<u16> v(n);
        for (auto& x : v) x = to_bf16(shift + scale * rng.normal());
        return put(v.data(), n * 2);
    }
};

tatara_q4_matrix as_matrix(const QuantizedWeight& w) { return tatara_q4_matrix{w.words, w.scales, w.biases, w.rows, 0}; }

double ms_since(Clock::time_point t0) { return std::chrono::duration<double, std::milli>(Clock::now() - t0).count(); }

} // namespace

int main(int argc, char** argv) {
    std::uint32_t lanes = 8, context = 16384, tokens = 64, n_layers = 40, unit = 2048;
    std::vector<std::pair<std::uint32_t, std::uint32_t>> policies;   // --policy ID*1000+VALUE: tatara_ctx_set_policy(ID, VALUE)
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string key = argv[i];
        const auto value = static_cast<std::uint32_t>(std::strtoul(argv[i + 1], nullptr, 10));
        if (key == "--policy") { policies.emplace_back(value / 1000u, value % 1000u); continue; }
        if (key == "--lanes") lanes = value;
        else if (key == "--context") context = value;
        else if (key == "--tokens") tokens = value;
        else if (key == "--layers") n_layers = value;
        else if (key == "--unit") unit = value;
        else { std::fprintf(stderr, "unknown option %s\n", key.c_str()); return 2; }
    }
    // early joiners keep decoding while the later ones join: give every stream room for those waves too
    const std::uint32_t join_waves = lanes * ((context + unit - 1) / unit) + 16;
    const std::uint32_t capacity = context + tokens + join_waves + 16;
    tatara_ctx* ctx = nullptr;
    if (tatara_ctx_create(0, &ctx) != TATARA_OK) { std::fprintf(stderr, "no B200: %s\n", "tatara_ctx_create failed"); return 4; }
    for (const auto& pv : policies)
        if (tatara_ctx_set_policy(ctx, static_cast<tatara_policy>(pv.first), pv.second) != TATARA_OK) {
            std::fprintf(stderr, "policy %u = %u refused\n", pv.first, pv.second);
            return 2;
        }

    Rng rng{0x7A7A4A5EEDull};
    Store store;
    std::vector<PathLayer> layers;
    std::uint64_t q4_bytes_attention = 0, q4_bytes_gated = 0;
    for (std::uint32_t l = 0; l < n_layers; ++l) {
        PathLayer p;
        p.kind = (l % 4 == 3) ? LayerKind::FullAttention : LayerKind::GatedDelta;
        const std::uint64_t before = store.bytes;
        tatara_q4_matrix m[4];
        std::uint32_t n = 0;
        if (p.kind == LayerKind::FullAttention) {
            p.attention = AttentionWeights{store.vec(rng, 256, 0.1f, 1.0f), store.vec(rng, 256, 0.1f, 1.0f)};
            p.attention_q4 = AttentionProjection{store.q4(rng, 8192, kHidden, 0.005f), store.q4(rng, 512, kHidden, 0.005f),
                                                 store.q4(rng, 512, kHidden, 0.005f), store.q4(rng, kHidden, 4096, 0.02f)};
            m[n++] = as_matrix(p.attention_q4.query); m[n++] = as_matrix(p.attention_q4.key); m[n++] = as_matrix(p.attention_q4.value);
            q4_bytes_attention = store.bytes - before;
        } else {
            std::vector<u16> a_log(32);
            for (auto& x : a_log) x = to_bf16(std::log(1.0f + 15.0f * rng.uniform()));
            p.gated_delta = GatedDeltaWeights{store.vec(rng, 8192 * 4, 0.5f, 0.0f), store.put(a_log.data(), 64),
                                              store.vec(rng, 32, 0.5f, 0.0f), store.vec(rng, 128, 0.1f, 1.0f)};
            p.gated_delta_q4 = GatedDeltaProjection{store.q4(rng, 8192, kHidden, 0.005f), store.q4(rng, 4096, kHidden, 0.005f),
                                                    store.q4(rng, 32, kHidden, 0.005f), store.q4(rng, 32, kHidden, 0.005f),
                                                    store.q4(rng, kHidden, 4096, 0.01f)};
            m[n++] = as_matrix(p.gated_delta_q4.qkv); m[n++] = as_matrix(p.gated_delta_q4.z);
            m[n++] = as_matrix(p.gated_delta_q4.b); m[n++] = as_matrix(p.gated_delta_q4.a);
            q4_bytes_gated = store.bytes - before;
        }
        // load-time dequantisation for the prompt blocks (tensor-unit policy)
        const std::uint32_t width = p.kind == LayerKind::FullAttention ? kAttnProjectionRows : kGdnProjectionRows;
        void* dense = store.room(std::uint64_t{width} * kHidden * 2);
        void* out_dense = store.room(std::uint64_t{kHidden} * 4096 * 2);
        const tatara_q4_matrix om[1] = {as_matrix(p.kind == LayerKind::FullAttention ? p.attention_q4.out : p.gated_delta_q4.out)};
        if (tatara_q4_dequantize(ctx, nullptr, m, n, kHidden, dense) != TATARA_OK ||
            tatara_q4_dequantize(ctx, nullptr, om, 1, 4096, out_dense) != TATARA_OK) return 5;
        p.project_dense = dense;
        p.out_dense = out_dense;
        layers.push_back(p);
    }
    if (tatara_ctx_sync(ctx, nullptr) != TATARA_OK) return 6;
    const bool verbose = std::getenv("WAVE_BENCH_VERBOSE") != nullptr;
    const auto start = Clock::now();
    if (verbose) std::fprintf(stderr, "weights ready (%.1f MB of Q4)\n", store.bytes / 1e6);

    TokenBoundary boundary;
    boundary.embed = [](std::uint32_t token, std::uint32_t, u16* row) {
        // four values in [-2, 2) per draw: cheap enough that the host side of a 2048-row unit stays small
        Rng r{0x9E3779B97F4A7C15ull ^ (std::uint64_t{token} * 0xD1B54A32D192ED03ull + 1)};
        for (std::uint32_t i = 0; i < kHidden; i += 4) {
            const std::uint64_t bits = r.next();
            for (std::uint32_t j = 0; j < 4; ++j)
                row[i + j] = to_bf16(static_cast<float>(static_cast<std::int16_t>(bits >> (16 * j))) * (1.0f / 16384.0f));
        }
    };
    boundary.sample = [](const u16* row) {
        std::uint64_t h = 0xCBF29CE484222325ull;
        for (std::uint32_t i = 0; i < kHidden; ++i) h = (h ^ row[i]) * 0x100000001B3ull;
        return static_cast<std::uint32_t>(h % 50021u);
    };

    double join_ms = 0, wave_ms = 0;
    std::uint64_t graphs = 0, launches_per_wave = 0;
    {
        OwnerConfig config{0, 1, lanes, capacity, std::min<std::uint32_t>(lanes, 2), unit, 5000, {}};
        for (const auto& pv : policies) config.policies.emplace_back(pv.first, pv.second);
        MultiStreamOwner owner(config, layers, boundary);
        if (!owner) { std::fprintf(stderr, "owner failed to build\n"); return 7; }
        if (verbose) std::fprintf(stderr, "owner built, %.1f ms since start\n", ms_since(start));
        std::vector<std::shared_ptr<LaneChannel>> channels;
        for (std::uint32_t s = 0; s < lanes; ++s) {
            OwnerSubmission sub;
            sub.prompt.resize(context + 1);
            for (std::uint32_t i = 0; i <= context; ++i) sub.prompt[i] = (s * 7919u + i * 104729u) % 50021u;
            sub.maximum_tokens = tokens + join_waves;
            sub.channel = std::make_shared<LaneChannel>();
            sub.cancelled = std::make_shared<std::atomic<bool>>(false);
            channels.push_back(sub.channel);
            if (!owner.submit(std::move(sub))) return 8;
        }
        // joins: until every lane decodes (the early lanes already produce tokens meanwhile)
        const auto j0 = Clock::now();
        std::size_t rows = 0;
        const int wave_limit = static_cast<int>(join_waves) + 8;
        for (int guard = 0; guard < wave_limit && rows < lanes && owner.last_error() == CommandError::None; ++guard) {
            rows = owner.run_wave();
            if (verbose) std::fprintf(stderr, "wave %d: %zu rows, %.1f ms since start\n", guard, rows, ms_since(start));
            if (ms_since(j0) > 120000.0) break;   // this program is a timing aid: never sit on a GPU
        }
        join_ms = ms_since(j0);
        if (rows != lanes || owner.last_error() != CommandError::None) {
            std::fprintf(stderr, "joins failed after %.0f ms: %zu of %u rows decode, join units %llu, last error %s, timed-out stream %d at step %d\n",
                         join_ms, rows, lanes, static_cast<unsigned long long>(owner.statistics().join_units),
                         to_string(owner.last_error()), owner.statistics().last_timeout_stream, owner.statistics().last_timeout_mark);
            std::_Exit(9);   // a submission may still be in flight: leave without waiting for it
        }
        // the last joiner has at least `tokens` tokens to go: time full waves
        for (int i = 0; i < 3; ++i) (void)owner.run_wave();
        const std::uint32_t timed = tokens > 8 ? tokens - 8 : 1;
        const auto w0 = Clock::now();
        for (std::uint32_t i = 0; i < timed; ++i)
            if (owner.run_wave() != lanes) { std::fprintf(stderr, "a wave lost rows\n"); return 10; }
        wave_ms = ms_since(w0) / timed;
        graphs = owner.statistics().graphs_captured;
        owner.stop();
    }

    // the same token walked eagerly with host tables at the same contexts (zeroed caches: timing only)
    double eager_ms = 0;
    {
        std::vector<LayerKind> schedule;
        for (const PathLayer& l : layers) schedule.push_back(l.kind);
        DecodeStatePool pool;
        std::vector<DecodeStateSlot> slots;
        DecodeBatchScratch scratch;
        if (!create_state_pool(lanes, capacity, schedule, pool, slots) || !create_batch_scratch(lanes, capacity, scratch)) return 11;
        DeviceBuffer hidden[2] = {DeviceBuffer(std::uint64_t{lanes} * kHidden * 2), DeviceBuffer(std::uint64_t{lanes} * kHidden * 2)};
        DeviceBuffer slab(std::uint64_t{lanes} * kGdnProjectionRows * 2);
        PinnedBuffer rows_in(std::uint64_t{lanes} * kHidden * 2), rows_out(std::uint64_t{lanes} * kHidden * 2);
        cudaStream_t stream = nullptr;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return 12;
        std::vector<std::uint32_t> input(lanes, 17);
        const std::uint32_t timed = tokens > 8 ? tokens - 8 : 1;
        Clock::time_point t0;
        for (std::uint32_t t = 0; t < timed + 3; ++t) {
            if (t == 3) t0 = Clock::now();
            std::vector<DecodeStream> streams;
            for (std::uint32_t s = 0; s < lanes; ++s) {
                streams.push_back({&slots[s], context + t});
                boundary.embed(input[s], context + t, rows_in.as<u16>() + std::uint64_t{s} * kHidden);
            }
            cudaMemcpyAsync(hidden[0].data(), rows_in.as<void>(), rows_in.bytes(), cudaMemcpyHostToDevice, stream);
            LayerPass pass(ctx, stream);
            std::uint32_t cur = 0;
            for (std::uint32_t l = 0; l < n_layers; ++l) {
                if (layers[l].kind == LayerKind::FullAttention) {
                    pass.encode_attention_project(layers[l].attention_q4, hidden[cur].data(), lanes, slab.data());
                    pass.encode_attention(pool, l, layers[l].attention, streams, slab.data(), scratch);
                    pass.encode_out_projection(layers[l].attention_q4.out, scratch.attended.data(), lanes, hidden[cur ^ 1].data(), kHidden);
                } else {
                    pass.encode_gated_delta_project(layers[l].gated_delta_q4, hidden[cur].data(), lanes, slab.data());
                    pass.encode_gated_delta(pool, l, layers[l].gated_delta, streams, slab.data(), scratch);
                    pass.encode_out_projection(layers[l].gated_delta_q4.out, scratch.gdn_gated.data(), lanes, hidden[cur ^ 1].data(), kHidden);
                }
                cur ^= 1u;
            }
            cudaMemcpyAsync(rows_out.as<void>(), hidden[cur].data(), rows_out.bytes(), cudaMemcpyDeviceToHost, stream);
            if (pass.commit_and_wait() != CommandError::None) { std::fprintf(stderr, "eager walk failed: %s\n", to_string(pass.error())); return 13; }
            advance_decode_state(pool, streams);
            for (std::uint32_t s = 0; s < lanes; ++s) input[s] = boundary.sample(rows_out.as<u16>() + std::uint64_t{s} * kHidden);
        }
        eager_ms = ms_since(t0) / timed;
        launches_per_wave = 0;
        for (std::uint32_t l = 0; l < n_layers; ++l) launches_per_wave += layers[l].kind == LayerKind::FullAttention ? 5 : 3;
        cudaStreamDestroy(stream);
    }
    tatara_ctx_destroy(ctx);

    // bytes one wave must read: every layer's Q4 weights once, every lane's K/V rows and gated-delta state
    const std::uint32_t n_attention = n_layers / 4, n_gated = n_layers - n_attention;
    const double kv_bytes = double(lanes) * n_attention * 2.0 * 2.0 * 256.0 * 2.0 * (context + tokens / 2.0);
    const double state_bytes = double(lanes) * n_gated * 2.0 * (kGdnRecurrentStateValues * 4.0 + kGdnConvStateValues * 2.0);
    const double weight_bytes = double(n_attention) * q4_bytes_attention + double(n_gated) * q4_bytes_gated;
    const double wave_bytes = kv_bytes + state_bytes + weight_bytes;
    std::printf(
        "{\"workload\": \"wave_loop\", \"layers\": %u, \"lanes\": %u, \"context\": %u, \"join_unit_rows\": %u, "
        "\"join_ms_total\": %.3f, \"join_rows_per_s\": %.1f, \"wave_ms_graph\": %.4f, \"wave_ms_eager_host_tables\": %.4f, "
        "\"tokens_per_s_graph\": %.1f, \"kernel_launches_per_wave\": %llu, \"graphs_captured\": %llu, "
        "\"wave_bytes\": %.0f, \"wave_gbs\": %.1f, \"timing\": \"host clock around run_wave (embed, graph launch, sync, sample)\"}\n",
        n_layers, lanes, context, unit, join_ms, double(lanes) * context / (join_ms * 1e-3), wave_ms, eager_ms,
        lanes / (wave_ms * 1e-3), static_cast<unsigned long long>(launches_per_wave), static_cast<unsigned long long>(graphs),
        wave_bytes, wave_bytes / (wave_ms * 1e-3) / 1e9);
    return 0;
}
