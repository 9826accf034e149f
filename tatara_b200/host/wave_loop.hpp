// The engine's wave loop over this library's slice of the token walk (reference:
// MultiStreamOwner, tools/native/tatara_serve.cpp:1173-1200, 1293-1777; encode_token_batch,
// src/runtime/decode_step.cpp:1002-1426).  Header-only C++17 above hybrid_layers.hpp.
//
// What is kept from the reference: the owner thread's loop (admit joiners onto free lanes,
// preferring a lane group with no join in flight; advance every joining prompt by one unit
// submission per wave beside the decode work; one batched submission per lane group; settle:
// advance_decode_state, ++context, ++produced, stop ids / maximum_tokens / cancellation), the
// lane / submission / channel vocabulary, the wave statistics, and the rule that a stream's
// bytes do not depend on which other streams share its wave.
//
// What is different, because this is a CUDA device and not a Metal queue: a wave's decode token
// is not re-encoded.  Per lane group and per row count it is captured ONCE as a CUDA graph whose
// first nodes copy the wave's lane tables (state stripes, contexts, gated-delta parities) and the
// rows' input vectors from pinned host memory; the kernels read the tables from device memory, so
// the same graph serves every later wave of that size whatever its streams and contexts.
// Everything of a wave goes into ONE CUDA stream, decode graphs first and the joining prompts'
// units behind them: the kernels of this library each fill the device, and its cluster /
// tensor-memory kernels (tatara_project_dense, tatara_attn_prefill) are only ever issued with
// nothing else in flight.  join_unit_rows bounds what a joining prompt adds to a wave.
//
// The walk covers the layers this library implements: per layer the fused projection, the
// attention or gated-delta step and the out projection.  Embedding, the MoE / norm stages between
// layers and the LM head + sampler are outside it; TokenBoundary stands in for them on the host
// (embed: token -> first layer's input row; sample: last layer's output row -> token).
#pragma once

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>

#include "hybrid_layers.hpp"

namespace tatara::engine {

namespace rt = tatara::runtime;

enum class LaneDoneReason : std::uint8_t { Stopped, Length, Cancelled, Failed };

struct LaneChannel {
    std::mutex mutex;
    std::condition_variable ready;
    std::deque<std::uint32_t> tokens;
    bool done{false};
    LaneDoneReason reason{LaneDoneReason::Failed};
};

struct OwnerSubmission {
    std::vector<std::uint32_t> prompt;
    std::vector<std::uint32_t> stop_ids;
    std::uint32_t maximum_tokens{0};
    std::shared_ptr<LaneChannel> channel;
    std::shared_ptr<std::atomic<bool>> cancelled;
};

// One layer of the walk with everything its three steps bind.
struct PathLayer {
    rt::LayerKind kind{rt::LayerKind::GatedDelta};
    rt::AttentionWeights attention{};
    rt::AttentionProjection attention_q4{};
    rt::GatedDeltaWeights gated_delta{};
    rt::GatedDeltaProjection gated_delta_q4{};
    // Tensor-unit policy for prompt blocks: the same weights dequantised to bf16 (tatara_q4_dequantize).
    // Null keeps the exact per-row sequence for prompt blocks too.
    const void* project_dense{nullptr};   // [9216 or 12352][2048] bf16
    const void* out_dense{nullptr};       // [2048][4096] bf16
};

struct TokenBoundary {
    std::function<void(std::uint32_t token, std::uint32_t position, std::uint16_t* row)> embed;  // row: [2048] bf16
    std::function<std::uint32_t(const std::uint16_t* row)> sample;
};

struct OwnerConfig {
    int device{0};
    std::uint32_t groups{1};
    std::uint32_t lanes_per_group{8};   // the reference stripes up to eight lanes over one pool group
    std::uint32_t capacity{4096};
    std::uint32_t join_streams{2};      // join slots: prompts that advance side by side, one unit each per wave
    std::uint32_t join_unit_rows{256};  // prompt rows one join submission places
    std::uint32_t wait_limit_ms{30000}; // a submission that has not completed by then fails its lanes
    // tatara_ctx_set_policy(id, value) for every context the owner creates (its lane groups' and the join slots')
    std::vector<std::pair<std::uint32_t, std::uint64_t>> policies;
};

struct WaveStatistics {
    std::uint64_t wave_count{0}, wave_rows_total{0}, wave_rows_max{0}, full_wave_count{0};
    double wave_ms_total{0}, full_wave_ms_total{0};
    std::uint64_t graphs_captured{0}, graph_launches{0}, join_units{0};
    std::uint64_t wait_timeouts{0};
    int last_timeout_stream{-1};   // lane group index, or 1000 + join slot index
    int last_timeout_mark{-1};     // join slots: first step of the unit that had not completed (3 * layer + step)
};

class PinnedBuffer {
  public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(std::uint64_t bytes) : bytes_(bytes) {
        if (bytes == 0 || cudaHostAlloc(&ptr_, bytes, cudaHostAllocDefault) != cudaSuccess) {
            ptr_ = nullptr;
            bytes_ = 0;
        } else {
            std::memset(ptr_, 0, bytes);
        }
    }
    PinnedBuffer(PinnedBuffer&& o) noexcept : ptr_(std::exchange(o.ptr_, nullptr)), bytes_(std::exchange(o.bytes_, 0)) {}
    PinnedBuffer& operator=(PinnedBuffer&& o) noexcept {
        if (this != &o) {
            if (ptr_ != nullptr) cudaFreeHost(ptr_);
            ptr_ = std::exchange(o.ptr_, nullptr);
            bytes_ = std::exchange(o.bytes_, 0);
        }
        return *this;
    }
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    ~PinnedBuffer() {
        if (ptr_ != nullptr) cudaFreeHost(ptr_);
    }
    explicit operator bool() const noexcept { return ptr_ != nullptr; }
    template <typename T> T* as() const noexcept { return static_cast<T*>(ptr_); }
    std::uint64_t bytes() const noexcept { return bytes_; }

  private:
    void* ptr_ = nullptr;
    std::uint64_t bytes_ = 0;
};

// One pool group: lanes striped over shared state pools with their own batch scratch
// (OwnerLaneGroup, tools/native/tatara_serve.cpp:1191-1197), plus what the captured wave needs:
// a context of its own (the owner's stream), the lane tables and row vectors in pinned and device
// memory, and one executable graph per row count.
struct OwnerLaneGroup {
    rt::DecodeStatePool pool;
    std::vector<rt::DecodeStateSlot> slots;
    rt::DecodeBatchScratch batch_scratch;
    tatara_ctx* ctx{nullptr};
    cudaStream_t stream{nullptr};
    PinnedBuffer tables_host, rows_in_host, rows_out_host;
    rt::DeviceBuffer tables, hidden[2], projection_slab;
    std::vector<cudaGraphExec_t> graphs;   // index = rows in the wave
};

// A join slot: one prompt head being placed, one unit per wave (JoiningLane, tatara_serve.cpp:1343-1347).
// stream and ctx are the owner's (shared by every slot).
struct JoinStream {
    cudaStream_t stream{nullptr};
    tatara_ctx* ctx{nullptr};
    PinnedBuffer rows_host;
    rt::DeviceBuffer hidden[2], projection_slab, query, gate, attended, qk, value, z, decay, beta, y, gated, scan_scratch;
    std::vector<cudaEvent_t> marks;   // one per step of a unit (projection, layer body, out projection per layer)
};

class MultiStreamOwner {
  public:
    struct Lane {
        rt::DecodeStateSlot* slot{nullptr};
        std::uint32_t stripe{0};
        std::uint32_t group{0};
        bool dirty{false};
        bool active{false};
        OwnerSubmission request;
        std::uint32_t context{0};
        std::uint32_t pending_input{0};
        std::uint64_t produced{0};
    };
    struct JoiningLane {
        Lane* lane{nullptr};
        std::uint32_t head{0};     // prompt tokens the join places (all but the last)
        std::uint32_t placed{0};
        std::uint32_t in_flight{0};
        JoinStream io;
    };

    MultiStreamOwner(const OwnerConfig& config, std::vector<PathLayer> layers, TokenBoundary boundary)
        : config_(config), layers_(std::move(layers)), boundary_(std::move(boundary)) {
        ok_ = build();
    }
    MultiStreamOwner(const MultiStreamOwner&) = delete;
    MultiStreamOwner& operator=(const MultiStreamOwner&) = delete;
    ~MultiStreamOwner() {
        // After a wait that ran out the stream may never drain: leave its resources to the context
        // instead of blocking the owner's thread for good.
        if (stats_.wait_timeouts != 0) return;
        if (stream_ != nullptr) cudaStreamSynchronize(stream_);
        for (OwnerLaneGroup& g : groups_) {
            for (cudaGraphExec_t e : g.graphs)
                if (e != nullptr) cudaGraphExecDestroy(e);
            if (g.ctx != nullptr) tatara_ctx_destroy(g.ctx);
        }
        if (stream_ != nullptr) cudaStreamDestroy(stream_);
        for (JoiningLane& j : joining_)
            for (cudaEvent_t e : j.io.marks) cudaEventDestroy(e);
        if (join_ctx_ != nullptr) tatara_ctx_destroy(join_ctx_);
    }
    explicit operator bool() const noexcept { return ok_; }
    const WaveStatistics& statistics() const noexcept { return stats_; }
    const std::vector<Lane>& lanes() const noexcept { return lanes_; }
    rt::CommandError last_error() const noexcept { return last_error_; }

    // Queues a request; false when the prompt is empty, does not fit a lane or the owner is stopping.
    bool submit(OwnerSubmission submission) {
        if (submission.prompt.empty() || submission.prompt.size() >= config_.capacity || !submission.channel ||
            !submission.cancelled)
            return false;
        {
            std::lock_guard<std::mutex> guard(queue_mutex_);
            if (!running_) return false;
            queue_.push_back(std::move(submission));
            ++outstanding_;
        }
        queue_ready_.notify_all();
        return true;
    }
    void stop() {
        {
            std::lock_guard<std::mutex> guard(queue_mutex_);
            running_ = false;
        }
        queue_ready_.notify_all();
    }
    std::uint64_t outstanding() {
        std::lock_guard<std::mutex> guard(queue_mutex_);
        return outstanding_;
    }

    // The owner thread's loop: waves until stopped and drained.
    void run() {
        while (true) {
            (void)run_wave();
            std::unique_lock<std::mutex> guard(queue_mutex_);
            const bool any_active =
                std::any_of(lanes_.begin(), lanes_.end(), [](const Lane& l) { return l.active; });
            const bool any_joining =
                std::any_of(joining_.begin(), joining_.end(), [](const JoiningLane& j) { return j.lane != nullptr; });
            if (!running_ && queue_.empty() && !any_active && !any_joining) return;
            if (!any_active && queue_.empty() && !any_joining)
                queue_ready_.wait_for(guard, std::chrono::milliseconds(5), [&] { return !queue_.empty() || !running_; });
        }
    }

    // One iteration of the loop: admit, one unit per joining prompt, one decode token for every
    // active lane, settle.  Returns the number of rows that decoded in this wave.
    std::size_t run_wave() {
        admit_joiners();

        const auto wave_start = std::chrono::steady_clock::now();
        wave_.clear();
        for (Lane& lane : lanes_) {
            if (!lane.active) continue;
            if (lane.request.cancelled->load()) {
                finish(lane, LaneDoneReason::Cancelled);
                continue;
            }
            wave_.push_back(&lane);
        }
        for (std::vector<Lane*>& plan : plans_) plan.clear();
        for (Lane* lane : wave_) plans_[lane->group].push_back(lane);
        submitted_.assign(groups_.size(), false);
        for (std::size_t g = 0; g < plans_.size(); ++g) {
            if (plans_[g].empty()) continue;
            const rt::CommandError e = submit_token_batch(groups_[g], plans_[g]);
            if (e != rt::CommandError::None) {
                last_error_ = e;
                for (Lane* lane : plans_[g]) finish(*lane, LaneDoneReason::Failed);
                continue;
            }
            submitted_[g] = true;
        }
        for (JoiningLane& stream : joining_) submit_join_units(stream);   // behind the decode graphs
        for (JoiningLane& stream : joining_) settle_join_units(stream);
        for (std::size_t g = 0; g < plans_.size(); ++g) {
            if (!submitted_[g]) continue;
            OwnerLaneGroup& group = groups_[g];
            const tatara_status st = wait_until_completed(group.ctx, group.stream, static_cast<int>(g));
            if (st != TATARA_OK) {
                last_error_ = rt::to_command_error(st);
                for (Lane* lane : plans_[g]) finish(*lane, LaneDoneReason::Failed);
                continue;
            }
            for (std::size_t row = 0; row < plans_[g].size(); ++row)
                settle(group, *plans_[g][row], boundary_.sample(group.rows_out_host.as<std::uint16_t>() + row * rt::kHidden));
        }
        const std::size_t rows = wave_.size();
        if (rows > 0) {
            const double wave_ms =
                std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - wave_start).count();
            stats_.wave_count += 1;
            stats_.wave_ms_total += wave_ms;
            stats_.wave_rows_total += rows;
            stats_.wave_rows_max = std::max<std::uint64_t>(stats_.wave_rows_max, rows);
            if (rows == stats_.wave_rows_max) {
                stats_.full_wave_count += 1;
                stats_.full_wave_ms_total += wave_ms;
            }
        }
        return rows;
    }

  private:
    static constexpr std::uint64_t kRowBytes = std::uint64_t{rt::kHidden} * 2;

    // wait_until_completed with a limit: the owner thread never blocks for good on a submission
    // (every device-side wait of the library is bounded too, so this is the last line).
    tatara_status wait_until_completed(tatara_ctx* ctx, cudaStream_t stream, int which) {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(config_.wait_limit_ms);
        while (true) {
            const cudaError_t q = cudaStreamQuery(stream);
            if (q == cudaSuccess) return tatara_ctx_sync(ctx, stream);
            if (q != cudaErrorNotReady) return TATARA_CUDA_ERROR;
            if (std::chrono::steady_clock::now() > deadline) {
                stats_.wait_timeouts += 1;
                stats_.last_timeout_stream = which;
                return TATARA_DEVICE_WAIT_TIMEOUT;
            }
        }
    }

    bool apply_policies(tatara_ctx* ctx) const {
        // A wave walks the layers in order (projection, step, out projection, next layer): no kernel reads
        // the state a gated-delta step writes before that step's launch has completed, so the step may let
        // its successors be staged early.  A caller's own policies come after and may undo this.
        if (tatara_ctx_set_policy(ctx, TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS, 1) != TATARA_OK) return false;
        for (const auto& pv : config_.policies)
            if (tatara_ctx_set_policy(ctx, static_cast<tatara_policy>(pv.first), pv.second) != TATARA_OK) return false;
        return true;
    }

    bool build() {
        if (layers_.empty() || config_.groups == 0 || config_.lanes_per_group == 0 ||
            config_.lanes_per_group > rt::kMaximumBatchRows || config_.join_unit_rows == 0 || !boundary_.embed ||
            !boundary_.sample || cudaSetDevice(config_.device) != cudaSuccess)
            return false;
        std::vector<rt::LayerKind> schedule;
        for (const PathLayer& l : layers_) {
            schedule.push_back(l.kind);
            if (l.kind == rt::LayerKind::GatedDelta) gdn_index_.push_back(gdn_layers_++);
            else gdn_index_.push_back(0);
        }
        if (cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking) != cudaSuccess) return false;
        const std::uint32_t rows = config_.lanes_per_group;
        groups_.resize(config_.groups);
        plans_.resize(config_.groups);
        for (std::uint32_t g = 0; g < config_.groups; ++g) {
            OwnerLaneGroup& group = groups_[g];
            if (!rt::create_state_pool(rows, config_.capacity, schedule, group.pool, group.slots) ||
                !rt::create_batch_scratch(rows, config_.capacity, group.batch_scratch) ||
                tatara_ctx_create(config_.device, &group.ctx) != TATARA_OK || !apply_policies(group.ctx))
                return false;
            group.stream = stream_;
            group.tables_host = PinnedBuffer(table_bytes());
            group.rows_in_host = PinnedBuffer(rows * kRowBytes);
            group.rows_out_host = PinnedBuffer(rows * kRowBytes);
            group.tables = rt::DeviceBuffer(table_bytes());
            group.hidden[0] = rt::DeviceBuffer(rows * kRowBytes);
            group.hidden[1] = rt::DeviceBuffer(rows * kRowBytes);
            group.projection_slab = rt::DeviceBuffer(std::uint64_t{rows} * rt::kGdnProjectionRows * 2);
            if (!group.tables_host || !group.rows_in_host || !group.rows_out_host || !group.tables || !group.hidden[0] ||
                !group.hidden[1] || !group.projection_slab)
                return false;
            group.graphs.assign(rows + 1, nullptr);
            for (std::uint32_t s = 0; s < rows; ++s) {
                Lane lane;
                lane.slot = &group.slots[s];
                lane.stripe = s;
                lane.group = g;
                lanes_.push_back(std::move(lane));
            }
        }
        joining_.resize(config_.join_streams);
        const std::uint64_t u = config_.join_unit_rows;
        if (tatara_ctx_create(config_.device, &join_ctx_) != TATARA_OK || !apply_policies(join_ctx_)) return false;
        for (JoiningLane& j : joining_) {
            JoinStream& io = j.io;
            io.ctx = join_ctx_;
            io.stream = stream_;
            io.marks.assign(3 * layers_.size(), nullptr);
            for (cudaEvent_t& e : io.marks)
                if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return false;
            io.rows_host = PinnedBuffer(u * kRowBytes);
            io.hidden[0] = rt::DeviceBuffer(u * kRowBytes);
            io.hidden[1] = rt::DeviceBuffer(u * kRowBytes);
            io.projection_slab = rt::DeviceBuffer(u * rt::kGdnProjectionRows * 2);
            const std::uint64_t wide = u * rt::kAttnQueryValues * 2;
            io.query = rt::DeviceBuffer(wide);
            io.gate = rt::DeviceBuffer(wide);
            io.attended = rt::DeviceBuffer(wide);
            io.qk = rt::DeviceBuffer(wide);
            io.value = rt::DeviceBuffer(wide);
            io.z = rt::DeviceBuffer(wide);
            io.y = rt::DeviceBuffer(wide);
            io.gated = rt::DeviceBuffer(wide);
            io.decay = rt::DeviceBuffer(u * 32 * 4);
            io.beta = rt::DeviceBuffer(u * 32 * 4);
            io.scan_scratch = rt::DeviceBuffer(tatara_gdn_prefill_scratch_bytes(config_.join_unit_rows));
            if (!io.rows_host || !io.hidden[0] || !io.hidden[1] || !io.projection_slab || !io.query || !io.gate ||
                !io.attended || !io.qk || !io.value || !io.z || !io.y || !io.gated || !io.decay || !io.beta ||
                !io.scan_scratch)
                return false;
        }
        // every buffer above was zero-filled on the default stream; the owner's stream does not order behind it
        return cudaDeviceSynchronize() == cudaSuccess;
    }

    // Lane tables of one wave: [rows] attention rows, then [gated-delta layers][rows] rows.
    std::uint64_t gdn_table_offset() const { return std::uint64_t{config_.lanes_per_group} * sizeof(tatara_attn_lane); }
    std::uint64_t table_bytes() const {
        return gdn_table_offset() +
               std::uint64_t{std::max<std::uint32_t>(gdn_layers_, 1)} * config_.lanes_per_group * sizeof(tatara_gdn_lane);
    }

    void finish(Lane& lane, LaneDoneReason reason) {
        {
            std::lock_guard<std::mutex> guard(lane.request.channel->mutex);
            lane.request.channel->done = true;
            lane.request.channel->reason = reason;
        }
        lane.request.channel->ready.notify_all();
        lane.request = OwnerSubmission{};
        lane.active = false;
        lane.dirty = true;
        std::lock_guard<std::mutex> guard(queue_mutex_);
        --outstanding_;
    }
    void push_token(Lane& lane, std::uint32_t token) {
        {
            std::lock_guard<std::mutex> guard(lane.request.channel->mutex);
            lane.request.channel->tokens.push_back(token);
        }
        lane.request.channel->ready.notify_all();
    }

    // Zeroes the slot's gated-delta state and clears its parities.  K/V rows need no reset: a
    // position is always written (qk_rope) before any query attends it.
    bool reset_state_slot(Lane& lane) {
        OwnerLaneGroup& group = groups_[lane.group];
        for (std::size_t l = 0; l < group.pool.layers.size(); ++l) {
            rt::DecodeStatePoolLayer& pl = group.pool.layers[l];
            if (pl.kind != rt::LayerKind::GatedDelta) continue;
            auto* conv = static_cast<std::uint8_t*>(pl.first.data()) + 2ull * lane.stripe * pl.first_stride * 2;
            auto* rec = static_cast<std::uint8_t*>(pl.second.data()) + 2ull * lane.stripe * pl.second_stride * 4;
            if (cudaMemsetAsync(conv, 0, 2 * pl.first_stride * 2, group.stream) != cudaSuccess ||
                cudaMemsetAsync(rec, 0, 2 * pl.second_stride * 4, group.stream) != cudaSuccess)
                return false;
        }
        if (cudaStreamSynchronize(group.stream) != cudaSuccess) return false;
        lane.slot->swapped.assign(group.pool.layers.size(), false);
        lane.slot->status = rt::DecodeStateSlotStatus::Ready;
        return true;
    }

    // Admit joiners while join slots are available, preferring a free lane in a group with no
    // join in flight (tatara_serve.cpp:1471-1524).
    void admit_joiners() {
        while (true) {
            const bool stream_free =
                std::any_of(joining_.begin(), joining_.end(), [](const JoiningLane& j) { return j.lane == nullptr; });
            if (!stream_free) break;
            OwnerSubmission next;
            Lane* free_lane = nullptr;
            {
                std::lock_guard<std::mutex> guard(queue_mutex_);
                if (queue_.empty()) break;
                Lane* fallback = nullptr;
                for (Lane& lane : lanes_) {
                    bool lane_joining = false, group_joining = false;
                    for (const JoiningLane& stream : joining_) {
                        lane_joining = lane_joining || stream.lane == &lane;
                        group_joining = group_joining || (stream.lane != nullptr && stream.lane->group == lane.group);
                    }
                    if (lane.active || lane_joining) continue;
                    if (!group_joining) {
                        free_lane = &lane;
                        break;
                    }
                    if (fallback == nullptr) fallback = &lane;
                }
                if (free_lane == nullptr) free_lane = fallback;
                if (free_lane == nullptr) break;
                next = std::move(queue_.front());
                queue_.pop_front();
            }
            (void)begin_join(*free_lane, std::move(next));
        }
    }

    bool begin_join(Lane& lane, OwnerSubmission submission) {
        lane.request = std::move(submission);
        if (lane.dirty && !reset_state_slot(lane)) {
            finish(lane, LaneDoneReason::Failed);
            return false;
        }
        lane.dirty = false;
        const std::vector<std::uint32_t>& prompt = lane.request.prompt;
        const auto head = static_cast<std::uint32_t>(prompt.size()) - 1u;
        if (head == 0) {
            lane.context = 0;
            lane.pending_input = prompt.back();
            lane.produced = 0;
            lane.active = true;
            return true;
        }
        for (JoiningLane& candidate : joining_) {
            if (candidate.lane != nullptr) continue;
            candidate.lane = &lane;
            candidate.head = head;
            candidate.placed = 0;
            candidate.in_flight = 0;
            return true;
        }
        return false;
    }

    // Encodes one unit of the in-flight join: rows [placed, placed + n) of the prompt head.
    void submit_join_units(JoiningLane& stream) {
        if (stream.lane == nullptr) return;
        Lane& lane = *stream.lane;
        if (lane.request.cancelled->load()) {
            finish(lane, LaneDoneReason::Cancelled);
            stream.lane = nullptr;
            return;
        }
        const std::uint32_t rows = std::min(config_.join_unit_rows, stream.head - stream.placed);
        for (std::uint32_t r = 0; r < rows; ++r)
            boundary_.embed(lane.request.prompt[stream.placed + r], stream.placed + r,
                            stream.io.rows_host.as<std::uint16_t>() + std::uint64_t{r} * rt::kHidden);
        const rt::CommandError e = encode_prefill_unit(stream, lane, rows);
        if (e != rt::CommandError::None) {
            last_error_ = e;
            cudaStreamSynchronize(stream.io.stream);
            finish(lane, LaneDoneReason::Failed);
            stream.lane = nullptr;
            return;
        }
        stream.in_flight = rows;
        stats_.join_units += 1;
    }

    void settle_join_units(JoiningLane& stream) {
        if (stream.lane == nullptr || stream.in_flight == 0) return;
        Lane& lane = *stream.lane;
        const tatara_status st =
            wait_until_completed(stream.io.ctx, stream.io.stream, 1000 + static_cast<int>(&stream - joining_.data()));
        if (st != TATARA_OK) {
            last_error_ = rt::to_command_error(st);
            if (st == TATARA_DEVICE_WAIT_TIMEOUT)
                for (std::size_t m = 0; m < stream.io.marks.size(); ++m)
                    if (cudaEventQuery(stream.io.marks[m]) != cudaSuccess) {
                        if (stats_.last_timeout_mark < 0) stats_.last_timeout_mark = static_cast<int>(m);
                        break;
                    }
            finish(lane, LaneDoneReason::Failed);
            stream.lane = nullptr;
            return;
        }
        // the unit wrote the other parity of every gated-delta pair
        const rt::DecodeStream one{lane.slot, stream.placed};
        rt::advance_decode_state(groups_[lane.group].pool, {one});
        stream.placed += stream.in_flight;
        stream.in_flight = 0;
        if (stream.placed == stream.head) {
            lane.context = stream.head;
            lane.pending_input = lane.request.prompt.back();
            lane.produced = 0;
            lane.active = true;
            stream.lane = nullptr;
        }
    }

    static tatara_q4_matrix as_matrix(const rt::QuantizedWeight& w) noexcept {
        return tatara_q4_matrix{w.words, w.scales, w.biases, w.rows, 0};
    }

    // Prompt rows through every layer: projection, qk_rope + causal block attention or conv + gates +
    // chunked recurrence + gate-norm, out projection (src/runtime/prefill_step.cpp:1450-1465, 1661-1683,
    // 1936-1943, 2003-2024).
    rt::CommandError encode_prefill_unit(JoiningLane& stream, Lane& lane, std::uint32_t rows) {
        JoinStream& io = stream.io;
        OwnerLaneGroup& group = groups_[lane.group];
        cudaStream_t s = io.stream;
        if (cudaMemcpyAsync(io.hidden[0].data(), io.rows_host.as<void>(), rows * kRowBytes, cudaMemcpyHostToDevice, s) !=
            cudaSuccess)
            return rt::CommandError::CudaError;
        std::uint32_t cur = 0;
        tatara_status st = TATARA_OK;
        for (std::size_t l = 0; l < layers_.size() && st == TATARA_OK; ++l) {
            const PathLayer& layer = layers_[l];
            rt::DecodeStatePoolLayer& pl = group.pool.layers[l];
            const void* in = io.hidden[cur].data();
            void* out = io.hidden[cur ^ 1u].data();
            const bool attention = layer.kind == rt::LayerKind::FullAttention;
            const std::uint32_t width = attention ? rt::kAttnProjectionRows : rt::kGdnProjectionRows;
            if (layer.project_dense != nullptr) {
                st = tatara_project_dense(io.ctx, s, in, rt::kHidden, rows, layer.project_dense, width, rt::kHidden,
                                          io.projection_slab.data(), width);
            } else if (attention) {
                const tatara_q4_matrix m[3] = {as_matrix(layer.attention_q4.query), as_matrix(layer.attention_q4.key),
                                               as_matrix(layer.attention_q4.value)};
                st = tatara_q4_project(io.ctx, s, in, rt::kHidden, rows, m, 3, rt::kHidden, io.projection_slab.data(), width);
            } else {
                const tatara_q4_matrix m[4] = {as_matrix(layer.gated_delta_q4.qkv), as_matrix(layer.gated_delta_q4.z),
                                               as_matrix(layer.gated_delta_q4.b), as_matrix(layer.gated_delta_q4.a)};
                st = tatara_q4_project(io.ctx, s, in, rt::kHidden, rows, m, 4, rt::kHidden, io.projection_slab.data(), width);
            }
            if (st != TATARA_OK) break;
            cudaEventRecord(io.marks[3 * l], s);
            const void* branch_in = nullptr;
            if (attention) {
                auto* keys = static_cast<std::uint16_t*>(pl.first.data()) + std::uint64_t{lane.stripe} * pl.first_stride;
                auto* values = static_cast<std::uint16_t*>(pl.second.data()) + std::uint64_t{lane.stripe} * pl.second_stride;
                st = tatara_attn_qk_rope(io.ctx, s, io.projection_slab.data(), layer.attention.q_norm, layer.attention.k_norm,
                                         io.query.data(), io.gate.data(), keys, values, stream.placed, config_.capacity, rows);
                if (st != TATARA_OK) break;
                st = tatara_attn_prefill(io.ctx, s, io.query.data(), io.gate.data(), keys, values, stream.placed, rows,
                                         config_.capacity, io.attended.data());
                branch_in = io.attended.data();
            } else {
                const std::uint64_t pin = 2ull * lane.stripe + (lane.slot->swapped[l] ? 1u : 0u);
                const std::uint64_t pout = 2ull * lane.stripe + (lane.slot->swapped[l] ? 0u : 1u);
                auto* conv = static_cast<std::uint16_t*>(pl.first.data());
                auto* rec = static_cast<float*>(pl.second.data());
                st = tatara_gdn_prepare(io.ctx, s, io.projection_slab.data(), conv + pin * pl.first_stride,
                                        layer.gated_delta.conv, io.qk.data(), io.value.data(), io.z.data(),
                                        conv + pout * pl.first_stride, rows);
                if (st != TATARA_OK) break;
                st = tatara_gdn_gates(io.ctx, s, io.projection_slab.data(), width, layer.gated_delta.a_log,
                                      layer.gated_delta.dt_bias, io.decay.data(), io.beta.data(), rows);
                if (st != TATARA_OK) break;
                st = tatara_gdn_prefill(io.ctx, s, io.qk.data(), io.value.data(), io.decay.data(), io.beta.data(),
                                        rec + pin * pl.second_stride, io.y.data(), rec + pout * pl.second_stride, rows, 64,
                                        io.scan_scratch.data(), io.scan_scratch.bytes());
                if (st != TATARA_OK) break;
                st = tatara_gdn_gate_norm(io.ctx, s, io.y.data(), io.z.data(), layer.gated_delta.norm, io.gated.data(), rows);
                branch_in = io.gated.data();
            }
            if (st != TATARA_OK) break;
            cudaEventRecord(io.marks[3 * l + 1], s);
            const rt::QuantizedWeight& ow = attention ? layer.attention_q4.out : layer.gated_delta_q4.out;
            if (layer.out_dense != nullptr) {
                st = tatara_project_dense(io.ctx, s, branch_in, rt::kAttnQueryValues, rows, layer.out_dense, rt::kHidden,
                                          rt::kAttnQueryValues, out, rt::kHidden);
            } else {
                const tatara_q4_matrix m[1] = {as_matrix(ow)};
                st = tatara_q4_project(io.ctx, s, branch_in, rt::kAttnQueryValues, rows, m, 1, rt::kAttnQueryValues, out,
                                       rt::kHidden);
            }
            cudaEventRecord(io.marks[3 * l + 2], s);
            cur ^= 1u;
        }
        return rt::to_command_error(st);
    }

    // One decode token for the group's rows.  Validation of the stream group happens here, before
    // anything is enqueued (decode_step.cpp:812-824); the work itself is the captured graph.
    rt::CommandError submit_token_batch(OwnerLaneGroup& group, const std::vector<Lane*>& rows) {
        const auto n = static_cast<std::uint32_t>(rows.size());
        if (n == 0 || n > config_.lanes_per_group) return rt::CommandError::InvalidStreamGroup;
        auto* attn = group.tables_host.as<tatara_attn_lane>();
        auto* gdn = reinterpret_cast<tatara_gdn_lane*>(group.tables_host.as<std::uint8_t>() + gdn_table_offset());
        for (std::uint32_t r = 0; r < n; ++r) {
            const Lane& lane = *rows[r];
            const rt::DecodeStateSlot& slot = *lane.slot;
            if (slot.status != rt::DecodeStateSlotStatus::Ready || slot.stripe >= group.pool.stripes)
                return rt::CommandError::StateSlotMismatch;
            if (!rt::context_in_capacity(lane.context, slot.capacity)) return rt::CommandError::ContextOutOfRange;
            std::uint64_t kv_stride = 0;
            for (std::size_t l = 0; l < layers_.size(); ++l) {
                const rt::DecodeStatePoolLayer& pl = group.pool.layers[l];
                if (pl.kind == rt::LayerKind::FullAttention) {
                    kv_stride = pl.first_stride;
                    continue;
                }
                const std::uint64_t in = 2ull * slot.stripe + (slot.swapped[l] ? 1u : 0u);
                const std::uint64_t out = 2ull * slot.stripe + (slot.swapped[l] ? 0u : 1u);
                gdn[std::uint64_t{gdn_index_[l]} * config_.lanes_per_group + r] = tatara_gdn_lane{
                    in * pl.first_stride, out * pl.first_stride, in * pl.second_stride, out * pl.second_stride};
            }
            attn[r] = tatara_attn_lane{std::uint64_t{slot.stripe} * kv_stride, lane.context, 0};
            boundary_.embed(lane.pending_input, lane.context,
                            group.rows_in_host.as<std::uint16_t>() + std::uint64_t{r} * rt::kHidden);
        }
        if (group.graphs[n] == nullptr) {
            const rt::CommandError e = capture_token_batch(group, n);
            if (e != rt::CommandError::None) return e;
        }
        if (cudaGraphLaunch(group.graphs[n], group.stream) != cudaSuccess) return rt::CommandError::CudaError;
        stats_.graph_launches += 1;
        return rt::CommandError::None;
    }

    rt::CommandError capture_token_batch(OwnerLaneGroup& group, std::uint32_t n) {
        if (cudaStreamBeginCapture(group.stream, cudaStreamCaptureModeRelaxed) != cudaSuccess)
            return rt::CommandError::CudaError;
        const rt::CommandError e = encode_token_batch(group, n);
        cudaGraph_t graph = nullptr;
        const cudaError_t ended = cudaStreamEndCapture(group.stream, &graph);
        if (e != rt::CommandError::None || ended != cudaSuccess || graph == nullptr) {
            if (graph != nullptr) cudaGraphDestroy(graph);
            (void)cudaGetLastError();
            return e != rt::CommandError::None ? e : rt::CommandError::CudaError;
        }
        cudaGraphExec_t exec = nullptr;
        const cudaError_t made = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (made != cudaSuccess) return rt::CommandError::CudaError;
        group.graphs[n] = exec;
        stats_.graphs_captured += 1;
        return rt::CommandError::None;
    }

    // encode_token_batch over this library's layers, every table read from device memory.
    rt::CommandError encode_token_batch(OwnerLaneGroup& group, std::uint32_t n) {
        cudaStream_t s = group.stream;
        if (cudaMemcpyAsync(group.tables.data(), group.tables_host.as<void>(), table_bytes(), cudaMemcpyHostToDevice, s) !=
                cudaSuccess ||
            cudaMemcpyAsync(group.hidden[0].data(), group.rows_in_host.as<void>(), n * kRowBytes, cudaMemcpyHostToDevice,
                            s) != cudaSuccess)
            return rt::CommandError::CudaError;
        const auto* attn = static_cast<const tatara_attn_lane*>(group.tables.data());
        const auto* gdn = reinterpret_cast<const tatara_gdn_lane*>(static_cast<const std::uint8_t*>(group.tables.data()) +
                                                                    gdn_table_offset());
        rt::DecodeBatchScratch& scratch = group.batch_scratch;
        std::uint32_t cur = 0;
        tatara_status st = TATARA_OK;
        for (std::size_t l = 0; l < layers_.size(); ++l) {
            const PathLayer& layer = layers_[l];
            rt::DecodeStatePoolLayer& pl = group.pool.layers[l];
            const void* in = group.hidden[cur].data();
            void* out = group.hidden[cur ^ 1u].data();
            const void* branch_in = nullptr;
            const rt::QuantizedWeight* ow = nullptr;
            if (layer.kind == rt::LayerKind::FullAttention) {
                const tatara_q4_matrix m[3] = {as_matrix(layer.attention_q4.query), as_matrix(layer.attention_q4.key),
                                               as_matrix(layer.attention_q4.value)};
                st = tatara_q4_project(group.ctx, s, in, rt::kHidden, n, m, 3, rt::kHidden, group.projection_slab.data(),
                                       rt::kAttnProjectionRows);
                if (st != TATARA_OK) break;
                st = tatara_attn_qk_rope_batch_indirect(group.ctx, s, group.projection_slab.data(), layer.attention.q_norm,
                                                        layer.attention.k_norm, scratch.query.data(), scratch.gate.data(),
                                                        pl.first.data(), pl.second.data(), config_.capacity, attn, n,
                                                        rt::kAttnProjectionRows, rt::kAttnQueryValues);
                if (st != TATARA_OK) break;
                st = tatara_attn_decode_batch_indirect(group.ctx, s, scratch.query.data(), scratch.gate.data(),
                                                       pl.first.data(), pl.second.data(), attn, n, config_.capacity,
                                                       rt::kAttnQueryValues, scratch.attended.data(), scratch.records.data(),
                                                       scratch.records.bytes());
                branch_in = scratch.attended.data();
                ow = &layer.attention_q4.out;
            } else {
                const tatara_q4_matrix m[4] = {as_matrix(layer.gated_delta_q4.qkv), as_matrix(layer.gated_delta_q4.z),
                                               as_matrix(layer.gated_delta_q4.b), as_matrix(layer.gated_delta_q4.a)};
                st = tatara_q4_project(group.ctx, s, in, rt::kHidden, n, m, 4, rt::kHidden, group.projection_slab.data(),
                                       rt::kGdnProjectionRows);
                if (st != TATARA_OK) break;
                st = tatara_gdn_decode_batch_indirect(
                    group.ctx, s, group.projection_slab.data(), rt::kGdnProjectionRows, layer.gated_delta.conv,
                    layer.gated_delta.a_log, layer.gated_delta.dt_bias, layer.gated_delta.norm, pl.first.data(),
                    pl.second.data(), gdn + std::uint64_t{gdn_index_[l]} * config_.lanes_per_group, n, scratch.gdn_y.data(),
                    scratch.gdn_gated.data());
                branch_in = scratch.gdn_gated.data();
                ow = &layer.gated_delta_q4.out;
            }
            if (st != TATARA_OK) break;
            const tatara_q4_matrix m[1] = {as_matrix(*ow)};
            st = tatara_q4_project(group.ctx, s, branch_in, rt::kAttnQueryValues, n, m, 1, rt::kAttnQueryValues, out,
                                   rt::kHidden);
            if (st != TATARA_OK) break;
            cur ^= 1u;
        }
        if (st != TATARA_OK) return rt::to_command_error(st);
        if (cudaMemcpyAsync(group.rows_out_host.as<void>(), group.hidden[cur].data(), n * kRowBytes, cudaMemcpyDeviceToHost,
                            s) != cudaSuccess)
            return rt::CommandError::CudaError;
        return rt::CommandError::None;
    }

    void settle(OwnerLaneGroup& group, Lane& lane, std::uint32_t token) {
        const rt::DecodeStream one{lane.slot, lane.context};
        rt::advance_decode_state(group.pool, {one});
        ++lane.context;
        ++lane.produced;
        push_token(lane, token);
        const bool stop_hit =
            std::find(lane.request.stop_ids.begin(), lane.request.stop_ids.end(), token) != lane.request.stop_ids.end();
        if (stop_hit) {
            finish(lane, LaneDoneReason::Stopped);
        } else if (lane.produced >= lane.request.maximum_tokens) {
            finish(lane, LaneDoneReason::Length);
        } else if (lane.context >= config_.capacity) {
            finish(lane, LaneDoneReason::Length);   // the cache is full: the next position does not exist
        } else {
            lane.pending_input = token;
        }
    }

    OwnerConfig config_;
    std::vector<PathLayer> layers_;
    TokenBoundary boundary_;
    bool ok_{false};
    std::vector<std::uint32_t> gdn_index_;
    std::uint32_t gdn_layers_{0};
    std::vector<OwnerLaneGroup> groups_;
    std::vector<Lane> lanes_;
    std::vector<JoiningLane> joining_;
    tatara_ctx* join_ctx_{nullptr};
    cudaStream_t stream_{nullptr};   // every submission of the owner
    std::vector<Lane*> wave_;
    std::vector<std::vector<Lane*>> plans_;
    std::vector<bool> submitted_;
    WaveStatistics stats_;
    rt::CommandError last_error_{rt::CommandError::None};

    std::mutex queue_mutex_;
    std::condition_variable queue_ready_;
    std::deque<OwnerSubmission> queue_;
    std::uint64_t outstanding_{0};
    bool running_{true};
};

} // namespace tatara::engine
