// Split-KV decode attention for the gated GQA layers (reference semantics:
// attention.metal:200-276 single kernel, :373-1108 partitioned families + combine).
//
// Two kernels:
//   1. attn_decode_partition_kernel -- persistent CTAs walk work items (lane, kv head,
//      key partition).  One K/V read serves all 8 query heads of the GQA group: scores and
//      P.V are mma.sync m16n8k16 tiles with the 8 heads in the M dimension.  Each warp owns a
//      private cp.async ring of 16-key K and V slices (16-byte coalesced loads, XOR-swizzled
//      rows, ldmatrix reads) that runs ahead across item boundaries, so HBM stays busy while
//      a finished item is merged and its 258-float records are written.
//   2. attn_combine_kernel -- log-sum-exp merge of a lane's records, normalisation and the
//      sigmoid output gate (or, for split-KV across GPUs, one merged un-normalised record).
//
// Lossless concurrency: the partition size is a function of the lane's own key count only
// (tb::partition_keys), every record is computed by one warp-order-fixed procedure and the
// combine walks records in index order, so a lane's output bits do not depend on which other
// lanes share the launch or on which CTA ran which item.
#include "common.cuh"

#include <cstring>
#include <mutex>

namespace tb {

constexpr uint32_t kDecWarps = 4;
constexpr uint32_t kDecThreads = kDecWarps * 32;
constexpr uint32_t kDecStages = 3;
constexpr uint32_t kSliceKeys = 16;
constexpr uint32_t kRowBytes = kHeadDim * 2;                 // 512
constexpr uint32_t kSliceBytes = kSliceKeys * kRowBytes;     // 8 KiB per plane
constexpr uint32_t kStageBytes = 2 * kSliceBytes;            // K then V
constexpr uint32_t kRingBytes = kDecStages * kStageBytes;    // per warp
constexpr uint32_t kMergeStride = kHeadDim + 4u;   // floats per (warp, head) row of the merge buffer: the padding spreads the heads over the banks
constexpr uint32_t kMergeFloats = kDecWarps * kHeadsPerKv * kMergeStride;
constexpr uint32_t kDecSmemBytes = kDecWarps * kRingBytes + kMergeFloats * 4 +
                                   kDecWarps * kHeadsPerKv * 2 * 4 + (TATARA_MAX_LANES + 1) * 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecLane {
    uint64_t kv_offset;  // elements into the K / V pools
    uint64_t rec_offset; // floats into the record scratch
    uint32_t key_begin, key_end;
    uint32_t part_keys, nparts;
    uint32_t item_start; // first work item of this lane
    uint32_t row;        // q / gate / out row
};

struct DecTables;   // the same tables in device memory (lane tables that a CUDA graph can replay)
template <uint32_t N>
struct DecParams {
    const DecTables* tables;   // null: the tables below, built on the host for this call
    const __nv_bfloat16* q;
    const __nv_bfloat16* keys;
    const __nv_bfloat16* values;
    float* records;
    uint64_t query_stride;
    uint32_t capacity;
    uint32_t n_lanes;
    uint32_t total_items;
    uint32_t l2_prefetch_keys; // K/V rows of a CTA's first item requested into L2 before the dependency wait
    // Merge in the same launch (single lane, gated output): the CTAs count their finished items in
    // merge_counters[0] and leave through merge_counters[1]; null = the merge is a second kernel.
    uint32_t* merge_counters;
    uint32_t* merge_status;
    const __nv_bfloat16* gate;
    __nv_bfloat16* out;
    DecLane lane[N];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// K / V rows are read once per token: they are marked evict-first in L2 so that the stream does
// not push out what the step re-reads (q, gate, the partial records).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes), "l"(policy)
                 : "memory");
}
// Asks for `bytes` (a multiple of 16, from a 16-byte aligned address) to be brought into L2; nothing
// is written to shared memory or registers, so the request may precede the dependency wait even for
// rows the predecessor is still writing (L2 is the point of coherence: a later store updates the line).
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8) = A(16x16) * B(16x8) + C with rows 8..15 of A zero: only rows 0..7 are kept.
__device__ __forceinline__ void mma_top_rows(float& d0, float& d1, uint32_t a0, uint32_t a2,
                                             uint32_t b0, uint32_t b1) {
    float z0, z1;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%10,%10};\n"
        : "+f"(d0), "+f"(d1), "=f"(z0), "=f"(z1)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.0f));
}
// D(16x8) += A(16x16) * B(16x8), bf16 in, f32 accumulate.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Transposes an 8x8 matrix of 16-bit elements held one row per four lanes (lane 4g + t: row g, columns 2t, 2t+1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Position of one warp in its stream of 16-key slices.
struct SliceCursor {
    uint32_t item, slice, nkeys, lane, kv, part;
    const uint8_t* kbase;
    const uint8_t* vbase;
    bool valid;
};

__device__ const DecLane& table_lane(const DecTables* t, uint32_t i);
__device__ uint32_t tables_n_lanes(const DecTables* t);
__device__ uint32_t tables_total_items(const DecTables* t);
// The schedule a kernel works from: the by-value tables of its parameters (kInd = false, the
// host built them for this call) or their copy in device memory (kInd = true).
template <uint32_t N, bool kInd>
__device__ __forceinline__ const DecLane& lane_at(const DecParams<N>& p, uint32_t i) {
    if constexpr (kInd) return table_lane(p.tables, i);
    else return p.lane[i];
}
template <uint32_t N, bool kInd>
__device__ __forceinline__ uint32_t lanes_in(const DecParams<N>& p) {
    if constexpr (kInd) return tables_n_lanes(p.tables);
    else return p.n_lanes;
}
template <uint32_t N, bool kInd>
__device__ __forceinline__ uint32_t items_in(const DecParams<N>& p) {
    if constexpr (kInd) return tables_total_items(p.tables);
    else return p.total_items;
}
template <uint32_t N, bool kInd>
__device__ __forceinline__ void cursor_load_item(SliceCursor& c, const DecParams<N>& p,
                                                 const uint32_t* item_start) {
    uint32_t lo = 0, hi = lanes_in<N, kInd>(p); // last lane with item_start <= item
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (item_start[mid] <= c.item) lo = mid; else hi = mid;
    }
    const DecLane& l = lane_at<N, kInd>(p, lo);
    const uint32_t local = c.item - l.item_start;
    c.lane = lo;
    c.part = local >> 1;
    c.kv = local & 1u;
    const uint32_t begin = l.key_begin + c.part * l.part_keys;
    const uint32_t end = min(l.key_end, begin + l.part_keys);
    c.nkeys = end - begin;
    const uint64_t first = (l.kv_offset + (uint64_t(c.kv) * p.capacity + begin) * kHeadDim) * 2ull;
    c.kbase = reinterpret_cast<const uint8_t*>(p.keys) + first;
    c.vbase = reinterpret_cast<const uint8_t*>(p.values) + first;
}

template <uint32_t N, bool kInd>
__device__ __forceinline__ void cursor_settle(SliceCursor& c, const DecParams<N>& p,
                                              const uint32_t* item_start, uint32_t warp) {
    while (c.valid && c.slice * kSliceKeys >= c.nkeys) {
        c.item += gridDim.x;
        if (c.item >= items_in<N, kInd>(p)) {
            c.valid = false;
            break;
        }
        cursor_load_item<N, kInd>(c, p, item_start);
        c.slice = warp;
    }
}

// Issues the 16-key K and V slice under the cursor into one ring stage (rows past the
// partition end are zero-filled), 32 x 16-byte cp.async per lane.
__device__ __forceinline__ void issue_slice(const SliceCursor& c, uint32_t stage_addr, uint32_t lane, uint64_t policy) {
    const uint32_t first = c.slice * kSliceKeys;
    const uint32_t rows = min(kSliceKeys, c.nkeys - first);
    const uint8_t* ksrc = c.kbase + uint64_t(first) * kRowBytes + lane * 16u;
    const uint8_t* vsrc = c.vbase + uint64_t(first) * kRowBytes + lane * 16u;
#pragma unroll
    for (uint32_t row = 0; row < kSliceKeys; ++row) {
        const bool live = row < rows;
        const uint32_t off = live ? row * kRowBytes : 0u;
        const uint32_t dst = stage_addr + row * kRowBytes + ((lane ^ (row & 7u)) << 4);
        cp_async_16(dst, ksrc + off, live ? 16u : 0u, policy);
        cp_async_16(dst + kSliceBytes, vsrc + off, live ? 16u : 0u, policy);
    }
}

// One CTA per (head, 64-dim quarter, lane).  The merge is defined over 32 phases: phase f sums
// records f, f+32, ... in index order (four in flight per thread), a thread owns a float2 of the
// quarter; then the 32 phase partials are summed in phase order.  Every order is fixed by nparts
// alone, whatever the CTA size: a single lane runs one phase per warp (32 warps, lowest
// latency), a batch runs four phases per warp (8 warps, many small CTAs per SM), the partition
// kernel's own tail eight (4 warps).
constexpr uint32_t kCombinePhases = 32, kCombineDims = 64, kCombineUnroll = 4;

// The merge of one (head, quarter): records `base + part * part_stride`, part < nparts.  Leaves the
// 64 un-normalised sums in red_acc[0][0..63], the sum of weights in red_acc[0][64] and returns the
// maximum; ends with a CTA barrier.  Called by every thread of a CTA of kWarps warps.
template <uint32_t kWarps>
__device__ __forceinline__ float merge_records(const float* base, uint64_t part_stride, uint32_t nparts,
                                               uint32_t quarter, float* red_max,
                                               float (*red_acc)[kCombineDims + 1]) {
    constexpr uint32_t kCombineThreads = kWarps * 32u;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t d = quarter * kCombineDims + lane * 2u;
    constexpr uint32_t kOwn = kCombinePhases / kWarps, kRound = kCombinePhases * kCombineUnroll;
    // The first round of records (parts 0..127: every record of a lane cut by tb::partition_keys)
    // is requested before the maximum is known, so the merge costs one trip to L2, not two.
    // (ld.global.cg: the records were written by other CTAs, possibly of this same launch)
    float lm[kOwn][kCombineUnroll], ls[kOwn][kCombineUnroll];
    float2 v[kOwn][kCombineUnroll];
    auto load_round = [&](uint32_t round) {
#pragma unroll
        for (uint32_t j = 0; j < kOwn; ++j) {
#pragma unroll
            for (uint32_t u = 0; u < kCombineUnroll; ++u) {
                const uint32_t part = round + (warp + j * kWarps) + u * kCombinePhases;
                const bool live = part < nparts;
                const float* rec = base + (live ? part : 0u) * part_stride;
                lm[j][u] = live ? __ldcg(rec + kHeadDim) : -INFINITY;
                ls[j][u] = __ldcg(rec + kHeadDim + 1u);
                v[j][u] = __ldcg(reinterpret_cast<const float2*>(rec + d));
            }
        }
    };
    load_round(0);
    float big = -INFINITY;
#pragma unroll
    for (uint32_t j = 0; j < kOwn; ++j)
#pragma unroll
        for (uint32_t u = 0; u < kCombineUnroll; ++u) big = fmaxf(big, lm[j][u]);
    for (uint32_t part = kRound + threadIdx.x; part < nparts; part += kCombineThreads)
        big = fmaxf(big, __ldcg(base + part * part_stride + kHeadDim));
#pragma unroll
    for (int off = 16; off; off >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
    if (lane == 0) red_max[warp] = big;
    __syncthreads();
    big = red_max[0];
#pragma unroll
    for (uint32_t i = 1; i < kWarps; ++i) big = fmaxf(big, red_max[i]);

    // One accumulator set per phase this warp owns.
    float a0[kOwn], a1[kOwn], denom[kOwn];
#pragma unroll
    for (uint32_t j = 0; j < kOwn; ++j) a0[j] = a1[j] = denom[j] = 0.0f;
    for (uint32_t round = 0; round < nparts; round += kRound) {
        if (round != 0) load_round(round);
#pragma unroll
        for (uint32_t j = 0; j < kOwn; ++j) {
#pragma unroll
            for (uint32_t u = 0; u < kCombineUnroll; ++u) {
                const float w = lm[j][u] == -INFINITY ? 0.0f : expf(lm[j][u] - big);
                a0[j] = fmaf(w, v[j][u].x, a0[j]);
                a1[j] = fmaf(w, v[j][u].y, a1[j]);
                denom[j] = fmaf(w, ls[j][u], denom[j]);
            }
        }
    }
#pragma unroll
    for (uint32_t j = 0; j < kOwn; ++j) {
        const uint32_t phase = warp + j * kWarps;
        red_acc[phase][lane * 2u] = a0[j];
        red_acc[phase][lane * 2u + 1u] = a1[j];
        if (lane == 0) red_acc[phase][kCombineDims] = denom[j];
    }
    __syncthreads();
    if (threadIdx.x < kCombineDims + 1u) {
        float total = 0.0f;
#pragma unroll
        for (uint32_t ph = 0; ph < kCombinePhases; ++ph) total += red_acc[ph][threadIdx.x];
        red_acc[0][threadIdx.x] = total;
    }
    __syncthreads();
    return big;
}

// The merge in the partition kernel's own launch (one lane, gated output).  Every CTA adds the items it
// has finished to merge_counters[0] (its record stores made visible first); CTA c then takes the
// (head, quarter) pieces c, c + grid, ... of the 64: waits, with a time limit, until the counter has
// reached the lane's item count, merges with the arithmetic of attn_combine_kernel (merge_records,
// eight phases per warp) and stores the gated output.  All CTAs of the grid are resident together
// (at most one per SM, and the grid is never larger than the SM count), so the wait is for CTAs that
// are running.  The last CTA to leave puts both counters back to zero for the next launch.  The
// scratch the merge needs lies over the first warp's K/V ring, which is dead by then.
constexpr unsigned long long kMergeWaitLimitNs = 2000000000ull;
template <uint32_t N>
__device__ __forceinline__ void fused_merge_tail(const DecParams<N>& p, uint8_t* smem, uint32_t total_items) {
    __syncthreads();   // every record of this CTA's items is written, every ring slot is idle
    float* red_max = reinterpret_cast<float*>(smem);
    float (*red_acc)[kCombineDims + 1] = reinterpret_cast<float (*)[kCombineDims + 1]>(smem + 128);
    volatile uint32_t* arrived = reinterpret_cast<volatile uint32_t*>(smem + 128 + kCombinePhases * (kCombineDims + 1) * 4);
    if (threadIdx.x == 0) {
        const uint32_t mine = blockIdx.x < total_items ? (total_items - 1u - blockIdx.x) / gridDim.x + 1u : 0u;
        if (mine != 0u) {
            __threadfence();
            atomicAdd(p.merge_counters, mine);
        }
    }
    const DecLane& dl = p.lane[0];
    for (uint32_t piece = blockIdx.x; piece < kQHeads * 4u; piece += gridDim.x) {
        const uint32_t head = piece >> 2, quarter = piece & 3u;
        const uint64_t at = dl.row * p.query_stride + head * kHeadDim + quarter * kCombineDims + threadIdx.x;
        float gate_logit = 0.0f;
        if (threadIdx.x < kCombineDims) gate_logit = bf2f(p.gate[at]);
        if (threadIdx.x == 0) {
            unsigned long long t0 = 0;
            uint32_t ok = 1u;
            for (uint32_t spin = 0;; ++spin) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.merge_counters) : "memory");
                if (v >= total_items) break;
                __nanosleep(20);
                if ((spin & 255u) == 255u) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                    if (t0 == 0) t0 = now;
                    if (now - t0 > kMergeWaitLimitNs) {
                        ok = 0u;
                        atomicCAS(p.merge_status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
                        p.merge_status[kStatusDetail] = blockIdx.x;
                        break;
                    }
                }
            }
            *arrived = ok;
        }
        __syncthreads();
        if (*arrived == 0u) break;   // nothing more is written by this CTA
        const float* base = p.records + dl.rec_offset + uint64_t(head) * dl.nparts * kRecordFloats;
        (void)merge_records<kDecWarps>(base, kRecordFloats, dl.nparts, quarter, red_max, red_acc);
        if (threadIdx.x < kCombineDims) {
            const float acc = red_acc[0][threadIdx.x], total = red_acc[0][kCombineDims];
            p.out[at] = f2bf((acc / total) * (1.0f / (1.0f + expf(-gate_logit))));
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (atomicAdd(p.merge_counters + 1, 1u) == gridDim.x - 1u) {   // nobody reads the counters any more
            p.merge_counters[0] = 0u;
            p.merge_counters[1] = 0u;
        }
    }
}

template <uint32_t N, bool kInd = false>
__global__ void __launch_bounds__(kDecThreads, 1)
attn_decode_partition_kernel(const __grid_constant__ DecParams<N> p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    float* merge_o = reinterpret_cast<float*>(smem + kDecWarps * kRingBytes);
    float* merge_ml = merge_o + kMergeFloats;
    uint32_t* item_start = reinterpret_cast<uint32_t*>(merge_ml + kDecWarps * kHeadsPerKv * 2);
    // (a device copy of the tables is written by a setup kernel that precedes this one in plain stream order)
    const uint32_t n_lanes = lanes_in<N, kInd>(p), total_items = items_in<N, kInd>(p);
    for (uint32_t i = threadIdx.x; i <= n_lanes; i += kDecThreads)
        item_start[i] = i < n_lanes ? lane_at<N, kInd>(p, i).item_start : total_items;
    __syncthreads();
    const uint32_t ring = smem_u32(smem + warp * kRingBytes);
    const uint64_t stream_policy = l2_evict_first_policy();

    // Producer cursor: runs kDecStages-1 slices ahead of the consumer, across items.
    SliceCursor pc{};
    pc.item = blockIdx.x;
    pc.valid = pc.item < total_items;
    bool early = false;
    if (pc.valid) {
        cursor_load_item<N, kInd>(pc, p, item_start);
        pc.slice = warp;
        // Every partition but a lane's last is full (at least 128 keys = 2 slices for each warp) and
        // holds only keys written before this token, so its first slices can be requested at once.
        early = pc.part + 1u < lane_at<N, kInd>(p, pc.lane).nparts;
        // The ring holds (kDecStages - 1) slices per warp before the dependency wait; the rows after
        // those are asked into L2 now, so that the K/V stream out of HBM keeps running while this CTA
        // waits for its predecessor and for q (one 16-row request of each plane per thread and pass).
        // Only when every CTA has a single item: a batch with several items per CTA keeps HBM busy
        // across items by itself, and the extra lines only compete for L2 (measured: 32 lanes 1.5 % slower).
        if (p.l2_prefetch_keys != 0u && total_items <= gridDim.x) {
            // (a quarter of the item, capped: measured best at 128 rows of a 443-key item, 256 of 886, 384-512 of
            // 3543 -- more only competes in L2 with the step that is still streaming)
            const uint32_t ring_keys = early ? kDecWarps * (kDecStages - 1u) * kSliceKeys : 0u;
            const uint32_t window = min(p.l2_prefetch_keys, ((pc.nkeys >> 2) + 15u) & ~15u);
            const uint32_t stop = min(pc.nkeys, ring_keys + window);
            for (uint32_t row = ring_keys + threadIdx.x * kSliceKeys; row < stop; row += kDecThreads * kSliceKeys) {
                const uint32_t bytes = min(kSliceKeys, stop - row) * kRowBytes;
                l2_prefetch_bulk(pc.kbase + uint64_t(row) * kRowBytes, bytes);
                l2_prefetch_bulk(pc.vbase + uint64_t(row) * kRowBytes, bytes);
            }
        }
        cursor_settle<N, kInd>(pc, p, item_start, warp);
    }
    uint32_t issued = 0, consumed = 0;
    auto fill_ring = [&]() {
#pragma unroll
        for (uint32_t i = 0; i + 1 < kDecStages; ++i) {
            if (pc.valid) {
                issue_slice(pc, ring + (issued % kDecStages) * kStageBytes, lane, stream_policy);
                pc.slice += kDecWarps;
                cursor_settle<N, kInd>(pc, p, item_start, warp);
            }
            cp_async_commit();
            ++issued;
        }
    };
    // Launched with programmatic stream serialization: everything above, and the first K/V slices
    // of partitions that cannot contain the row the predecessor appends, overlap the tail of the
    // previous kernel in the stream.  q, the appended row and the record scratch are touched only
    // after griddepcontrol.wait (the predecessor has completed and its writes are visible).
    if (early) fill_ring();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Let a programmatic dependent (the combine) be staged; it still waits for this grid to finish.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!early) fill_ring();

    // Scores and P.V run TRANSPOSED, so that every row of the 16-row MMA tile carries data (with the
    // 8 heads in M half of each MMA multiplied zeros):
    //     S^T [16 keys x 8 heads]  = K [16 keys x 256] . Q^T       A = K slice (ldmatrix), B = Q (registers)
    //     O^T [256 dims x 8 heads] += V^T [dims x 16 keys] . P^T    A = V slice (ldmatrix.trans), B = P^T
    // The accumulator of S^T holds (key g | g+8, heads 2t, 2t+1) per lane; P^T as a B operand wants
    // (keys 2t, 2t+1 | +8, head g): one movmatrix per 8 keys transposes the packed probabilities.
    // Per-lane ldmatrix address pieces (fragment layouts of mma.m16n8k16: A = 4 matrices ordered
    // (rows lo, cols lo), (rows hi, cols lo), (rows lo, cols hi), (rows hi, cols hi)).
    const uint32_t lm_j = lane >> 3, lm_r = lane & 7u;
    const uint32_t k_row_off = ((lm_j & 1u) * 8u + lm_r) * kRowBytes;   // K: rows = keys, cols = dims
    const uint32_t k_chunk_lo = lm_j >> 1;
    const uint32_t v_row_off = ((lm_j >> 1) * 8u + lm_r) * kRowBytes;   // V^T: rows = dims (j & 1), cols = keys (j >> 1)
    const uint32_t v_chunk_lo = lm_j & 1u;
    const float score_scale = kAttnScale * kLog2e;

    SliceCursor cc{};
    for (cc.item = blockIdx.x; cc.item < total_items; cc.item += gridDim.x) {
        cursor_load_item<N, kInd>(cc, p, item_start);
        const DecLane& dl = lane_at<N, kInd>(p, cc.lane);
        // Q of head (kv*8 + g) as the B operand of every k-step: dims 16ks + 2t, +1 | + 8, + 9.
        uint32_t qa[16][2];
        {
            const __nv_bfloat16* qrow =
                p.q + dl.row * p.query_stride + (cc.kv * kHeadsPerKv + g) * kHeadDim;
#pragma unroll
            for (uint32_t ks = 0; ks < 16; ++ks) {
                qa[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16u + 2u * t);
                qa[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16u + 8u + 2u * t);
            }
        }
        // O^T: tile nt = dims 16nt .. +15; o[nt] = (dim g, head 2t), (dim g, head 2t+1), (dim g+8, 2t), (dim g+8, 2t+1)
        float o[16][4];
#pragma unroll
        for (uint32_t nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // heads 2t and 2t+1

        for (uint32_t slice = warp; slice * kSliceKeys < cc.nkeys; slice += kDecWarps) {
            // keep the ring full, then wait for the oldest slice
            if (pc.valid) {
                issue_slice(pc, ring + (issued % kDecStages) * kStageBytes, lane, stream_policy);
                pc.slice += kDecWarps;
                cursor_settle<N, kInd>(pc, p, item_start, warp);
            }
            cp_async_commit();
            ++issued;
            cp_async_wait<kDecStages - 1>();
            __syncwarp();
            const uint32_t kst = ring + (consumed % kDecStages) * kStageBytes;
            const uint32_t vst = kst + kSliceBytes;

            float sa[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // two chains over the 16 k-steps
#pragma unroll
            for (uint32_t ks = 0; ks < 16; ks += 2) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(kst + k_row_off + (((ks * 2u + k_chunk_lo) ^ lm_r) << 4), a0, a1, a2, a3);
                mma_16816(sa, a0, a1, a2, a3, qa[ks][0], qa[ks][1]);
                ldmatrix_x4(kst + k_row_off + ((((ks + 1u) * 2u + k_chunk_lo) ^ lm_r) << 4), a0, a1, a2, a3);
                mma_16816(sb, a0, a1, a2, a3, qa[ks + 1][0], qa[ks + 1][1]);
            }
            // lane (g, t): keys g and g + 8 of the slice, heads 2t and 2t + 1
            const uint32_t key0 = slice * kSliceKeys + g;
            const bool live0 = key0 < cc.nkeys, live1 = key0 + 8u < cc.nkeys;
            const float s00 = live0 ? (sa[0] + sb[0]) * score_scale : -INFINITY;   // key g,   head 2t
            const float s01 = live0 ? (sa[1] + sb[1]) * score_scale : -INFINITY;   // key g,   head 2t+1
            const float s10 = live1 ? (sa[2] + sb[2]) * score_scale : -INFINITY;   // key g+8, head 2t
            const float s11 = live1 ? (sa[3] + sb[3]) * score_scale : -INFINITY;   // key g+8, head 2t+1
            float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
            for (uint32_t off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);   // finite: key 0 of every slice is live
            const float alpha0 = exp2f(m0 - n0), alpha1 = exp2f(m1 - n1);
            const float p00 = exp2f(s00 - n0), p01 = exp2f(s01 - n1), p10 = exp2f(s10 - n0), p11 = exp2f(s11 - n1);
            l0 = l0 * alpha0 + (p00 + p10);
            l1 = l1 * alpha1 + (p01 + p11);
            m0 = n0;
            m1 = n1;
            const uint32_t pb0 = movmatrix_trans(pack_bf16x2(p00, p01));   // keys 2t, 2t+1 of head g
            const uint32_t pb1 = movmatrix_trans(pack_bf16x2(p10, p11));   // keys 2t+8, 2t+9 of head g
            // a factor of exactly 1 leaves every bit as it is, so the rescale is skipped when no lane needs it
            const bool rescale = __any_sync(0xffffffffu, alpha0 != 1.0f || alpha1 != 1.0f);
#pragma unroll
            for (uint32_t nt = 0; nt < 16; ++nt) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4_trans(vst + v_row_off + (((nt * 2u + v_chunk_lo) ^ lm_r) << 4), a0, a1, a2, a3);
                if (rescale) {
                    o[nt][0] *= alpha0;
                    o[nt][1] *= alpha1;
                    o[nt][2] *= alpha0;
                    o[nt][3] *= alpha1;
                }
                mma_16816(o[nt], a0, a1, a2, a3, pb0, pb1);
            }
            __syncwarp(); // every lane is done with this stage before it is refilled
            ++consumed;
        }

        // ---- merge the four warps of this item and write its 8 records --------------------
#pragma unroll
        for (uint32_t off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
        }
        {
            float* mo0 = merge_o + (warp * kHeadsPerKv + 2u * t) * kMergeStride + g;
            float* mo1 = mo0 + kMergeStride;
#pragma unroll
            for (uint32_t nt = 0; nt < 16; ++nt) {
                mo0[nt * 16u] = o[nt][0];
                mo1[nt * 16u] = o[nt][1];
                mo0[nt * 16u + 8u] = o[nt][2];
                mo1[nt * 16u + 8u] = o[nt][3];
            }
        }
        if (g == 0) {
            merge_ml[(warp * kHeadsPerKv + 2u * t) * 2u] = m0;
            merge_ml[(warp * kHeadsPerKv + 2u * t) * 2u + 1u] = l0;
            merge_ml[(warp * kHeadsPerKv + 2u * t + 1u) * 2u] = m1;
            merge_ml[(warp * kHeadsPerKv + 2u * t + 1u) * 2u + 1u] = l1;
        }
        __syncthreads();
        {
            const uint32_t h = threadIdx.x >> 4, d0 = (threadIdx.x & 15u) * 16u;
            float mw[kDecWarps], big = -INFINITY;
#pragma unroll
            for (uint32_t w = 0; w < kDecWarps; ++w) {
                mw[w] = merge_ml[(w * kHeadsPerKv + h) * 2u];
                big = fmaxf(big, mw[w]);
            }
            float acc[16], lsum = 0.0f;
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) acc[i] = 0.0f;
#pragma unroll
            for (uint32_t w = 0; w < kDecWarps; ++w) {
                const float wt = mw[w] == -INFINITY ? 0.0f : exp2f(mw[w] - big);
                lsum = fmaf(wt, merge_ml[(w * kHeadsPerKv + h) * 2u + 1u], lsum);
                const float4* src =
                    reinterpret_cast<const float4*>(merge_o + (w * kHeadsPerKv + h) * kMergeStride + d0);
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const float4 v = src[i];
                    acc[4 * i] = fmaf(wt, v.x, acc[4 * i]);
                    acc[4 * i + 1] = fmaf(wt, v.y, acc[4 * i + 1]);
                    acc[4 * i + 2] = fmaf(wt, v.z, acc[4 * i + 2]);
                    acc[4 * i + 3] = fmaf(wt, v.w, acc[4 * i + 3]);
                }
            }
            float* rec = p.records + dl.rec_offset +
                         (uint64_t(cc.kv * kHeadsPerKv + h) * dl.nparts + cc.part) * kRecordFloats;
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i)
                *reinterpret_cast<float2*>(rec + d0 + 2u * i) = make_float2(acc[2 * i], acc[2 * i + 1]);
            if ((threadIdx.x & 15u) == 0u) {
                rec[kHeadDim] = big * kLn2; // stored in natural-log units, as the reference record
                rec[kHeadDim + 1u] = lsum;
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if constexpr (N == 1 && !kInd) {
        if (p.merge_counters != nullptr) fused_merge_tail<N>(p, smem, total_items);
    }
}

// ---- combine ---------------------------------------------------------------------------
struct CombineLane {
    const float* records; // record (h, p) at records + h*head_stride + p*part_stride
    uint64_t head_stride, part_stride;
    uint32_t nparts;
    uint32_t row;
};
// Both kernels' lane tables in device memory, written by attn_decode_setup_kernel from a lane
// table that itself lives in device memory: nothing about a token's contexts is a kernel
// argument, so one captured CUDA graph serves every token.
struct DecTables {
    uint32_t n_lanes, total_items, pad0, pad1;
    DecLane dec[TATARA_MAX_LANES];
    CombineLane comb[TATARA_MAX_LANES];
};
static_assert(sizeof(DecTables) <= kLaneScheduleBytes, "lane schedule buffer");
__device__ __forceinline__ const DecLane& table_lane(const DecTables* t, uint32_t i) { return t->dec[i]; }
__device__ __forceinline__ uint32_t tables_n_lanes(const DecTables* t) { return t->n_lanes; }
__device__ __forceinline__ uint32_t tables_total_items(const DecTables* t) { return t->total_items; }
constexpr uint32_t kMaxPeers = 8;
constexpr uint32_t kCombineDimsPerCta = 64;
// Peer exchange of the split-KV merge (one process per GPU, buffers mapped through CUDA IPC).
struct PeerExchange {
    float* peer_out[kMaxPeers];      // push: slot [rank] of every rank's gather buffer ([16][258] f32)
    uint32_t* peer_flag[kMaxPeers];  // push: word [rank] of every rank's flag array
    const uint32_t* wait_flags;      // wait: this rank's flag array, or null
    uint32_t* done_counter;          // local counter of finished CTAs (self-resetting)
    uint32_t* status;                // device status word of the context
    // Step counter in this rank's own memory, or null.  With a counter the epoch of a call is
    // counter + 1, the pointers above address parity 0 and the parity in use is epoch & 1 (the strides
    // below lead to parity 1); the waiting merge advances the counter when its last CTA is done.  So a
    // step has no host-side argument that changes from token to token, and a captured graph replays.
    uint32_t* step;
    uint32_t out_parity_floats, flag_parity_words;
    uint32_t world, epoch, wait_limit_us;
    // Single-kernel exchange (tatara_attn_decode_split): every rank's buffer of 8-byte words
    // {f32 value, u32 epoch}, [2 parities][source rank][16 heads][4 quarters][kExchangeWords]; a word is
    // stored whole, so a reader that sees this step's epoch in the upper half holds the value too and
    // no fence or separate flag is needed.  ll[r] == null outside that call.
    unsigned long long* ll[kMaxPeers];
    uint32_t ll_rank;
};
constexpr uint32_t kExchangeWords = kCombineDimsPerCta + 2u;   // a quarter of the numerator, max, sum
__device__ __forceinline__ uint32_t exchange_epoch(const PeerExchange& px) {
    if (px.step == nullptr) return px.epoch;
    uint32_t done;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(done) : "l"(px.step) : "memory");
    return done + 1u;
}
template <uint32_t N>
struct CombineParams {
    const DecTables* tables;   // null: the lane table below
    const __nv_bfloat16* gate;
    __nv_bfloat16* out;  // [row][16][256] gated output, or null
    float* record_out;   // [lane][16][258] merged un-normalised record, or null
    uint64_t query_stride;
    PeerExchange px;     // all null / zero outside the multi-GPU split-KV calls
    CombineLane lane[N];
};
__device__ __forceinline__ unsigned long long combine_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

template <uint32_t N>
constexpr uint32_t combine_warps() { return N == 1 ? 32u : 8u; }

template <uint32_t N, bool kInd = false>
__global__ void __launch_bounds__(combine_warps<N>() * 32u)
attn_combine_kernel(const __grid_constant__ CombineParams<N> p) {
    constexpr uint32_t kWarps = combine_warps<N>();
    __shared__ float red_max[kCombinePhases];
    __shared__ float red_acc[kCombinePhases][kCombineDims + 1];
    // The next kernel of the stream may be staged as soon as every CTA of this grid is resident:
    // whatever it does before its own dependency wait must not depend on this grid (the decode
    // partition kernel only requests old K/V rows there).  Then wait for the partition kernel's
    // records (this grid is its programmatic dependent).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t px_epoch = p.px.world != 0u ? exchange_epoch(p.px) : 0u;
    const uint32_t px_parity = p.px.step != nullptr ? (px_epoch & 1u) : 0u;
    if (p.px.wait_flags != nullptr) {
        // Split-KV merge: the records of the other ranks are pushed into this GPU's memory by
        // kernels running on THEIR GPUs; wait, with a time limit, until every rank's flag carries
        // this step's epoch.  On expiry the CTA latches DeviceWaitTimeout and writes nothing.
        __shared__ uint32_t arrived;
        if (threadIdx.x == 0) {
            const unsigned long long t0 = combine_now_ns();
            const uint32_t* flags = p.px.wait_flags + px_parity * p.px.flag_parity_words;
            uint32_t ok = 1u;
            for (uint32_t r = 0; r < p.px.world && ok; ++r) {
                for (;;) {
                    uint32_t v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
                    if (v == px_epoch) break;
                    if (combine_now_ns() - t0 > 1000ull * p.px.wait_limit_us) {
                        ok = 0u;
                        atomicCAS(p.px.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
                        p.px.status[kStatusDetail] = r;
                        break;
                    }
                    __nanosleep(64);
                }
            }
            arrived = ok;
        }
        __syncthreads();
        if (arrived == 0u) return;   // (the step counter stays: the caller sees the status and starts over)
    }
    const CombineLane& cl = kInd ? p.tables->comb[blockIdx.y] : p.lane[blockIdx.y];
    if (kInd && cl.nparts == 0u) return;   // a lane the setup kernel rejected (context beyond capacity): status is latched
    const uint32_t head = blockIdx.x >> 2, quarter = blockIdx.x & 3u;
    const float* base = cl.records + head * cl.head_stride +
                        (p.px.wait_flags != nullptr ? uint64_t(px_parity) * p.px.out_parity_floats : 0ull);
    // the gate logit of the dim this thread finishes: requested now, used after the merge
    float gate_logit = 0.0f;
    if (threadIdx.x < kCombineDims && p.out != nullptr && p.gate != nullptr)
        gate_logit = bf2f(p.gate[cl.row * p.query_stride + head * kHeadDim + quarter * kCombineDims + threadIdx.x]);
    const float big = merge_records<kWarps>(base, cl.part_stride, cl.nparts, quarter, red_max, red_acc);
    if (p.px.world != 0u && p.px.ll[0] != nullptr) {
        // ---- split-KV across GPUs in this one kernel: store this rank's merged slice into every
        // rank's buffer, wait (bounded) for every rank's slice of this (head, quarter), merge the
        // world's records in rank order with the arithmetic of the merge above, gate, store.
        static_assert(kCombineDims == kCombineDimsPerCta, "exchange slice");
        static_assert(kMaxPeers * kExchangeWords <= combine_warps<1>() * 32u, "one poller per word");
        __shared__ float got[kMaxPeers][kExchangeWords];
        __shared__ uint32_t exchange_failed;
        const uint32_t world = p.px.world;
        const uint64_t slice = (uint64_t(head) * 4u + quarter) * kExchangeWords;
        const uint64_t per_rank = uint64_t(kQHeads) * 4u * kExchangeWords;
        if (threadIdx.x == 0) exchange_failed = 0u;
        if (threadIdx.x < kExchangeWords) {
            const float value = threadIdx.x < kCombineDims ? red_acc[0][threadIdx.x]
                                : threadIdx.x == kCombineDims ? big : red_acc[0][kCombineDims];
            const unsigned long long word = (unsigned long long)__float_as_uint(value) | ((unsigned long long)px_epoch << 32);
            const uint64_t at = (uint64_t(px_parity) * world + p.px.ll_rank) * per_rank + slice + threadIdx.x;
            for (uint32_t r = 0; r < world; ++r)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.px.ll[r] + at), "l"(word) : "memory");
        }
        __syncthreads();
        if (threadIdx.x < world * kExchangeWords) {
            const uint32_t r = threadIdx.x / kExchangeWords, t = threadIdx.x % kExchangeWords;
            const unsigned long long* src = p.px.ll[p.px.ll_rank] + (uint64_t(px_parity) * world + r) * per_rank + slice + t;
            const unsigned long long t0 = combine_now_ns();
            for (uint32_t spin = 0;; ++spin) {
                unsigned long long word;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
                if (uint32_t(word >> 32) == px_epoch) {
                    got[r][t] = __uint_as_float(uint32_t(word));
                    break;
                }
                __nanosleep(32);
                if ((spin & 63u) == 63u && combine_now_ns() - t0 > 1000ull * p.px.wait_limit_us) {
                    exchange_failed = 1u;
                    if (t == 0) {
                        atomicCAS(p.px.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
                        p.px.status[kStatusDetail] = r;
                    }
                    break;
                }
            }
        }
        __syncthreads();
        if (exchange_failed != 0u) return;   // nothing written; the step counter stays
        if (threadIdx.x < kCombineDims) {
            float top = -INFINITY;
            for (uint32_t r = 0; r < world; ++r) top = fmaxf(top, got[r][kCombineDims]);
            float num = 0.0f, den = 0.0f;
            for (uint32_t r = 0; r < world; ++r) {
                const float w = got[r][kCombineDims] == -INFINITY ? 0.0f : expf(got[r][kCombineDims] - top);
                num = __fadd_rn(num, __fmul_rn(w, got[r][threadIdx.x]));
                den = __fadd_rn(den, __fmul_rn(w, got[r][kCombineDims + 1u]));
            }
            num = __fadd_rn(num, 0.0f);   // (the phases of the merge above that hold no record add +0)
            den = __fadd_rn(den, 0.0f);
            const uint64_t at = cl.row * p.query_stride + head * kHeadDim + quarter * kCombineDims + threadIdx.x;
            p.out[at] = f2bf((num / den) * (1.0f / (1.0f + expf(-gate_logit))));
        }
        __syncthreads();
        if (threadIdx.x == 0 && p.px.step != nullptr) {
            const uint32_t total_ctas = gridDim.x * gridDim.y;
            if (atomicAdd(p.px.done_counter, 1u) == total_ctas - 1u) {
                *p.px.done_counter = 0u;
                asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.px.step), "r"(px_epoch) : "memory");
            }
        }
        return;
    }
    if (threadIdx.x < kCombineDims) {
        const uint32_t dd = quarter * kCombineDims + threadIdx.x;
        const float acc = red_acc[0][threadIdx.x], total = red_acc[0][kCombineDims];
        if (p.px.world != 0u && p.px.wait_flags == nullptr) {
            // push this head's slice of the merged record into every rank's gather buffer
            for (uint32_t r = 0; r < p.px.world; ++r) {
                float* ro = p.px.peer_out[r] + uint64_t(px_parity) * p.px.out_parity_floats + head * kRecordFloats;
                ro[dd] = acc;
                if (dd == 0) {
                    ro[kHeadDim] = big;
                    ro[kHeadDim + 1u] = total;
                }
            }
        } else if (p.record_out != nullptr) {
            float* ro = p.record_out + (uint64_t(blockIdx.y) * kQHeads + head) * kRecordFloats;
            ro[dd] = acc;
            if (dd == 0) {
                ro[kHeadDim] = big;
                ro[kHeadDim + 1u] = total;
            }
        } else {
            const uint64_t at = cl.row * p.query_stride + head * kHeadDim + dd;
            p.out[at] = f2bf((acc / total) * (1.0f / (1.0f + expf(-gate_logit))));
        }
    }
    if (p.px.world != 0u && p.px.wait_flags == nullptr) {
        // The CTA that finishes last raises this rank's flag on every rank: each CTA makes its
        // peer stores visible system-wide, then counts itself; the counter resets for the next call.
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t total_ctas = gridDim.x * gridDim.y;
            if (atomicAdd(p.px.done_counter, 1u) == total_ctas - 1u) {
                *p.px.done_counter = 0u;
                __threadfence_system();
                for (uint32_t r = 0; r < p.px.world; ++r)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.px.peer_flag[r] + px_parity * p.px.flag_parity_words),
                                 "r"(px_epoch) : "memory");
            }
        }
    }
    if (p.px.wait_flags != nullptr && p.px.step != nullptr) {
        // Every CTA has read the step counter by now; the one that finishes last moves it on.
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t total_ctas = gridDim.x * gridDim.y;
            if (atomicAdd(p.px.done_counter, 1u) == total_ctas - 1u) {
                *p.px.done_counter = 0u;
                asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p.px.step), "r"(px_epoch) : "memory");
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------
struct DecodeRequest {
    const void* q;
    const void* gate;
    const void* keys;
    const void* values;
    void* out;        // gated output rows, or null
    void* record_out; // merged records, or null
    void* scratch;
    uint64_t scratch_bytes;
    uint64_t query_stride;
    uint32_t capacity;
    const PeerExchange* px = nullptr;
};

template <uint32_t N>
static tatara_status launch_decode(tatara_ctx* ctx, cudaStream_t stream, const DecodeRequest& r,
                                   const tatara_attn_lane* lanes, const uint32_t* key_begin,
                                   const uint32_t* key_end, const uint32_t* rows, uint32_t n_lanes,
                                   const char* what) {
    DecParams<N> dp{};
    CombineParams<N> cp{};
    dp.q = static_cast<const __nv_bfloat16*>(r.q);
    dp.keys = static_cast<const __nv_bfloat16*>(r.keys);
    dp.values = static_cast<const __nv_bfloat16*>(r.values);
    dp.records = static_cast<float*>(r.scratch);
    dp.query_stride = r.query_stride;
    dp.capacity = r.capacity;
    dp.l2_prefetch_keys = ctx->decode_l2_prefetch_keys;
    dp.n_lanes = n_lanes;
    uint64_t rec_floats = 0;
    uint32_t items = 0;
    for (uint32_t i = 0; i < n_lanes; ++i) {
        DecLane& l = dp.lane[i];
        l.kv_offset = lanes[i].kv_offset;
        l.key_begin = key_begin[i];
        l.key_end = key_end[i];
        const uint32_t n = l.key_end - l.key_begin;
        l.part_keys = partition_keys(n);
        l.nparts = partition_count(n);
        l.item_start = items;
        l.rec_offset = rec_floats;
        l.row = rows[i];
        items += l.nparts * kKvHeads;
        cp.lane[i].records = dp.records + rec_floats;
        cp.lane[i].head_stride = uint64_t(l.nparts) * kRecordFloats;
        cp.lane[i].part_stride = kRecordFloats;
        cp.lane[i].nparts = l.nparts;
        cp.lane[i].row = rows[i];
        rec_floats += uint64_t(l.nparts) * kQHeads * kRecordFloats;
    }
    if (rec_floats * sizeof(float) > r.scratch_bytes) return fail(ctx, TATARA_SCRATCH_TOO_SMALL, what);
    dp.total_items = items;
    cp.gate = static_cast<const __nv_bfloat16*>(r.gate);
    cp.out = static_cast<__nv_bfloat16*>(r.out);
    cp.record_out = static_cast<float*>(r.record_out);
    cp.query_stride = r.query_stride;
    if (r.px != nullptr) cp.px = *r.px;

    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(attn_decode_partition_kernel<1>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_decode_partition_kernel<TATARA_MAX_LANES>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes) != cudaSuccess ||
            // the merge runs between two partition kernels: same shared-memory carve-out as theirs,
            // so that the SMs are not reconfigured at every kernel boundary of a decode step
            cudaFuncSetAttribute(attn_combine_kernel<1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
            cudaFuncSetAttribute(attn_combine_kernel<TATARA_MAX_LANES>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return check_launch(ctx, "attn_decode: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    uint32_t grid = items < uint32_t(ctx->sm_count) ? items : uint32_t(ctx->sm_count);
    // One lane with a gated output and no exchange: the merge runs in the partition kernel's own
    // launch (TATARA_POLICY_DECODE_FUSED_MERGE).  At least 64 CTAs then, one per (head, quarter) piece.
    bool fused = false;
    if constexpr (N == 1) {
        fused = ctx->decode_fused_merge != 0u && ctx->merge_counters != nullptr && r.out != nullptr &&
                r.record_out == nullptr && r.px == nullptr && r.gate != nullptr && ctx->sm_count >= 64;
        if (fused) {
            if (grid < kQHeads * 4u) grid = kQHeads * 4u;
            dp.merge_counters = ctx->merge_counters + 2u * (ctx->merge_slot++ % kMergeCounterSlots);
            dp.merge_status = ctx->device_status;
            dp.gate = static_cast<const __nv_bfloat16*>(r.gate);
            dp.out = static_cast<__nv_bfloat16*>(r.out);
        }
    }
    // Both kernels are launched with programmatic stream serialization: each may be staged while
    // its predecessor in the stream drains and blocks in griddepcontrol.wait until that
    // predecessor has finished (a predecessor that never signals simply finishes first).
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = kDecSmemBytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, attn_decode_partition_kernel<N>, dp);
    tatara_status st = check_launch(ctx, what);
    if (st != TATARA_OK || fused) return st;
    cfg.gridDim = dim3(kQHeads * 4, n_lanes);
    cfg.blockDim = dim3(combine_warps<N>() * 32u);
    cfg.dynamicSmemBytes = 0;
    (void)cudaLaunchKernelEx(&cfg, attn_combine_kernel<N>, cp);
    return check_launch(ctx, what);
}

// ---- lane tables in device memory -------------------------------------------------------
// One CTA of 256 threads: thread i derives lane i's cut (tb::partition_keys of its own key count)
// and an exclusive scan over the lanes gives the item and record offsets -- the same tables
// launch_decode builds on the host, so a lane's output bits do not depend on which path ran.
__global__ void __launch_bounds__(TATARA_MAX_LANES)
attn_decode_setup_kernel(const tatara_attn_lane* __restrict__ lanes, uint32_t n_lanes, uint32_t capacity,
                         float* records, DecTables* t, uint32_t* status) {
    __shared__ uint32_t warp_total[TATARA_MAX_LANES / 32];
    const uint32_t i = threadIdx.x, lane = i & 31u, warp = i >> 5;
    uint32_t nparts = 0, part_keys = 16, n = 0;
    uint64_t kv_offset = 0;
    if (i < n_lanes) {
        const tatara_attn_lane l = lanes[i];
        kv_offset = l.kv_offset;
        if (l.context < capacity) {
            n = l.context + 1u;
            part_keys = partition_keys(n);
            nparts = partition_count(n);
        } else {   // nothing is read or written for this lane; the host sees the status at the next sync
            atomicCAS(status + kStatusCode, 0u, uint32_t(TATARA_CONTEXT_OUT_OF_RANGE));
            status[kStatusDetail] = i;
        }
    }
    uint32_t incl = nparts;   // inclusive scan of the partition counts
#pragma unroll
    for (uint32_t off = 1; off < 32; off <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
    }
    if (lane == 31u) warp_total[warp] = incl;
    __syncthreads();
    uint32_t before = 0, total = 0;
    for (uint32_t w = 0; w < TATARA_MAX_LANES / 32; ++w) {
        if (w < warp) before += warp_total[w];
        total += warp_total[w];
    }
    const uint32_t prefix = before + incl - nparts;
    if (i < n_lanes) {
        const uint64_t rec_floats = uint64_t(prefix) * kQHeads * kRecordFloats;
        t->dec[i] = DecLane{kv_offset, rec_floats, 0u, n, part_keys, nparts, prefix * kKvHeads, i};
        t->comb[i] = CombineLane{records + rec_floats, uint64_t(nparts) * kRecordFloats, kRecordFloats, nparts, i};
    }
    if (i == 0) {
        t->n_lanes = n_lanes;
        t->total_items = total * kKvHeads;
    }
}

// After a token: every attention lane's context moves on by one position and every gated-delta
// lane's in / out state offsets trade places (src/runtime/decode_step.cpp:1432-1441 on the host).
__global__ void lanes_advance_kernel(tatara_attn_lane* attn, uint32_t n_attn, tatara_gdn_lane* gdn, uint32_t n_gdn) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_attn) attn[i].context += 1u;
    if (i < n_gdn) {
        const tatara_gdn_lane g = gdn[i];
        gdn[i] = tatara_gdn_lane{g.conv_out, g.conv_in, g.rec_out, g.rec_in};
    }
}

template <uint32_t N>
static tatara_status launch_decode_indirect(tatara_ctx* ctx, cudaStream_t stream, const DecodeRequest& r,
                                            const tatara_attn_lane* lanes_device, uint32_t n_lanes, const char* what) {
    auto* tables = static_cast<DecTables*>(ctx->lane_schedule);
    attn_decode_setup_kernel<<<1, TATARA_MAX_LANES, 0, stream>>>(lanes_device, n_lanes, r.capacity,
                                                                 static_cast<float*>(r.scratch), tables, ctx->device_status);
    tatara_status st = check_launch(ctx, what);
    if (st != TATARA_OK) return st;
    DecParams<N> dp{};
    CombineParams<N> cp{};
    dp.tables = tables;
    dp.q = static_cast<const __nv_bfloat16*>(r.q);
    dp.keys = static_cast<const __nv_bfloat16*>(r.keys);
    dp.values = static_cast<const __nv_bfloat16*>(r.values);
    dp.records = static_cast<float*>(r.scratch);
    dp.query_stride = r.query_stride;
    dp.capacity = r.capacity;
    dp.l2_prefetch_keys = ctx->decode_l2_prefetch_keys;
    cp.tables = tables;
    cp.gate = static_cast<const __nv_bfloat16*>(r.gate);
    cp.out = static_cast<__nv_bfloat16*>(r.out);
    cp.query_stride = r.query_stride;
    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(attn_decode_partition_kernel<N, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kDecSmemBytes) != cudaSuccess ||
            cudaFuncSetAttribute(attn_combine_kernel<N, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return check_launch(ctx, "attn_decode: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    // The item count is only known on the device: every SM gets a (persistent) CTA.  The partition
    // kernel follows the setup kernel in plain stream order (it reads the tables at once); the merge
    // is its programmatic dependent as in the host-table path.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(uint32_t(ctx->sm_count));
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = kDecSmemBytes;
    cfg.stream = stream;
    (void)cudaLaunchKernelEx(&cfg, attn_decode_partition_kernel<N, true>, dp);
    st = check_launch(ctx, what);
    if (st != TATARA_OK) return st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(kQHeads * 4, n_lanes);
    cfg.blockDim = dim3(combine_warps<N>() * 32u);
    cfg.dynamicSmemBytes = 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, attn_combine_kernel<N, true>, cp);
    return check_launch(ctx, what);
}

} // namespace tb

using namespace tb;

extern "C" tatara_status tatara_attn_decode_batch_indirect(tatara_ctx* ctx, void* stream, const void* q,
                                                           const void* gate, const void* keys_pool,
                                                           const void* values_pool,
                                                           const tatara_attn_lane* lanes_device, uint32_t n_lanes,
                                                           uint32_t capacity, uint32_t query_stride, void* out,
                                                           void* scratch, uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!q || !gate || !keys_pool || !values_pool || !out || !scratch || !lanes_device)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_batch_indirect: null buffer");
    if (!aligned(q, 4) || !aligned(keys_pool, 16) || !aligned(values_pool, 16) || !aligned(scratch, 16) ||
        !aligned(lanes_device, 8))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_batch_indirect: misaligned buffer");
    if (n_lanes == 0 || n_lanes > TATARA_MAX_LANES)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_decode_batch_indirect: lanes");
    if (capacity == 0) return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode_batch_indirect: capacity");
    if (query_stride < kQHeads * kHeadDim)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_decode_batch_indirect: query stride");
    // contexts are not known here: the scratch must cover the worst cut of every lane
    if (scratch_bytes < tatara_attn_decode_scratch_bytes(capacity, n_lanes))
        return fail(ctx, TATARA_SCRATCH_TOO_SMALL, "attn_decode_batch_indirect: scratch");
    const DecodeRequest r{q, gate, keys_pool, values_pool, out, nullptr, scratch, scratch_bytes, query_stride, capacity};
    if (n_lanes == 1)
        return launch_decode_indirect<1>(ctx, static_cast<cudaStream_t>(stream), r, lanes_device, 1,
                                         "attn_decode_batch_indirect");
    return launch_decode_indirect<TATARA_MAX_LANES>(ctx, static_cast<cudaStream_t>(stream), r, lanes_device, n_lanes,
                                                    "attn_decode_batch_indirect");
}

extern "C" tatara_status tatara_lanes_advance(tatara_ctx* ctx, void* stream, tatara_attn_lane* attn_lanes_device,
                                              uint32_t n_attn, tatara_gdn_lane* gdn_lanes_device, uint32_t n_gdn) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if ((n_attn != 0 && attn_lanes_device == nullptr) || (n_gdn != 0 && gdn_lanes_device == nullptr))
        return fail(ctx, TATARA_INVALID_BUFFER, "lanes_advance: null table");
    if (n_attn > TATARA_MAX_LANES || n_gdn > TATARA_MAX_LANES || (n_attn | n_gdn) == 0)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "lanes_advance: lanes");
    lanes_advance_kernel<<<1, TATARA_MAX_LANES, 0, static_cast<cudaStream_t>(stream)>>>(attn_lanes_device, n_attn,
                                                                                      gdn_lanes_device, n_gdn);
    return check_launch(ctx, "lanes_advance");
}

extern "C" tatara_status tatara_attn_decode(tatara_ctx* ctx, void* stream, const void* q,
                                            const void* gate, const void* keys, const void* values,
                                            uint32_t context, uint32_t capacity, void* out,
                                            void* scratch, uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!q || !gate || !keys || !values || !out || !scratch)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode: null buffer");
    if (!aligned(q, 4) || !aligned(keys, 16) || !aligned(values, 16) || !aligned(scratch, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode: misaligned buffer");
    if (capacity == 0 || context >= capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode: context >= capacity");
    const DecodeRequest r{q, gate, keys, values, out, nullptr, scratch, scratch_bytes,
                          kQHeads * kHeadDim, capacity};
    const tatara_attn_lane lane{0, context, 0};
    const uint32_t begin = 0, end = context + 1u, row = 0;
    return launch_decode<1>(ctx, static_cast<cudaStream_t>(stream), r, &lane, &begin, &end, &row, 1,
                            "attn_decode");
}

extern "C" tatara_status tatara_attn_decode_batch(tatara_ctx* ctx, void* stream, const void* q,
                                                  const void* gate, const void* keys_pool,
                                                  const void* values_pool,
                                                  const tatara_attn_lane* lanes, uint32_t n_lanes,
                                                  uint32_t capacity, uint32_t query_stride,
                                                  void* out, void* scratch, uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!q || !gate || !keys_pool || !values_pool || !out || !scratch || !lanes)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_batch: null buffer");
    if (!aligned(q, 4) || !aligned(keys_pool, 16) || !aligned(values_pool, 16) || !aligned(scratch, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_batch: misaligned buffer");
    if (n_lanes == 0 || n_lanes > TATARA_MAX_LANES)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_decode_batch: lane count");
    if (query_stride < kQHeads * kHeadDim || (query_stride & 1u))
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_decode_batch: query_stride");
    uint32_t begin[TATARA_MAX_LANES], end[TATARA_MAX_LANES], rows[TATARA_MAX_LANES];
    for (uint32_t i = 0; i < n_lanes; ++i) {
        if (capacity == 0 || lanes[i].context >= capacity)
            return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode_batch: context >= capacity");
        if (lanes[i].kv_offset % 8u)
            return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_batch: kv_offset not 16-byte aligned");
        begin[i] = 0;
        end[i] = lanes[i].context + 1u;
        rows[i] = i;
    }
    const DecodeRequest r{q, gate, keys_pool, values_pool, out, nullptr, scratch, scratch_bytes,
                          query_stride, capacity};
    return launch_decode<TATARA_MAX_LANES>(ctx, static_cast<cudaStream_t>(stream), r, lanes, begin, end,
                                           rows, n_lanes, "attn_decode_batch");
}

extern "C" tatara_status tatara_attn_decode_partial(tatara_ctx* ctx, void* stream, const void* q,
                                                    const void* keys, const void* values,
                                                    uint32_t key_begin, uint32_t key_end,
                                                    uint32_t capacity, void* records_out,
                                                    void* scratch, uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!q || !keys || !values || !records_out || !scratch)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_partial: null buffer");
    if (!aligned(q, 4) || !aligned(keys, 16) || !aligned(values, 16) || !aligned(scratch, 16) ||
        !aligned(records_out, 8))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_partial: misaligned buffer");
    if (capacity == 0 || key_begin >= key_end || key_end > capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode_partial: key range");
    const DecodeRequest r{q, nullptr, keys, values, nullptr, records_out, scratch, scratch_bytes,
                          kQHeads * kHeadDim, capacity};
    const tatara_attn_lane lane{0, key_end - 1u, 0};
    const uint32_t row = 0;
    return launch_decode<1>(ctx, static_cast<cudaStream_t>(stream), r, &lane, &key_begin, &key_end, &row,
                            1, "attn_decode_partial");
}

extern "C" tatara_status tatara_attn_combine(tatara_ctx* ctx, void* stream, const void* records,
                                             uint32_t nparts, uint64_t head_stride,
                                             uint64_t part_stride, const void* gate, void* out) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!records || !gate || !out) return fail(ctx, TATARA_INVALID_BUFFER, "attn_combine: null buffer");
    if (!aligned(records, 8) || (head_stride & 1u) || (part_stride & 1u))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_combine: records must be 8-byte aligned");
    if (nparts == 0) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_combine: nparts");
    CombineParams<1> cp{};
    cp.gate = static_cast<const __nv_bfloat16*>(gate);
    cp.out = static_cast<__nv_bfloat16*>(out);
    cp.record_out = nullptr;
    cp.query_stride = kQHeads * kHeadDim;
    cp.lane[0] = CombineLane{static_cast<const float*>(records), head_stride, part_stride, nparts, 0};
    attn_combine_kernel<1><<<dim3(kQHeads * 4, 1), combine_warps<1>() * 32u, 0, static_cast<cudaStream_t>(stream)>>>(cp);
    return check_launch(ctx, "attn_combine");
}

extern "C" tatara_status tatara_attn_prefill_control(tatara_ctx* ctx, void* stream, const void* query,
                                                     const void* gate, const void* keys,
                                                     const void* values, uint32_t context_base,
                                                     uint32_t rows, uint32_t capacity, void* out,
                                                     void* scratch, uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!query || !gate || !keys || !values || !out || !scratch)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_prefill_control: null buffer");
    if (!aligned(query, 4) || !aligned(keys, 16) || !aligned(values, 16) || !aligned(scratch, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_prefill_control: misaligned buffer");
    if (rows == 0) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_prefill_control: rows");
    if (capacity == 0 || uint64_t(context_base) + rows > capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_prefill_control: rows past capacity");
    const DecodeRequest r{query, gate, keys, values, out, nullptr, scratch, scratch_bytes,
                          kQHeads * kHeadDim, capacity};
    tatara_attn_lane lanes[TATARA_MAX_LANES];
    uint32_t begin[TATARA_MAX_LANES], end[TATARA_MAX_LANES], row_index[TATARA_MAX_LANES];
    for (uint32_t first = 0; first < rows; first += TATARA_MAX_LANES) {
        const uint32_t n = rows - first < TATARA_MAX_LANES ? rows - first : TATARA_MAX_LANES;
        for (uint32_t i = 0; i < n; ++i) {
            lanes[i] = tatara_attn_lane{0, context_base + first + i, 0};
            begin[i] = 0;
            end[i] = context_base + first + i + 1u;
            row_index[i] = first + i;
        }
        const tatara_status st = launch_decode<TATARA_MAX_LANES>(
            ctx, static_cast<cudaStream_t>(stream), r, lanes, begin, end, row_index, n, "attn_prefill_control");
        if (st != TATARA_OK) return st;
    }
    return TATARA_OK;
}

// ---- allocation-free decode ---------------------------------------------------------------
// Record scratch that lives inside the library image instead of in caller memory.  Every GPU
// that loads the library holds these 1.2 MB until the process exits.
namespace tb {
// tb::partition_keys never cuts a lane into more than 74 partitions (128-key partitions up to
// 9472 keys, 74 equal ones beyond), so 74 x 16 records serve any key count; the cap on the key
// count is the model's maximum context (include/tatara/runtime/prefill_geometry.h:14).
constexpr uint32_t kStaticMaxKeys = 262144;
constexpr uint32_t kStaticMaxParts = kSmCount / kKvHeads;
static __device__ __align__(256) float g_static_records[kStaticMaxParts * kQHeads * kRecordFloats];

struct StaticSetup {
    std::once_flag once;
    cudaError_t error = cudaErrorNotReady;
    float* records = nullptr; // device address of g_static_records on that device
    int sm_count = 0;
};
static StaticSetup g_static_setup[64];
} // namespace tb

extern "C" tatara_status tatara_attn_decode_static(tatara_ctx* ctx, void* stream, const void* q,
                                                   const void* gate, const void* keys,
                                                   const void* values, uint32_t context,
                                                   uint32_t capacity, void* out) {
    // ctx may be null: it is used for the error text and the launch counter only.
    if (!q || !gate || !keys || !values || !out)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_static: null buffer");
    if (!aligned(q, 4) || !aligned(keys, 16) || !aligned(values, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_static: misaligned buffer");
    if (capacity == 0 || context >= capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode_static: context >= capacity");
    if (context >= kStaticMaxKeys || partition_count(context + 1u) > kStaticMaxParts)
        return fail(ctx, TATARA_SCRATCH_TOO_SMALL,
                    "attn_decode_static: the built-in scratch covers at most 262144 attended keys; "
                    "use tatara_attn_decode with caller scratch beyond that");
    const uint32_t n = context + 1u;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
        return fail(ctx, TATARA_INVALID_DEVICE, "attn_decode_static: no current device");
    StaticSetup& setup = g_static_setup[device];
    // Once per device, with that device current; a second host thread that arrives meanwhile waits
    // here until the first has finished.  In host code the array's name is only a stand-in for the
    // symbol; the address a kernel may use comes from the runtime.
    std::call_once(setup.once, [&setup, device]() {
        float* address = nullptr;
        cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_records);
        if (err == cudaSuccess)
            err = cudaDeviceGetAttribute(&setup.sm_count, cudaDevAttrMultiProcessorCount, device);
        if (err == cudaSuccess)
            err = cudaFuncSetAttribute(attn_decode_partition_kernel<1>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes);
        if (err == cudaSuccess && address == nullptr) err = cudaErrorInvalidSymbol;
        setup.records = address;
        setup.error = err;
    });
    if (setup.error != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(ctx, TATARA_CUDA_ERROR, "attn_decode_static: set-up of the built-in scratch failed");
    }
    DecParams<1> dp{};
    dp.q = static_cast<const __nv_bfloat16*>(q);
    dp.keys = static_cast<const __nv_bfloat16*>(keys);
    dp.values = static_cast<const __nv_bfloat16*>(values);
    dp.records = setup.records;
    dp.query_stride = kQHeads * kHeadDim;
    dp.capacity = capacity;
    dp.l2_prefetch_keys = ctx != nullptr ? ctx->decode_l2_prefetch_keys : kDecodeL2PrefetchKeys;
    dp.n_lanes = 1;
    DecLane& l = dp.lane[0];
    l.kv_offset = 0;
    l.rec_offset = 0;
    l.key_begin = 0;
    l.key_end = n;
    l.part_keys = partition_keys(n);
    l.nparts = partition_count(n);
    l.item_start = 0;
    l.row = 0;
    dp.total_items = l.nparts * kKvHeads;
    CombineParams<1> cp{};
    cp.gate = static_cast<const __nv_bfloat16*>(gate);
    cp.out = static_cast<__nv_bfloat16*>(out);
    cp.record_out = nullptr;
    cp.query_stride = kQHeads * kHeadDim;
    cp.lane[0] = CombineLane{setup.records, uint64_t(l.nparts) * kRecordFloats, kRecordFloats, l.nparts, 0};
    const uint32_t grid = dp.total_items < uint32_t(setup.sm_count) ? dp.total_items : uint32_t(setup.sm_count);
    auto s = static_cast<cudaStream_t>(stream);
    attn_decode_partition_kernel<1><<<grid, kDecThreads, kDecSmemBytes, s>>>(dp);
    attn_combine_kernel<1><<<dim3(kQHeads * 4, 1), combine_warps<1>() * 32u, 0, s>>>(cp);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(ctx, TATARA_CUDA_ERROR, cudaGetErrorString(err));
    if (ctx != nullptr) ctx->launches += 2;
    return TATARA_OK;
}

// ---- split-KV across GPUs over peer memory -----------------------------------------------
extern "C" tatara_status tatara_peer_buffer_create(tatara_ctx* ctx, uint64_t bytes, void** ptr, void* handle64) {
    if (ctx == nullptr || ptr == nullptr || handle64 == nullptr) return TATARA_INVALID_BUFFER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess ||
        cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p) != cudaSuccess) {
        (void)cudaGetLastError();
        if (p != nullptr) cudaFree(p);
        return fail(ctx, TATARA_CUDA_ERROR, "peer_buffer_create: allocation or IPC export failed");
    }
    cudaDeviceSynchronize();
    *ptr = p;
    return TATARA_OK;
}

extern "C" tatara_status tatara_peer_buffer_open(tatara_ctx* ctx, const void* handle64, void** ptr) {
    if (ctx == nullptr || ptr == nullptr || handle64 == nullptr) return TATARA_INVALID_BUFFER;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(ctx, TATARA_CUDA_ERROR, "peer_buffer_open: cudaIpcOpenMemHandle failed");
    }
    return TATARA_OK;
}

extern "C" tatara_status tatara_peer_buffer_close(tatara_ctx* ctx, void* ptr, int owned) {
    if (ctx == nullptr || ptr == nullptr) return TATARA_INVALID_BUFFER;
    const cudaError_t err = owned ? cudaFree(ptr) : cudaIpcCloseMemHandle(ptr);
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(ctx, TATARA_CUDA_ERROR, "peer_buffer_close failed");
    }
    return TATARA_OK;
}

extern "C" tatara_status tatara_attn_decode_partial_push(tatara_ctx* ctx, void* stream, const void* q,
                                                         const void* keys, const void* values,
                                                         uint32_t key_begin, uint32_t key_end,
                                                         uint32_t capacity, void* const* peer_gather,
                                                         void* const* peer_flags, uint32_t rank,
                                                         uint32_t world, uint32_t epoch, void* scratch,
                                                         uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!q || !keys || !values || !scratch || !peer_gather || !peer_flags)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_partial_push: null buffer");
    if (!aligned(q, 4) || !aligned(keys, 16) || !aligned(values, 16) || !aligned(scratch, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_partial_push: misaligned buffer");
    if (world == 0 || world > kMaxPeers || rank >= world || epoch == 0)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_decode_partial_push: rank / world / epoch");
    if (capacity == 0 || key_begin >= key_end || key_end > capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode_partial_push: key range");
    PeerExchange px{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!peer_gather[r] || !peer_flags[r] || !aligned(peer_gather[r], 8))
            return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_partial_push: peer pointer");
        px.peer_out[r] = static_cast<float*>(peer_gather[r]) + uint64_t(rank) * kQHeads * kRecordFloats;
        px.peer_flag[r] = static_cast<uint32_t*>(peer_flags[r]) + rank;
    }
    px.done_counter = ctx->device_status + 2;
    px.status = ctx->device_status;
    px.world = world;
    px.epoch = epoch;
    DecodeRequest r{q, nullptr, keys, values, nullptr, nullptr, scratch, scratch_bytes, kQHeads * kHeadDim, capacity};
    r.px = &px;
    const tatara_attn_lane lane{0, key_end - 1u, 0};
    const uint32_t row = 0;
    return launch_decode<1>(ctx, static_cast<cudaStream_t>(stream), r, &lane, &key_begin, &key_end, &row, 1,
                            "attn_decode_partial_push");
}

extern "C" uint64_t tatara_split_buffer_bytes(uint32_t world) {
    // [2 parities][world source ranks][16 heads][4 quarters][66] 8-byte words | u32 step counter (+ padding to 16 bytes)
    return 2ull * world * kQHeads * 4ull * kExchangeWords * sizeof(unsigned long long) + 16ull;
}

extern "C" tatara_status tatara_attn_decode_split(tatara_ctx* ctx, void* stream, const void* q, const void* gate,
                                                  const void* keys, const void* values, uint32_t key_begin,
                                                  uint32_t key_end, uint32_t capacity, void* const* peer_buffers,
                                                  uint32_t rank, uint32_t world, uint32_t wait_limit_us, void* out,
                                                  void* scratch, uint64_t scratch_bytes) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!q || !gate || !keys || !values || !out || !scratch || !peer_buffers)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_split: null buffer");
    if (!aligned(q, 4) || !aligned(keys, 16) || !aligned(values, 16) || !aligned(scratch, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_split: misaligned buffer");
    if (world == 0 || world > kMaxPeers || rank >= world || wait_limit_us == 0 || wait_limit_us > 2000000u)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_decode_split: rank / world / time limit");
    if (capacity == 0 || key_begin >= key_end || key_end > capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_decode_split: key range");
    PeerExchange px{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!peer_buffers[r] || !aligned(peer_buffers[r], 16))
            return fail(ctx, TATARA_INVALID_BUFFER, "attn_decode_split: peer buffer");
        px.ll[r] = static_cast<unsigned long long*>(peer_buffers[r]);
    }
    px.ll_rank = rank;
    px.step = reinterpret_cast<uint32_t*>(px.ll[rank] + 2ull * world * kQHeads * 4ull * kExchangeWords);
    px.done_counter = ctx->device_status + 3;
    px.status = ctx->device_status;
    px.world = world;
    px.wait_limit_us = wait_limit_us;
    // Two kernels, as the single-GPU decode: the partitions of this rank's key range, then one merge
    // kernel that also carries the exchange (programmatic dependent of the first).
    DecodeRequest r{q, gate, keys, values, out, nullptr, scratch, scratch_bytes, kQHeads * kHeadDim, capacity};
    r.px = &px;
    const tatara_attn_lane lane{0, key_end - 1u, 0};
    const uint32_t row = 0;
    return launch_decode<1>(ctx, static_cast<cudaStream_t>(stream), r, &lane, &key_begin, &key_end, &row, 1,
                            "attn_decode_split");
}

extern "C" tatara_status tatara_attn_combine_wait(tatara_ctx* ctx, void* stream, const void* gather,
                                                  const void* flags, uint32_t world, uint32_t epoch,
                                                  uint32_t wait_limit_us, const void* gate, void* out) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!gather || !flags || !gate || !out) return fail(ctx, TATARA_INVALID_BUFFER, "attn_combine_wait: null buffer");
    if (!aligned(gather, 8) || !aligned(flags, 4))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_combine_wait: misaligned buffer");
    if (world == 0 || world > kMaxPeers || epoch == 0 || wait_limit_us == 0 || wait_limit_us > 2000000u)
        return fail(ctx, TATARA_INVALID_STREAM_GROUP, "attn_combine_wait: world / epoch / time limit");
    CombineParams<1> cp{};
    cp.gate = static_cast<const __nv_bfloat16*>(gate);
    cp.out = static_cast<__nv_bfloat16*>(out);
    cp.query_stride = kQHeads * kHeadDim;
    // gather layout [rank][head][258]: head stride 258, part (= rank) stride 16*258
    cp.lane[0] = CombineLane{static_cast<const float*>(gather), kRecordFloats, uint64_t(kQHeads) * kRecordFloats, world, 0};
    cp.px.wait_flags = static_cast<const uint32_t*>(flags);
    cp.px.status = ctx->device_status;
    cp.px.world = world;
    cp.px.epoch = epoch;
    cp.px.wait_limit_us = wait_limit_us;
    attn_combine_kernel<1><<<dim3(kQHeads * 4, 1), combine_warps<1>() * 32u, 0, static_cast<cudaStream_t>(stream)>>>(cp);
    return check_launch(ctx, "attn_combine_wait");
}
