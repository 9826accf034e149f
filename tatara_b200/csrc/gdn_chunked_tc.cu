// Chunk-64 evaluation of the Gated DeltaNet recurrence on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands brought in by TMA).  The reference
// evaluates the same recurrence one step at a time (prefill_gdn.metal:137-281; CPU model
// tests/native/kernel_reference.cpp:498-563).
//
// Per v-head, state S [128 v][128 k], a chunk of C = 64 steps, G_r = sum_{i<=r} log(decay_i):
//     A[r,i] = beta_r e^{G_r-G_i} (k_r.k_i) (i < r),      T = (I + A)^-1
//     W = T diag(beta e^{G}) K,   U = T diag(beta) V,      P[r,i] = e^{G_r-G_i} (q_r.k_i) (i <= r)
//     Delta = U - W S0^T,   S_C = e^{G_C} S0 + Delta^T diag(s) K,   s_i = e^{G_C-G_i}
//     O     = diag(e^{G}) Q S0^T + P Delta
// Written as a TRANSITION per chunk, everything that does not involve the state moves out of the
// serial part:
//     S_C = e^{G_C} S0 + Us^T K - S0 M',        M' = (diag(s) W)^T K            [128 k' x 128 k]
//     O^T = O0^T + S0 Q~^T,                     Q~ = diag(e^{G}) Q - P W,  O0 = P U
// Two kernels:
//   gdn_tc_prepare_kernel -- no state.  Persistent CTAs of 256 threads (two per SM) walk the (chunk,
//     v-head) units: six small MMA groups ([K;Q] K^T, K^T T_W^T, V^T T_U^T, Ws^T K, W^T P^T, U^T P^T)
//     with the f32 inverse of the unit lower-triangular (I + A) between the first and the second
//     (16 x 16 diagonal blocks by forward substitution, then block doubling: no bf16 enters the solve).
//     -M', Us^T, Q~^T, O0^T leave as bf16 images of the 128-byte-swizzled shared-memory tiles the scan
//     wants (bulk copies out of shared memory: one coalesced stream per tile).
//   gdn_tc_scan_kernel -- one CTA per v-head walks the chunks.  The state is the f32 accumulator of
//     the transition MMAs in tensor memory; between two chunks four warps read it (tcgen05.ld),
//     scale it by e^{G_C} in f32 in place (tcgen05.st) and store its bf16 copy beside it in tensor
//     memory, from where the MMAs take it as their A operand.  The dependent chain of a chunk is that
//     round trip plus twelve MMAs; the output MMAs, the epilogue and the operand ring run beside it.
// Every mbarrier wait is bounded; on expiry the CTA latches DeviceWaitTimeout, frees its tensor
// memory and returns.
#include "tc05.cuh"

namespace tb {

constexpr uint32_t kTcChunk = 64;
constexpr uint32_t kUnitM = 128u * 128u * 2u;   // -M'   [128 k'][128 k] bf16
constexpr uint32_t kUnitU = 128u * 64u * 2u;    // Us^T  [128 v][64 i]  bf16
constexpr uint32_t kUnitQ = 128u * 64u * 2u;    // Q~^T  [128 k'][64 r] bf16
constexpr uint32_t kUnitO = 128u * 64u * 2u;    // O0^T  [128 v][64 r]  bf16

struct TcPlanes {
    uint8_t* m;
    uint8_t* u;
    uint8_t* q;
    uint8_t* o;
    float* gamma;     // e^{G_C} per unit
};

__host__ __device__ inline uint64_t tc_units(uint32_t rows) {
    return uint64_t((rows + kTcChunk - 1u) / kTcChunk) * kGdnValueHeads;
}
uint64_t gdn_tc_scratch_bytes(uint32_t rows) {
    const uint64_t units = tc_units(rows);   // four planes, then e^{G_C} per unit, then the ready word per unit
    return units * (kUnitM + kUnitU + kUnitQ + kUnitO) + 2u * ((units * 4u + 127u) & ~uint64_t(127));
}

// kind::f16 instruction descriptor with both majors selectable (bit 15: A is MN-major, bit 16: B).
__host__ __device__ constexpr uint32_t instr_desc2(uint32_t m, uint32_t n, bool a_mn, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn ? (1u << 15) : 0u) | (b_mn ? (1u << 16) : 0u) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Byte offset of the 16-byte chunk `chunk` of row `row` in a 128-byte-swizzled tile of 128-byte rows.
__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
}
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- kernel 1: per (chunk, v-head) ---------------------------------------------------------
// 256 threads: thread (row, half) = tensor-memory lane `row` (warp & 3 selects the lane quarter) and
// one half of the columns of whatever tile is being read (warps 0..3 the first half, 4..7 the second).
// A CTA runs this code once, so loops over column blocks stay rolled (16 columns per pass): what
// matters is the number of distinct instructions fetched, not the trip count.
constexpr uint32_t kPrKQ = 0;            // [K;Q] : 2 dim-atoms x [128 rows x 128 B]; rows 0..63 K, 64..127 Q
constexpr uint32_t kPrV = 32768;         // V : 2 v-atoms x [64 rows x 128 B]; later U^T [128 rows x 128 B]
constexpr uint32_t kPrA = 49152;         // A f32 [64][64] as [group][row][4]; later W^T [128 rows x 128 B]
constexpr uint32_t kPrWs = 65536;        // T f32 as [row group][column][4] during the solve; later Ws^T [128 rows x 128 B]
constexpr uint32_t kPrP = 81920;         // P [64 rows x 128 B]
constexpr uint32_t kPrTW = 90112;        // T diag(beta e^G)  [64 rows x 128 B]
constexpr uint32_t kPrTU = 98304;        // T diag(beta)      [64 rows x 128 B]
constexpr uint32_t kPrVec = 106496;      // g_cum | beta | s | e^G  (4 x 64 f32)
constexpr uint32_t kPrBar = 107520;
constexpr uint32_t kPrSmem = kPrBar + 64;
constexpr uint32_t kPrCols = 256;
constexpr uint32_t kPrThreads = 256;
constexpr uint32_t kPrStoreThread = 128;   // lane 0 of warp 4: issues the plane copies of a unit, see tc_prepare_units
// staging of the output planes (the images the scan copies back into shared memory), over dead tiles
constexpr uint32_t kPrStU = kPrTW;       // Us^T, written while K, Q, P, W^T, Ws^T, U^T are live
constexpr uint32_t kPrStM = kPrV;        // -M' : two tiles, 32 KiB   (final epilogue: everything but the Q rows is dead)
constexpr uint32_t kPrStQ = kPrWs;       // Q~^T
constexpr uint32_t kPrStO = kPrP;        // O0^T (runs over P, T_W)

struct TcPrepareParams {
    const float* decay;
    const float* beta;
    TcPlanes planes;
    uint32_t* status;
    uint32_t rows, n_units;
};

__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// One contiguous block of shared memory -> global memory through the bulk-copy engine.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// 16 f32 -> two 16-byte groups of bf16 at chunks c and c + 1 of a swizzled 128-byte row
__device__ __forceinline__ void store_bf16x16(uint8_t* tile, uint32_t row, uint32_t chunk, const float* v) {
    *reinterpret_cast<uint4*>(tile + sw128(row, chunk)) =
        make_uint4(pack_bf2(v[0], v[1]), pack_bf2(v[2], v[3]), pack_bf2(v[4], v[5]), pack_bf2(v[6], v[7]));
    *reinterpret_cast<uint4*>(tile + sw128(row, chunk + 1u)) =
        make_uint4(pack_bf2(v[8], v[9]), pack_bf2(v[10], v[11]), pack_bf2(v[12], v[13]), pack_bf2(v[14], v[15]));
}
// f32 [64][64] matrix stored as [16-byte group of four columns][row][4]: a warp that writes or reads one
// group of 32 consecutive rows touches 512 contiguous bytes, and a (row, group) address is an affine
// function of both -- the solve below steps through it with immediate offsets.
__device__ __forceinline__ uint32_t gmat(uint32_t row, uint32_t group) { return group * 1024u + row * 16u; }

// CTA barrier over the 256 threads of one prepare group: barrier kBar (0 = the whole CTA of the
// stand-alone kernel; 1, 2 = the two groups of a worker CTA of the fused kernel).
// (the barrier number is a run-time operand: the two groups of a worker CTA run the SAME code; as a template
// parameter it made two copies of the whole unit loop, twice the instruction-cache footprint per SM)
__device__ __forceinline__ void group_sync(uint32_t bar_id) { asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory"); }
__device__ __forceinline__ bool group_and(uint32_t bar_id, bool pred) {
    uint32_t r;
    asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n bar.red.and.pred q, %2, 256, p;\n selp.u32 %0, 1, 0, q;\n}"
                 : "=r"(r) : "r"(pred ? 1u : 0u), "r"(bar_id) : "memory");
    return r != 0u;
}

// The units first_unit, first_unit + unit_stride, ... by one group of 256 threads (tid = 0..255) that owns
// kPrSmem bytes of shared memory at `smem` (its two mbarriers initialised, abort flag cleared) and
// kPrCols columns of tensor memory at `tmem`.  `ready` (or null): one word per unit, set to `epoch` once
// the unit's planes are complete in global memory.
__device__ __forceinline__ void tc_prepare_units(const uint32_t bar_id, const CUtensorMap& map_qk, const CUtensorMap& map_v, const TcPrepareParams& p,
                                                 uint8_t* smem, uint32_t tmem, uint32_t tid, uint32_t first_unit,
                                                 uint32_t unit_stride, uint32_t* ready, uint32_t epoch) {
    const uint32_t warp = tid >> 5, lane = tid & 31u;
    const uint32_t row = (warp & 3u) * 32u + lane, half = warp >> 2;
    const uint32_t base = s2u(smem);
    const uint32_t bar_load = base + kPrBar, bar_mma = base + kPrBar + 8, bar_v = base + kPrBar + 32;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kPrBar + 16);
    float* g_cum = reinterpret_cast<float*>(smem + kPrVec);
    float* beta_s = g_cum + 64;
    float* s_end = g_cum + 128;    // e^{G_C - G_r}
    float* e_g = g_cum + 192;      // e^{G_r}
    const uint32_t tlane = ((warp & 3u) * 32u) << 16;
    bool ok = true;
    uint32_t mma_phase = 0;     // completions of bar_mma so far (three per unit)
    // Thread kPrStoreThread hands the four plane images of a unit to the copy engine (thread 0 only the Us^T image,
    // in the middle of the unit) and owns what follows from that, each at a point where it would otherwise idle:
    //  * the images must have LEFT shared memory before the next unit writes over them: it waits for that
    //    (`wait_group.read`) during the next unit's first MMA group, before the barrier in front of the masks -- the
    //    next unit's K and Q tiles load into a region that holds no image, and its V tile is asked for after that
    //    barrier (V is not needed before the second MMA group).  Waiting at the end of the unit held the whole
    //    group for 2.3 - 4.2 k cycles per unit.
    //  * the unit's ready word may only be released once the images are COMPLETE in global memory: it waits for that
    //    (`wait_group 0`) and stores the word (`st.release.gpu`) while warps 0 and 1 invert the diagonal blocks of
    //    the next unit.  Completed bulk copies are visible to the thread that waited for them, thread 0 has
    //    waited for its Us^T copy before the barriers in between, and a release at gpu scope is cumulative over
    //    what the thread has observed (e^{G_C}, written by warp 1 before those barriers, included).  On thread 0,
    //    with a proxy fence and a __threadfence in front, the release cost the group 1.5 - 3 k cycles per unit.
    uint32_t unreleased = 0xFFFFFFFFu;   // (store thread) the unit whose ready word is not out yet
    auto release_pending = [&]() {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (ready != nullptr && unreleased != 0xFFFFFFFFu)
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ready + unreleased), "r"(epoch) : "memory");
        unreleased = 0xFFFFFFFFu;
    };

    // The K and Q tiles of a unit (one mbarrier completion per unit), and the tiles of the unit after it into L2.
    // Issued by the store thread at the END of the previous unit, AHEAD of that unit's plane copies: the copy
    // engine of the SM takes its work in order, and behind 64 KiB of outgoing images the loads took 3 - 5 k cycles.
    auto issue_kq = [&](uint32_t u) {
        const uint32_t h = u % kGdnValueHeads, q = h >> 1, r0 = (u / kGdnValueHeads) * kTcChunk;
        mbar_expect_tx(bar_load, 32768u);
        for (uint32_t a = 0; a < 2; ++a) {
            tma_load_2d(base + kPrKQ + a * 16384u, &map_qk, bar_load, int(kGdnKOff + q * kGdnDim + a * 64u), int(r0));
            tma_load_2d(base + kPrKQ + a * 16384u + 8192u, &map_qk, bar_load, int(q * kGdnDim + a * 64u), int(r0));
        }
        const uint32_t next = u + unit_stride;
        if (next < p.n_units) {
            const uint32_t nh = next % kGdnValueHeads, nq = nh >> 1, nrow = (next / kGdnValueHeads) * kTcChunk;
            for (uint32_t a = 0; a < 2; ++a) {
                tma_prefetch_2d(&map_qk, int(kGdnKOff + nq * kGdnDim + a * 64u), int(nrow));
                tma_prefetch_2d(&map_qk, int(nq * kGdnDim + a * 64u), int(nrow));
                tma_prefetch_2d(&map_v, int(nh * kGdnDim + a * 64u), int(nrow));
            }
        }
    };
    if (tid == kPrStoreThread && first_unit < p.n_units) issue_kq(first_unit);
    // warp 1: the decay and beta of a unit's 64 steps (two per lane), loaded one unit ahead -- with the K and Q tiles
    // already there when a unit starts, a trip to memory for these at its top was the longest wait of the unit
    float gate_in[4] = {1.0f, 1.0f, 0.0f, 0.0f};   // decay of steps 2 lane, 2 lane + 1 (1: G stays flat), then beta
    auto load_gates = [&](uint32_t u) {
        const uint32_t h = u % kGdnValueHeads, r0 = (u / kGdnValueHeads) * kTcChunk + lane * 2u;
#pragma unroll
        for (uint32_t e = 0; e < 2; ++e) {
            const bool live = r0 + e < p.rows;
            gate_in[e] = live ? __ldg(p.decay + uint64_t(r0 + e) * kGdnValueHeads + h) : 1.0f;
            gate_in[2 + e] = live ? __ldg(p.beta + uint64_t(r0 + e) * kGdnValueHeads + h) : 0.0f;
        }
    };
    if (warp == 1 && first_unit < p.n_units) load_gates(first_unit);

    // Persistent CTAs: barriers and tensor memory are set up once, then the CTA walks its units.
    for (uint32_t it = 0, unit32 = first_unit; unit32 < p.n_units && ok; ++it, unit32 += unit_stride) {
    const uint32_t chunk = unit32 / kGdnValueHeads, head = unit32 % kGdnValueHeads;
    const uint32_t row0 = chunk * kTcChunk;
    const uint32_t live_rows = min(kTcChunk, p.rows - row0);
    const uint64_t unit = unit32;
    if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the previous unit's Us^T copy is complete (issued half a unit ago)
    if (warp == 1) {
        // inclusive cumulative log-decay over the 64 steps (two per lane); rows past the block keep G flat
        const uint32_t r0 = lane * 2u;
        const float g0 = r0 < live_rows ? fmaxf(logf(gate_in[0]), -100.0f) : 0.0f;
        const float g1 = r0 + 1u < live_rows ? fmaxf(logf(gate_in[1]), -100.0f) : 0.0f;
        const float b0 = gate_in[2], b1 = gate_in[3];
        if (unit32 + unit_stride < p.n_units) load_gates(unit32 + unit_stride);
        float incl = g0 + g1;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= uint32_t(off)) incl += up;
        }
        const float g_end = __shfl_sync(0xffffffffu, incl, 31);
        g_cum[r0] = incl - g1;
        g_cum[r0 + 1u] = incl;
        beta_s[r0] = b0;
        beta_s[r0 + 1u] = b1;
        s_end[r0] = __expf(g_end - (incl - g1));
        s_end[r0 + 1u] = __expf(g_end - incl);
        e_g[r0] = __expf(incl - g1);
        e_g[r0 + 1u] = __expf(incl);
        if (lane == 0) p.planes.gamma[unit] = __expf(g_end);
    }
    ok = mbar_wait(bar_load, it & 1u, abort_flag);

    // ---- MMA a: [K;Q] K^T -> rows 0..63 K K^T, rows 64..127 Q K^T (columns 0..63 of tensor memory)
    if (tid == 0 && ok) {
        tc_fence_after();
        constexpr uint32_t idesc = instr_desc2(128, 64, false, false);
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ++ks) {
            const uint32_t at = base + kPrKQ + (ks >> 2) * 16384u + (ks & 3u) * 32u;
            tc_mma(tmem, smem_desc(at, 16, 1024), smem_desc(at, 16, 1024), idesc, ks ? 1u : 0u);
        }
        tc_commit(bar_mma);
    }
    // the previous unit's -M' image (over V, A) and its O0^T image (over P) have left shared memory: the masks write
    // P and A; the Q~^T image (over T, written by the sweep) may still be on its way
    if (tid == kPrStoreThread) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    if (ok) ok = mbar_wait(bar_mma, mma_phase & 1u, abort_flag);
    ++mma_phase;
    group_sync(bar_id);   // the decay vectors of warp 1 are visible; P and A are free
    if (ok) {
        tc_fence_after();
        const uint32_t r = row & 63u;
        const float gr = g_cum[r], br = row < 64u ? beta_s[r] : 1.0f;
        const uint32_t bound = row < 64u ? r : r + 1u;      // A: columns i < r; P: i <= r
#pragma unroll 1
        for (uint32_t blk = 0; blk < 2; ++blk) {
            const uint32_t c0 = half * 32u + blk * 16u;
            float d[16];
            tmem_ld16(tmem + tlane + c0, d);
            tmem_wait_ld();
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) {
                // (computed for every column and selected afterwards: rows of a warp have different bounds,
                // and a branch per element diverges)
                const float scaled = br * __expf(fminf(gr - g_cum[c0 + i], 0.0f)) * d[i];
                d[i] = c0 + i < bound ? scaled : 0.0f;
            }
            if (row < 64u) {
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q)
                    *reinterpret_cast<float4*>(smem + kPrA + gmat(r, c0 / 4u + q)) = make_float4(d[4 * q], d[4 * q + 1], d[4 * q + 2], d[4 * q + 3]);
            } else {
                store_bf16x16(smem + kPrP, r, c0 / 8u, d);
            }
        }
        tc_fence_before();
    }
    group_sync(bar_id);
    if (tid == 0 && ok) {   // V is not needed before the second MMA group
        mbar_expect_tx(bar_v, 16384u);
        for (uint32_t a = 0; a < 2; ++a)
            tma_load_2d(base + kPrV + a * 8192u, &map_v, bar_v, int(head * kGdnDim + a * 64u), int(row0));
    }

    // ---- T = (I + A)^-1 in f32 (no bf16 enters the solve), by doubling: 16 x 16 diagonal blocks, then the two
    // 32 x 32 diagonal blocks, then the whole.  For a lower block-triangular [[P, 0], [B, Q]] the inverse is
    // [[P^-1, 0], [-Q^-1 B P^-1, Q^-1]], so each level is two products with all the work independent inside a step:
    //   (1) D_b = (I + A_bb)^-1, forward substitution, one column per thread (64 threads);
    //   (2a) X = A[b1, b0] D_b0 for the two pairs (b0, b1) = (0, 1), (2, 3);   (2b) T[b1, b0] = -D_b1 X;
    //   (3a) X = A[32.., ..32] T[..32, ..32];                                   (3b) T[32.., ..32] = -T[32.., 32..] X.
    // Five barrier-to-barrier steps instead of the nine of a sweep over panels of 16 rows (whose steps cost ~ 1 k
    // cycles each whatever the arithmetic in them), and a third of its shared-memory loads.  A thread owns four
    // consecutive rows of one column of a product; the triangular zeros of the left-hand factor of (2b), (3b) bound
    // its loop (uniformly for a warp).
    // Layouts: T (and with it D_b) is built in place as [row group][column][4 rows] (what the scaling pass below
    // reads); left-hand factors are wanted as [4-column group][row][4 columns]: A is stored so, D_1 and the 32 x 32
    // block T[32.., 32..] get a second copy in that form; the X of both levels is [row group][column][4 rows].
    float4* tc4 = reinterpret_cast<float4*>(smem + kPrWs);               // T: float4 (row group q, column j) at q * 64 + j
    float4* dr1 = reinterpret_cast<float4*>(smem + kPrTW);               // D_1 by rows: (column group g, row r) at g * 16 + r            1 KiB
    float4* thr = reinterpret_cast<float4*>(smem + kPrTW + 1024u);       // T[32.., 32..] by rows: (column group g, row r) at g * 32 + r   4 KiB
    float4* x2c = reinterpret_cast<float4*>(smem + kPrTW + 5120u);       // X of (2a): pair s, (row group q, column j) at s * 64 + q * 16 + j  2 KiB
    float4* x3c = reinterpret_cast<float4*>(smem + kPrTW + 7168u);       // X of (3a): (row group q, column j) at q * 32 + j               4 KiB
    if (tid == kPrStoreThread) release_pending();   // (its warp has little to do until the diagonal blocks are done)
    if (ok && tid < 64u) {
        const uint32_t b = tid >> 4, c = tid & 15u;
        float t[16];
#pragma unroll
        for (uint32_t rr = 0; rr < 16; ++rr) {
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (uint32_t q4 = 0; q4 < rr; q4 += 4) {
                const float4 av = *reinterpret_cast<const float4*>(smem + kPrA + gmat(16u * b + rr, 4u * b + q4 / 4u));   // zero at and above the diagonal
                s0 = fmaf(av.x, t[q4], s0);
                if (q4 + 1 < rr) s1 = fmaf(av.y, t[q4 + 1], s1);
                if (q4 + 2 < rr) s0 = fmaf(av.z, t[q4 + 2], s0);
                if (q4 + 3 < rr) s1 = fmaf(av.w, t[q4 + 3], s1);
            }
            t[rr] = (rr == c ? 1.0f : 0.0f) - (s0 + s1);
        }
#pragma unroll
        for (uint32_t g = 0; g < 4; ++g) tc4[(4u * b + g) * 64u + 16u * b + c] = make_float4(t[4 * g], t[4 * g + 1], t[4 * g + 2], t[4 * g + 3]);
        if (b == 1u) {
#pragma unroll
            for (uint32_t rr = 0; rr < 16; ++rr) reinterpret_cast<float*>(dr1 + (c >> 2) * 16u + rr)[c & 3u] = t[rr];
        } else if (b >= 2u) {
            const uint32_t o = (b - 2u) * 16u;   // position of the block inside T[32.., 32..]
#pragma unroll
            for (uint32_t rr = 0; rr < 16; ++rr) reinterpret_cast<float*>(thr + ((o + c) >> 2) * 32u + o + rr)[c & 3u] = t[rr];
        }
    } else if (tid >= 64u) {
        // the zero blocks of T above the diagonal blocks: (row block, column block) = (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
        for (uint32_t e = tid - 64u; e < 6u * 64u; e += 192u) {
            const uint32_t blk = e >> 6, q = (e >> 4) & 3u, col = e & 15u;
            const uint32_t rb = blk < 3u ? 0u : (blk < 5u ? 1u : 2u), cb = blk < 3u ? blk + 1u : (blk < 5u ? blk - 1u : 3u);
            tc4[(4u * rb + q) * 64u + 16u * cb + col] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    group_sync(bar_id);
    {
        auto dot4 = [](const float4& a, const float4& b, float acc) { return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, fmaf(a.x, b.x, acc)))); };
        const float4* a4 = reinterpret_cast<const float4*>(smem + kPrA);   // A: (column group g, row r) at g * 64 + r
        // (2a), (2b): threads 0..127 = (pair s, row group q of the 16, column j of the 16)
        const uint32_t s2 = (tid >> 6) & 1u, q2 = (tid >> 4) & 3u, j2 = tid & 15u, b0 = 2u * s2, b1 = b0 + 1u;
        if (tid < 128u) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (uint32_t g = 0; g < 4u; ++g) {            // (D_b0[k][j] = 0 for k < j, but a start that differs from lane to lane
                                                           // turns the one-address loads of A into gathers: 3.1 -> 2.0 k cycles in (3a))
                const float4 d = tc4[(4u * b0 + g) * 64u + 16u * b0 + j2];
#pragma unroll
                for (uint32_t rr = 0; rr < 4; ++rr) acc[rr] = dot4(a4[(4u * b0 + g) * 64u + 16u * b1 + 4u * q2 + rr], d, acc[rr]);
            }
            x2c[s2 * 64u + q2 * 16u + j2] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        group_sync(bar_id);
        if (tid < 128u) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (uint32_t g = 0; g <= q2; ++g) {           // D_b1[r][k] = 0 for k > r
                const float4 x = x2c[s2 * 64u + g * 16u + j2];
#pragma unroll
                for (uint32_t rr = 0; rr < 4; ++rr)
                    acc[rr] = dot4(s2 == 0u ? dr1[g * 16u + 4u * q2 + rr] : thr[(4u + g) * 32u + 16u + 4u * q2 + rr], x, acc[rr]);
            }
            tc4[(4u * b1 + q2) * 64u + 16u * b0 + j2] = make_float4(-acc[0], -acc[1], -acc[2], -acc[3]);
            if (s2 == 1u) {
#pragma unroll
                for (uint32_t rr = 0; rr < 4; ++rr) reinterpret_cast<float*>(thr + (j2 >> 2) * 32u + 16u + 4u * q2 + rr)[j2 & 3u] = -acc[rr];
            }
        }
        group_sync(bar_id);
        // (3a), (3b): all threads = (row group q of the 32, column j of the 32)
        const uint32_t q3 = tid >> 5, j3 = tid & 31u;
        {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (uint32_t g = 0; g < 8u; ++g) {            // (likewise: the zeros of T above its diagonal are stored zeros)
                const float4 t = tc4[g * 64u + j3];
#pragma unroll
                for (uint32_t rr = 0; rr < 4; ++rr) acc[rr] = dot4(a4[g * 64u + 32u + 4u * q3 + rr], t, acc[rr]);
            }
            x3c[q3 * 32u + j3] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        group_sync(bar_id);
        {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (uint32_t g = 0; g <= q3; ++g) {           // T[32.., 32..][r][k] = 0 for k > r
                const float4 x = x3c[g * 32u + j3];
#pragma unroll
                for (uint32_t rr = 0; rr < 4; ++rr) acc[rr] = dot4(thr[g * 32u + 4u * q3 + rr], x, acc[rr]);
            }
            tc4[(8u + q3) * 64u + j3] = make_float4(-acc[0], -acc[1], -acc[2], -acc[3]);
        }
        group_sync(bar_id);
    }
    if (ok) {   // (everyone is done with the by-rows copies before T_W and T_U are written over them)
        // T scaled by its columns' factors -> the K-major B tiles T_W and T_U (row r, element j).  A thread takes the
        // column pair 2 jp, 2 jp + 1 of eight rows: one packed conversion and one 4-byte store per row and tile.
        const uint32_t jp = tid & 31u, rh = tid >> 5;
        const float b0 = beta_s[2u * jp], b1 = beta_s[2u * jp + 1u], w0 = b0 * e_g[2u * jp], w1 = b1 * e_g[2u * jp + 1u];
        const uint32_t col = (jp & 3u) * 4u, chunk16 = jp >> 2;
#pragma unroll
        for (uint32_t rg = 0; rg < 2; ++rg) {
            const float4 ta = tc4[(2u * rh + rg) * 64u + 2u * jp], tb4 = tc4[(2u * rh + rg) * 64u + 2u * jp + 1u];
            const float ca[4] = {ta.x, ta.y, ta.z, ta.w}, cb[4] = {tb4.x, tb4.y, tb4.z, tb4.w};
#pragma unroll
            for (uint32_t e = 0; e < 4; ++e) {
                const uint32_t at = sw128(8u * rh + 4u * rg + e, chunk16) + col;
                *reinterpret_cast<uint32_t*>(smem + kPrTW + at) = pack_bf2(ca[e] * w0, cb[e] * w1);
                *reinterpret_cast<uint32_t*>(smem + kPrTU + at) = pack_bf2(ca[e] * b0, cb[e] * b1);
            }
        }
    }
    fence_async_smem();
    group_sync(bar_id);

    // ---- MMA b: W^T = K^T T_W^T (columns 64..127), MMA c: U^T = V^T T_U^T (columns 128..191)
    if (tid == 0 && ok) ok = mbar_wait(bar_v, it & 1u, abort_flag);   // (a failure reaches the others at the end of the unit)
    if (tid == 0 && ok) {
        tc_fence_after();
        constexpr uint32_t idesc = instr_desc2(128, 64, true, false);
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks)
            tc_mma(tmem + 64u, smem_desc(base + kPrKQ + ks * 2048u, 16384, 1024), smem_desc(base + kPrTW + ks * 32u, 16, 1024),
                   idesc, ks ? 1u : 0u);
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks)
            tc_mma(tmem + 128u, smem_desc(base + kPrV + ks * 2048u, 8192, 1024), smem_desc(base + kPrTU + ks * 32u, 16, 1024),
                   idesc, ks ? 1u : 0u);
        tc_commit(bar_mma);
    }
    if (ok) ok = mbar_wait(bar_mma, mma_phase & 1u, abort_flag);
    ++mma_phase;
    if (ok) {
        tc_fence_after();
        // passes 0, 1: W^T (columns 64..127) -> W^T and Ws^T tiles; passes 2, 3: U^T (128..191) -> U^T tile
        // (over V) and the Us^T plane image (over T_W, T_U).  This thread's columns: half*32 .. +31.
#pragma unroll 1
        for (uint32_t blk = 0; blk < 4; ++blk) {
            const uint32_t c0 = half * 32u + (blk & 1u) * 16u;
            const bool is_u = blk >= 2u;
            float w[16], ws[16];
            tmem_ld16(tmem + tlane + (is_u ? 128u : 64u) + c0, w);
            tmem_wait_ld();
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) ws[i] = w[i] * s_end[c0 + i];
            store_bf16x16(smem + (is_u ? kPrV : kPrA), row, c0 / 8u, w);
            store_bf16x16(smem + (is_u ? kPrStU : kPrWs), row, c0 / 8u, ws);
        }
        tc_fence_before();
    }
    fence_async_smem();
    group_sync(bar_id);

    // ---- MMA d: M' = Ws^T K (columns 0..127), e: X = W^T P^T (128..191), f: O0^T = U^T P^T (192..255)
    if (tid == 0 && ok) {
        bulk_store(p.planes.u + unit * kUnitU, base + kPrStU, kUnitU);
        bulk_store_commit();
        tc_fence_after();
        constexpr uint32_t idesc_m = instr_desc2(128, 128, false, true);
        constexpr uint32_t idesc_p = instr_desc2(128, 64, false, false);
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks)
            tc_mma(tmem, smem_desc(base + kPrWs + ks * 32u, 16, 1024), smem_desc(base + kPrKQ + ks * 2048u, 16384, 1024),
                   idesc_m, ks ? 1u : 0u);
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks)
            tc_mma(tmem + 128u, smem_desc(base + kPrA + ks * 32u, 16, 1024), smem_desc(base + kPrP + ks * 32u, 16, 1024),
                   idesc_p, ks ? 1u : 0u);
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks)
            tc_mma(tmem + 192u, smem_desc(base + kPrV + ks * 32u, 16, 1024), smem_desc(base + kPrP + ks * 32u, 16, 1024),
                   idesc_p, ks ? 1u : 0u);
        bulk_store_wait_read();     // the Us^T image has left shared memory before anyone passes the barrier: its place takes the O0^T image
        tc_commit(bar_mma);
    }
    if (ok) ok = mbar_wait(bar_mma, mma_phase & 1u, abort_flag);
    ++mma_phase;
    if (ok) {
        tc_fence_after();
        // -M' (this thread: k-columns half*64 .. +63 = tile `half` of the image), then Q~^T and O0^T (columns half*32 .. +31)
#pragma unroll 1
        for (uint32_t blk = 0; blk < 4; ++blk) {
            float v[16];
            tmem_ld16(tmem + tlane + half * 64u + blk * 16u, v);
            tmem_wait_ld();
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) v[i] = -v[i];
            store_bf16x16(smem + kPrStM + half * 16384u, row, blk * 2u, v);
        }
    }
    // The -M' image is half of what the unit sends out: it leaves now, while the other two images are still being
    // made (an SM writes about 32 bytes per cycle towards L2: all 64 KiB at the end of the unit took 3.5 - 4 k
    // cycles to leave shared memory, and the next unit needs that memory 1.2 k cycles into its run).
    fence_async_smem();
    group_sync(bar_id);
    if (tid == kPrStoreThread && ok) {
        bulk_store(p.planes.m + unit * kUnitM, base + kPrStM, kUnitM);
        bulk_store_commit();
    }
    if (ok) {
        const uint8_t* q_tile = smem + kPrKQ + (row >> 6) * 16384u;
        const uint32_t qchunk = (row & 63u) >> 3, qcol = (row & 7u) * 2u;
#pragma unroll 1
        for (uint32_t blk = 4; blk < 8; ++blk) {
            float v[16];
            {
                const bool is_o = blk >= 6u;
                const uint32_t c0 = half * 32u + (blk & 1u) * 16u;
                tmem_ld16(tmem + tlane + (is_o ? 192u : 128u) + c0, v);
                tmem_wait_ld();
                if (!is_o) {
                    // Q~^T row k' = row: e^{G_r} q_r[k'] - X[k'][r]; the Q rows sit at rows 64.. of the [K;Q] tile
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const uint32_t r = c0 + i;
                        const float q = bf2f(*reinterpret_cast<const __nv_bfloat16*>(q_tile + sw128(64u + r, qchunk) + qcol));
                        v[i] = e_g[r] * q - v[i];
                    }
                }
                store_bf16x16(smem + (is_o ? kPrStO : kPrStQ), row, c0 / 8u, v);
            }
        }
        tc_fence_before();
    }
    fence_async_smem();
    group_sync(bar_id);
    if (tid == kPrStoreThread && ok) {
        if (unit32 + unit_stride < p.n_units) issue_kq(unit32 + unit_stride);   // (everyone is past the Q rows)
        // two more copy groups, in the order in which the next unit needs their shared memory back (see the waits there)
        bulk_store(p.planes.o + unit * kUnitO, base + kPrStO, kUnitO);   // over P, T_W
        bulk_store_commit();
        bulk_store(p.planes.q + unit * kUnitQ, base + kPrStQ, kUnitQ);   // over T
        bulk_store_commit();
        unreleased = unit32;
    }
    ok = group_and(bar_id, ok);   // everyone is done with this unit's K and Q tiles; leave the loop together
    }   // units
    if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    group_sync(bar_id);
    if (tid == kPrStoreThread) release_pending();   // the last unit; nothing of this group is in flight when it returns
}

__global__ void __launch_bounds__(kPrThreads, 2)
gdn_tc_prepare_kernel(const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_v,
                      const TcPrepareParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    const uint32_t base = s2u(smem);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kPrBar + 16);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kPrBar + 24);
    if (tid == 0) {
        mbar_init(base + kPrBar, 1);
        mbar_init(base + kPrBar + 8, 1);
        mbar_init(base + kPrBar + 32, 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"(kPrCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    tc_prepare_units(0u, map_qk, map_v, p, smem, tmem, tid, blockIdx.x, gridDim.x, nullptr, 0u);
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) {
            atomicCAS(p.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
            p.status[kStatusDetail] = blockIdx.x;
        }
        __nanosleep(200000);   // let copies still in flight land before the shared memory is released
    }
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPrCols) : "memory");
    }
}

// ---- kernel 2: serial over chunks, one CTA per v-head ------------------------------------------
// Shared memory: a ring of three stages for the operands of the state transition (-M' 32 KiB, Us^T
// 16 KiB, K 16 KiB: released as soon as the two state MMA groups of a chunk have completed) and a
// ring of two for Q~^T (released after the output MMAs).  Tensor memory (512 columns): the state S
// (f32, 128 columns), two buffers of its bf16 copy (64 columns each: two bf16 per 32-bit column, the A
// operand of the MMAs is read from tensor memory), two output accumulators (64 columns each).
constexpr uint32_t kScRingA = 3, kScRingB = 2;
constexpr uint32_t kScStageM = 0, kScStageU = 32768, kScStageK = 49152, kScStageA = 65536;
constexpr uint32_t kScOffB = kScRingA * kScStageA, kScStageB = 16384;
constexpr uint32_t kScBar = kScOffB + kScRingB * kScStageB;
constexpr uint32_t kScSmem = kScBar + 256;
static_assert(kScSmem <= 232448, "shared memory budget");
constexpr uint32_t kScThreads = 320;                 // TMA warp, MMA warp, 4 state warps, 4 output warps
constexpr uint32_t kScCols = 512, kScColS = 0, kScColA = 128, kScColO = 256;
enum : uint32_t { kSbFullA = 0, kSbEmptyA = 3, kSbFullB = 6, kSbEmptyB = 8, kSbConv = 10, kSbState = 11, kSbOut = 12,
                  kSbOutFree = 14, kSbCount = 16 };

struct TcScanParams {
    const float* state_in;
    float* state_out;
    __nv_bfloat16* y;
    TcPlanes planes;
    uint32_t* status;
    uint32_t rows, nchunks;
};

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// D (tensor memory) (+)= A (tensor memory, bf16 pairs per column) x B (shared memory descriptor)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
        : "memory");
}
constexpr uint32_t kScAhead = 4;   // chunks whose plane images are asked into L2 ahead of the shared-memory ring

// Bounded wait until the planes of `unit` are complete (the word carries `epoch`); true at once without flags.
__device__ __forceinline__ bool unit_ready(const uint32_t* ready, uint64_t unit, uint32_t epoch, volatile uint32_t* abort_flag) {
    if (ready == nullptr) return true;
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ready + unit) : "memory");
        if (v == epoch) return true;
        if ((spin & 15u) == 15u) {
            if (*abort_flag) return false;
            const unsigned long long t = now_ns();
            if (t0 == 0) t0 = t;
            if (t - t0 > kWaitLimitNs) {
                *abort_flag = 1u;
                return false;
            }
        }
        __nanosleep(100);
    }
}

__device__ __forceinline__ void tc_scan_init_barriers(uint8_t* smem) {
    const uint32_t bars = s2u(smem) + kScBar;
    for (uint32_t s = 0; s < kScRingA; ++s) {
        mbar_init(bars + 8u * (kSbFullA + s), 1);
        mbar_init(bars + 8u * (kSbEmptyA + s), 1);
    }
    for (uint32_t s = 0; s < 2; ++s) {
        mbar_init(bars + 8u * (kSbFullB + s), 1);
        mbar_init(bars + 8u * (kSbEmptyB + s), 1);
        mbar_init(bars + 8u * (kSbOut + s), 1);
        mbar_init(bars + 8u * (kSbOutFree + s), 128);
    }
    mbar_init(bars + 8u * kSbConv, 128);
    mbar_init(bars + 8u * kSbState, 1);
    *reinterpret_cast<volatile uint32_t*>(smem + kScBar + 8 * kSbCount) = 0u;
}

// One v-head walked by 320 threads (tid = 0..319) that own kScSmem bytes at `smem` (barriers initialised) and
// kScCols columns of tensor memory at `tmem`.  `ready` (or null): see unit_ready.
__device__ __forceinline__ void tc_scan_head(const CUtensorMap& map_qk, const TcScanParams& p, uint8_t* smem, uint32_t tmem,
                                             uint32_t tid, uint32_t head, const uint32_t* ready, uint32_t epoch) {
    const uint32_t warp = tid >> 5, lane = tid & 31u;
    const uint32_t base = s2u(smem);
    const uint32_t bars = base + kScBar;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kScBar + 8 * kSbCount);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };
    const uint32_t qkh = head >> 1;
    const uint32_t nchunks = p.nchunks;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            auto prefetch = [&](uint32_t c) {
                const uint64_t unit = uint64_t(c) * kGdnValueHeads + head;
                bulk_prefetch_l2(p.planes.m + unit * kUnitM, kUnitM);
                bulk_prefetch_l2(p.planes.u + unit * kUnitU, kUnitU);
                bulk_prefetch_l2(p.planes.q + unit * kUnitQ, kUnitQ);
                bulk_prefetch_l2(p.planes.o + unit * kUnitO, kUnitO);
            };
            // (only when the planes are all there before the scan starts: beside the preparation they are not written
            // yet when the scan would ask for them four chunks ahead -- the prefetch then pulled 671 MB of stale lines
            // out of memory per 16 384 rows, and the planes arrive in L2 from their writers anyway: 0.470 -> 0.438 ms)
            const bool ahead = ready == nullptr;
            if (ahead)
                for (uint32_t c = 0; c < min(kScAhead, nchunks); ++c) prefetch(c);
            for (uint32_t c = 0; c < nchunks; ++c) {
                const uint32_t sa = c % kScRingA, ua = c / kScRingA, sb = c & 1u;
                const uint32_t st = base + sa * kScStageA;
                const uint64_t unit = uint64_t(c) * kGdnValueHeads + head;
                if (ahead && c + kScAhead < nchunks) prefetch(c + kScAhead);
                if (ua > 0u && !mbar_wait(bar(kSbEmptyA + sa), (ua - 1u) & 1u, abort_flag)) break;
                if (!unit_ready(ready, unit, epoch, abort_flag)) break;
                if (ready != nullptr) asm volatile("fence.proxy.async;" ::: "memory");   // the planes were written through the bulk-copy engine of another SM
                mbar_expect_tx(bar(kSbFullA + sa), kScStageA);
                bulk_load(st + kScStageM, p.planes.m + unit * kUnitM, kUnitM, bar(kSbFullA + sa));
                bulk_load(st + kScStageU, p.planes.u + unit * kUnitU, kUnitU, bar(kSbFullA + sa));
                tma_load_2d(st + kScStageK, &map_qk, bar(kSbFullA + sa), int(kGdnKOff + qkh * kGdnDim), int(c * kTcChunk));
                tma_load_2d(st + kScStageK + 8192u, &map_qk, bar(kSbFullA + sa), int(kGdnKOff + qkh * kGdnDim + 64u), int(c * kTcChunk));
                if (c >= 2u && !mbar_wait(bar(kSbEmptyB + sb), ((c >> 1) - 1u) & 1u, abort_flag)) break;
                mbar_expect_tx(bar(kSbFullB + sb), kScStageB);
                bulk_load(base + kScOffB + sb * kScStageB, p.planes.q + unit * kUnitQ, kUnitQ, bar(kSbFullB + sb));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc2(128, 128, false, true);
            constexpr uint32_t idesc_o = instr_desc2(128, 64, false, true);
            for (uint32_t c = 0; c < nchunks; ++c) {
                const uint32_t sa = c % kScRingA, ua = c / kScRingA, s = c & 1u;
                const uint32_t st = base + sa * kScStageA, a_s0 = tmem + kScColA + s * 64u;
                if (!mbar_wait(bar(kSbFullA + sa), ua & 1u, abort_flag)) break;
                if (!mbar_wait(bar(kSbConv), c & 1u, abort_flag)) break;   // e^{G_C} S0 and the bf16 copy of S0 are in tensor memory
                tc_fence_after();
                // S += Us^T K
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks)
                    tc_mma(tmem + kScColS, smem_desc(st + kScStageU + ks * 32u, 16, 1024),
                           smem_desc(st + kScStageK + ks * 2048u, 8192, 1024), idesc_s, 1u);
                // S += S0 (-M'): sixteen bf16 of the copy = eight columns per k-step
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks)
                    tc_mma_ts(tmem + kScColS, a_s0 + ks * 8u, smem_desc(st + kScStageM + ks * 2048u, 16384, 1024), idesc_s, 1u);
                tc_commit(bar(kSbState));
                tc_commit(bar(kSbEmptyA + sa));
                // O^T = S0 Q~^T into the output buffer of this chunk's parity
                if (!mbar_wait(bar(kSbFullB + s), (c >> 1) & 1u, abort_flag)) break;
                if (c >= 2u && !mbar_wait(bar(kSbOutFree + s), ((c >> 1) - 1u) & 1u, abort_flag)) break;
                tc_fence_after();
                const uint32_t qb = base + kScOffB + s * kScStageB;
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks)
                    tc_mma_ts(tmem + kScColO + s * 64u, a_s0 + ks * 8u, smem_desc(qb + ks * 2048u, 16384, 1024), idesc_o, ks ? 1u : 0u);
                tc_commit(bar(kSbOut + s));
                tc_commit(bar(kSbEmptyB + s));
            }
        }
    } else if (warp < 6) {
        // ---------------- state warps: thread = v row = tensor-memory lane ----------------
        const uint32_t quarter = warp & 3u, row = quarter * 32u + lane;
        const uint32_t tlane = (quarter * 32u) << 16;
        const float* in_row = p.state_in + (uint64_t(head) * kGdnDim + row) * kGdnDim;
        float* out_row = p.state_out + (uint64_t(head) * kGdnDim + row) * kGdnDim;
        bool ok = true;
        for (uint32_t c = 0; c <= nchunks && ok; ++c) {
            if (c < nchunks && !unit_ready(ready, uint64_t(c) * kGdnValueHeads + head, epoch, abort_flag)) { ok = false; break; }
            const float gamma = c < nchunks ? p.planes.gamma[uint64_t(c) * kGdnValueHeads + head] : 1.0f;
            if (c > 0u) {
                if (!mbar_wait(bar(kSbState), (c - 1u) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
            }
            // the bf16 copy of chunk c goes to buffer c & 1, which the MMAs of chunk c - 2 have left
            if (c >= 2u && c < nchunks && !mbar_wait(bar(kSbOut + (c & 1u)), ((c >> 1) - 1u) & 1u, abort_flag)) { ok = false; break; }
            const uint32_t copy = tmem + tlane + kScColA + (c & 1u) * 64u;
#pragma unroll
            for (uint32_t blk = 0; blk < 4; ++blk) {
                float v[32];
                if (c == 0u) {
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(v + 4 * i) = *reinterpret_cast<const float4*>(in_row + blk * 32u + 4u * i);
                } else {
                    tmem_ld32(tmem + tlane + kScColS + blk * 32u, v);
                    tmem_wait_ld();
                }
                if (c == nchunks) {
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(out_row + blk * 32u + 4u * i) = *reinterpret_cast<const float4*>(v + 4 * i);
                    continue;
                }
                uint32_t packed[16];    // k' = blk*32 + 2i, + 2i + 1 in column blk*16 + i of the copy
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) packed[i] = pack_bf2(v[2 * i], v[2 * i + 1]);
                tmem_st16(copy + blk * 16u, packed);
#pragma unroll
                for (uint32_t i = 0; i < 32; ++i) v[i] *= gamma;
                tmem_st32(tmem + tlane + kScColS + blk * 32u, v);
            }
            if (c == nchunks) break;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(kSbConv));
        }
    } else {
        // ---------------- output warps: thread = v row ----------------
        const uint32_t quarter = warp & 3u, row = quarter * 32u + lane;
        const uint32_t tlane = (quarter * 32u) << 16;
        for (uint32_t c = 0; c < nchunks; ++c) {
            const uint32_t s = c & 1u;
            const uint32_t live_rows = min(kTcChunk, p.rows - c * kTcChunk);
            if (!unit_ready(ready, uint64_t(c) * kGdnValueHeads + head, epoch, abort_flag)) break;
            uint4 o0[8];
            const uint8_t* o_img = p.planes.o + (uint64_t(c) * kGdnValueHeads + head) * kUnitO;   // the swizzled tile image
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) o0[i] = *reinterpret_cast<const uint4*>(o_img + sw128(row, i));
            if (!mbar_wait(bar(kSbOut + s), (c >> 1) & 1u, abort_flag)) break;
            tc_fence_after();
            float v[64];
            tmem_ld32(tmem + tlane + kScColO + s * 64u, v);
            tmem_ld32(tmem + tlane + kScColO + s * 64u + 32u, v + 32);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(kSbOutFree + s));
            __nv_bfloat16* y0 = p.y + uint64_t(c) * kTcChunk * kGdnV + head * kGdnDim + row;
            const __nv_bfloat16* o0h = reinterpret_cast<const __nv_bfloat16*>(o0);
#pragma unroll
            for (uint32_t r = 0; r < 64; ++r)
                if (r < live_rows) y0[uint64_t(r) * kGdnV] = f2bf(v[r] + bf2f(o0h[r]));
        }
    }

}

__global__ void __launch_bounds__(kScThreads, 1)
gdn_tc_scan_kernel(const __grid_constant__ CUtensorMap map_qk, const TcScanParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kScBar + 8 * kSbCount);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kScBar + 8 * kSbCount + 8);
    if (threadIdx.x == 0) {
        tc_scan_init_barriers(smem);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)), "r"(kScCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    tc_scan_head(map_qk, p, smem, tmem, threadIdx.x, blockIdx.x, nullptr, 0u);
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicCAS(p.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
            p.status[kStatusDetail] = blockIdx.x;
        }
        __nanosleep(200000);
        __syncthreads();
    }
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kScCols) : "memory");
    }
}

// ---- both in one launch: the scan of early chunks runs beside the preparation of later ones ---------
// One CTA of 512 threads per SM (a cooperative launch: the scan CTAs wait for words that worker CTAs set, so
// all of them must be resident together).  CTAs 0..31 walk one v-head each (threads 0..319); every other
// CTA is two prepare groups of 256 threads, each with its own half of the shared and tensor memory,
// taking units in chunk order (unit = slot, slot + slots, ...), so the planes of chunk c are complete
// about when the scans get there.  Two launches that wait on each other's flags could not share a GPU
// safely; one launch with roles can.
constexpr uint32_t kFuThreads = 512;
constexpr uint32_t kFuSmem = kScSmem > 2u * kPrSmem ? kScSmem : 2u * kPrSmem;
static_assert(2u * kPrSmem <= 232448 && kPrSmem % 1024u == 64u, "two prepare groups per CTA");
constexpr uint32_t kFuGroupStride = kPrSmem - 64u + 1024u;   // keeps the second group's tiles 1024-byte aligned

struct TcFusedParams {
    TcPrepareParams prep;
    TcScanParams scan;
    uint32_t* ready;
    uint32_t epoch;
};

__global__ void __launch_bounds__(kFuThreads, 1)
gdn_tc_fused_kernel(const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_v,
                    const TcFusedParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint32_t tmem_slot;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    const bool scan_role = blockIdx.x < kGdnValueHeads;
    const uint32_t group = tid >> 8;
    uint8_t* gsmem = smem + group * kFuGroupStride;
    if (scan_role) {
        if (tid == 0) {
            tc_scan_init_barriers(smem);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    } else if ((tid & 255u) == 0u) {
        mbar_init(s2u(gsmem) + kPrBar, 1);
        mbar_init(s2u(gsmem) + kPrBar + 8, 1);
        mbar_init(s2u(gsmem) + kPrBar + 32, 1);
        *reinterpret_cast<volatile uint32_t*>(gsmem + kPrBar + 16) = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool aborted = false;
    if (scan_role) {
        if (tid < kScThreads) tc_scan_head(map_qk, p.scan, smem, tmem, tid, blockIdx.x, p.ready, p.epoch);
    } else {
        const uint32_t slots = (gridDim.x - kGdnValueHeads) * 2u, slot = (blockIdx.x - kGdnValueHeads) * 2u + group;
        tc_prepare_units(1u + group, map_qk, map_v, p.prep, gsmem, tmem + group * kPrCols, tid & 255u, slot, slots,
                         p.ready, p.epoch);
    }
    tc_fence_before();
    __syncthreads();
    aborted = scan_role ? *reinterpret_cast<volatile uint32_t*>(smem + kScBar + 8 * kSbCount) != 0u
                        : (*reinterpret_cast<volatile uint32_t*>(smem + kPrBar + 16) |
                           *reinterpret_cast<volatile uint32_t*>(smem + kFuGroupStride + kPrBar + 16)) != 0u;
    if (aborted) {
        if (tid == 0) {
            atomicCAS(p.scan.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
            p.scan.status[kStatusDetail] = blockIdx.x;
        }
        __nanosleep(200000);
        __syncthreads();
    }
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// 2-D bf16 tensor map {cols, rows} with a {64, box_rows} box and the 128-byte swizzle.
static bool make_map2(CUtensorMap* map, const void* ptr, uint64_t cols, uint64_t rows, uint32_t box_rows) {
    EncodeTiled fn = encode_tiled_entry();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2ull};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

tatara_status launch_gdn_chunked_tc(tatara_ctx* ctx, cudaStream_t stream, const __nv_bfloat16* qk,
                                    const __nv_bfloat16* value, const float* decay, const float* beta,
                                    const float* state_in, __nv_bfloat16* y, float* state_out, uint32_t rows,
                                    void* scratch, uint64_t scratch_bytes) {
    if (scratch == nullptr || !aligned(scratch, 128))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill: the chunked form needs 128-byte aligned scratch");
    if (!aligned(qk, 16) || !aligned(value, 16) || !aligned(state_in, 16) || !aligned(state_out, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill: buffers must be 16-byte aligned");
    if (scratch_bytes < gdn_tc_scratch_bytes(rows))
        return fail(ctx, TATARA_SCRATCH_TOO_SMALL, "gdn_prefill: scratch smaller than tatara_gdn_prefill_scratch_bytes(rows)");
    const uint32_t nchunks = (rows + kTcChunk - 1u) / kTcChunk;
    const uint64_t units = tc_units(rows);
    TcPlanes planes{};
    uint8_t* at = static_cast<uint8_t*>(scratch);
    planes.m = at; at += units * kUnitM;
    planes.u = at; at += units * kUnitU;
    planes.q = at; at += units * kUnitQ;
    planes.o = at; at += units * kUnitO;
    planes.gamma = reinterpret_cast<float*>(at);
    CUtensorMap map_qk, map_v;
    if (!make_map2(&map_qk, qk, kGdnQk, rows, 64) || !make_map2(&map_v, value, kGdnV, rows, 64))
        return fail(ctx, TATARA_CUDA_ERROR, "gdn_prefill: tensor map encoding failed");
    uint32_t* ready = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(planes.gamma) + ((units * 4u + 127u) & ~uint64_t(127)));
    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(gdn_tc_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_tc_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_tc_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFuSmem) != cudaSuccess)
            return check_launch(ctx, "gdn_prefill: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    TcPrepareParams pp{decay, beta, planes, ctx->device_status, rows, uint32_t(units)};
    TcScanParams sp{state_in, state_out, y, planes, ctx->device_status, rows, nchunks};
    // One launch with roles (32 scan CTAs beside the prepare workers) when the device has SMs to spare for
    // workers and the block is long enough for the overlap to matter; else, or if the cooperative launch is
    // refused, prepare and scan as two launches.
    if (ctx->gdn_chunk_form == 0u && ctx->sm_count >= int(kGdnValueHeads) + 32 && nchunks >= 8u) {
        if (cudaMemsetAsync(ready, 0, units * 4u, stream) != cudaSuccess) return check_launch(ctx, "gdn_prefill(ready words)");
        TcFusedParams fp{pp, sp, ready, 1u};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(uint32_t(ctx->sm_count));
        cfg.blockDim = dim3(kFuThreads);
        cfg.dynamicSmemBytes = kFuSmem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, gdn_tc_fused_kernel, map_qk, map_v, fp) == cudaSuccess) {
            ++ctx->launches;
            return TATARA_OK;
        }
        (void)cudaGetLastError();   // not admitted as a cooperative launch (a partitioned device): two launches
    }
    const uint32_t prep_grid = units < 2u * uint32_t(ctx->sm_count) ? uint32_t(units) : 2u * uint32_t(ctx->sm_count);
    gdn_tc_prepare_kernel<<<prep_grid, kPrThreads, kPrSmem, stream>>>(map_qk, map_v, pp);
    tatara_status st = check_launch(ctx, "gdn_prefill(prepare)");
    if (st != TATARA_OK) return st;
    gdn_tc_scan_kernel<<<kGdnValueHeads, kScThreads, kScSmem, stream>>>(map_qk, sp);
    return check_launch(ctx, "gdn_prefill(scan)");
}

} // namespace tb

