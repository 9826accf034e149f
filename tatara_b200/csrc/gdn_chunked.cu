// Chunk-64 (WY / UT transform) evaluation of the Gated DeltaNet recurrence
// (the reference evaluates the same recurrence one step at a time:
// prefill_gdn.metal:137-196; its decode step: gdn.metal:151-171).
//
// Per v-head, with state S [128 v-dim][128 k-dim], a chunk of C = 64 steps and
// G_r = sum_{i<=r} log(decay_i):
//     delta_r = beta_r (v_r - e^{G_r} S0 k_r - sum_{i<r} e^{G_r-G_i} (k_i.k_r) delta_i)
//  => (I + A) Delta = diag(beta) V - diag(beta e^{G}) K S0^T,   A[r,i] = beta_r e^{G_r-G_i} (k_r.k_i), i < r
//  => Delta = U - W S0^T      with (I + A) U = diag(beta) V,  (I + A) W = diag(beta e^{G}) K
//     O     = diag(e^{G}) Q S0^T + P Delta,    P[r,i] = e^{G_r-G_i} (q_r.k_i), i <= r
//     S_C   = e^{G_C} S0 + sum_i e^{G_C-G_i} delta_i k_i^T
// Only decay ratios e^{G_r-G_i} with i <= r appear, so nothing overflows however fast a head
// forgets.  Two kernels:
//   gdn_chunk_prepare_kernel -- independent per (chunk, v-head): K K^T and Q K^T on the tensor
//     cores (mma.sync m16n8k16, bf16 in / f32 out), the two unit-lower-triangular solves by f32
//     forward substitution (one column of W or U per thread), results as bf16 scratch.
//   gdn_chunk_scan_kernel -- the serial part.  One CTA per (32 v-dims, v-head), two warps of 16
//     v-dims each; the state slice stays in f32 mma accumulators for the whole block and is
//     re-packed in registers as the bf16 A operand of the next chunk (accumulator -> A fragment
//     needs no shuffle), so the chunk-to-chunk dependency never leaves the register file.
//     W, Q, K, P and U^T tiles stream through a double-buffered cp.async ring.
#include "common.cuh"

namespace tb {

constexpr uint32_t kChunk = 64;
constexpr uint32_t kWBytes = kChunk * kGdnDim * 2;   // 16 KiB: W [64][128] bf16
constexpr uint32_t kUtBytes = kGdnDim * kChunk * 2;  // 16 KiB: U^T [128][64] bf16
constexpr uint32_t kPBytesC = kChunk * kChunk * 2;   // 8 KiB: P [64][64] bf16
constexpr uint32_t kGFloats = 136;                   // e^{G_r} [64] | e^{G_C-G_r} [64] | e^{G_C} | pad
constexpr uint32_t kChunkScratch = kWBytes + kUtBytes + kPBytesC + kGFloats * 4;

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void cpa16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cpa16z(uint32_t dst, const void* src, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(live ? 16u : 0u) : "memory");
}

// Byte offset of element (row, col) in a swizzled bf16 tile whose rows hold `kCols` elements:
// the 16-byte chunk index is XORed with (row & 7), which makes every ldmatrix phase conflict free.
template <uint32_t kCols>
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) {
    return row * (kCols * 2u) + ((chunk ^ (row & 7u)) << 4);
}

// ---- kernel 1: per (chunk, v-head) ------------------------------------------------------
constexpr uint32_t kPrepSmem = 3u * kChunk * 256u + kChunk * (kChunk + 4u) * 4u + 2u * kChunk * 4u;
__global__ void __launch_bounds__(256)
gdn_chunk_prepare_kernel(const __nv_bfloat16* __restrict__ qk, const __nv_bfloat16* __restrict__ value,
                         const float* __restrict__ decay, const float* __restrict__ beta,
                         uint8_t* __restrict__ scratch, uint32_t rows) {
    extern __shared__ __align__(1024) uint8_t prep_smem[];
    uint8_t* k_tile = prep_smem;
    uint8_t* q_tile = prep_smem + kChunk * 256u;
    uint8_t* v_tile = prep_smem + 2u * kChunk * 256u;
    float (*a_mat)[kChunk + 4] = reinterpret_cast<float (*)[kChunk + 4]>(prep_smem + 3u * kChunk * 256u);
    float* g_cum = reinterpret_cast<float*>(prep_smem + 3u * kChunk * 256u + kChunk * (kChunk + 4u) * 4u);
    float* beta_s = g_cum + kChunk;
    const uint32_t chunk = blockIdx.x, head = blockIdx.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t row0 = chunk * kChunk;
    const uint32_t live_rows = min(kChunk, rows - row0);
    const uint32_t qcol = (head >> 1) * kGdnDim;
    uint8_t* out = scratch + (uint64_t(chunk) * kGdnValueHeads + head) * kChunkScratch;

    // K and Q tiles (rows past the block end read as zero)
    for (uint32_t idx = threadIdx.x; idx < 2u * kChunk * 16u; idx += 256u) {
        const uint32_t which = idx >> 10, rem = idx & 1023u, r = rem >> 4, c = rem & 15u;
        const bool live = r < live_rows;
        const __nv_bfloat16* src = qk + uint64_t(row0 + (live ? r : 0u)) * kGdnQk + (which ? qcol : kGdnKOff + qcol) + c * 8u;
        cpa16z(sm_u32(which ? q_tile : k_tile) + swz<128>(r, c), src, live);
    }
    // this head's V rows (plain row-major tile; read back one column per thread)
    for (uint32_t idx = threadIdx.x; idx < kChunk * 16u; idx += 256u) {
        const uint32_t r = idx >> 4, c = idx & 15u;
        const bool live = r < live_rows;
        cpa16z(sm_u32(v_tile) + r * 256u + c * 16u,
               value + uint64_t(row0 + (live ? r : 0u)) * kGdnV + head * kGdnDim + c * 8u, live);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    if (warp == 0) {
        // inclusive cumulative log-decay over the 64 steps (two values per lane)
        float g0 = 0.0f, g1 = 0.0f;
        const uint32_t r0 = lane * 2u;
        if (r0 < live_rows) g0 = fmaxf(logf(decay[uint64_t(row0 + r0) * kGdnValueHeads + head]), -100.0f);
        if (r0 + 1u < live_rows) g1 = fmaxf(logf(decay[uint64_t(row0 + r0 + 1u) * kGdnValueHeads + head]), -100.0f);
        float pair = g0 + g1, incl = pair;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= uint32_t(off)) incl += up;
        }
        g_cum[r0] = incl - g1;
        g_cum[r0 + 1u] = incl;
        beta_s[r0] = r0 < live_rows ? beta[uint64_t(row0 + r0) * kGdnValueHeads + head] : 0.0f;
        beta_s[r0 + 1u] = r0 + 1u < live_rows ? beta[uint64_t(row0 + r0 + 1u) * kGdnValueHeads + head] : 0.0f;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();

    // warps 0..3: K K^T rows 16w..16w+15; warps 4..7: Q K^T rows 16(w-4)..
    {
        const uint32_t mt = warp & 3u;
        const bool is_q = warp >= 4u;
        const uint32_t a_base = sm_u32(is_q ? q_tile : k_tile), b_base = sm_u32(k_tile);
        const uint32_t j = lane >> 3, r = lane & 7u;
        float acc[8][4];
#pragma unroll
        for (uint32_t nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(a_base + swz<128>(mt * 16u + (j & 1u) * 8u + r, ks * 2u + (j >> 1)), a0, a1, a2, a3);
#pragma unroll
            for (uint32_t np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b_base + swz<128>(np * 16u + (j >> 1) * 8u + r, ks * 2u + (j & 1u)), b0, b1, b2, b3);
                mma16816(acc[2 * np], a0, a1, a2, a3, b0, b1);
                mma16816(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        const uint32_t g = lane >> 2, t = lane & 3u;
        __nv_bfloat16* p_out = reinterpret_cast<__nv_bfloat16*>(out + kWBytes + kUtBytes);
#pragma unroll
        for (uint32_t nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (uint32_t e = 0; e < 4; ++e) {
                const uint32_t row = mt * 16u + g + (e >> 1) * 8u, col = nt * 8u + 2u * t + (e & 1u);
                const float ratio = col <= row ? __expf(g_cum[row] - g_cum[col]) : 0.0f;
                if (is_q) {
                    p_out[row * kChunk + col] = f2bf(ratio * acc[nt][e]);                   // i <= r
                } else {
                    a_mat[row][col] = col < row ? beta_s[row] * ratio * acc[nt][e] : 0.0f;  // i < r
                }
            }
        }
    }
    __syncthreads();

    // forward substitution, one column per thread: threads 0..127 -> W[:, j], 128..255 -> U[:, j]
    {
        const bool is_u = threadIdx.x >= 128u;
        const uint32_t jcol = threadIdx.x & 127u;
        float x[kChunk];
        // right-hand sides first (64 independent loads in flight), then the in-place solve
#pragma unroll
        for (uint32_t r = 0; r < kChunk; ++r) {
            if (is_u) {
                x[r] = bf2f(*reinterpret_cast<const __nv_bfloat16*>(v_tile + r * 256u + jcol * 2u));
            } else {
                x[r] = bf2f(*reinterpret_cast<const __nv_bfloat16*>(k_tile + swz<128>(r, jcol >> 3) + (jcol & 7u) * 2u));
            }
        }
#pragma unroll
        for (uint32_t r = 0; r < kChunk; ++r) {
            const float rhs = is_u ? beta_s[r] * x[r] : beta_s[r] * __expf(g_cum[r]) * x[r];
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (uint32_t i = 0; i < r; i += 4) {
                // A is strictly lower triangular and zero elsewhere, so whole float4 groups are safe
                const float4 a = *reinterpret_cast<const float4*>(&a_mat[r][i]);
                s0 = fmaf(a.x, x[i], s0);
                if (i + 1 < r) s1 = fmaf(a.y, x[i + 1], s1);
                if (i + 2 < r) s2 = fmaf(a.z, x[i + 2], s2);
                if (i + 3 < r) s3 = fmaf(a.w, x[i + 3], s3);
            }
            x[r] = rhs - ((s0 + s1) + (s2 + s3));
        }
        if (is_u) {
            // U^T [128][64]: this thread's column is one contiguous 128-byte row
            uint4* dst = reinterpret_cast<uint4*>(out + kWBytes + jcol * (kChunk * 2u));
#pragma unroll
            for (uint32_t v4 = 0; v4 < 8; ++v4) {
                uint4 w;
                w.x = pack2(x[v4 * 8 + 0], x[v4 * 8 + 1]);
                w.y = pack2(x[v4 * 8 + 2], x[v4 * 8 + 3]);
                w.z = pack2(x[v4 * 8 + 4], x[v4 * 8 + 5]);
                w.w = pack2(x[v4 * 8 + 6], x[v4 * 8 + 7]);
                dst[v4] = w;
            }
        } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out);
#pragma unroll
            for (uint32_t r = 0; r < kChunk; ++r) dst[r * kGdnDim + jcol] = f2bf(x[r]);
        }
    }
    if (threadIdx.x < kChunk) {
        float* gout = reinterpret_cast<float*>(out + kWBytes + kUtBytes + kPBytesC);
        const float g_end = g_cum[kChunk - 1u];
        gout[threadIdx.x] = __expf(g_cum[threadIdx.x]);
        gout[kChunk + threadIdx.x] = __expf(g_end - g_cum[threadIdx.x]);
        if (threadIdx.x == 0) gout[2u * kChunk] = __expf(g_end);
    }
}

// ---- kernel 2: serial over chunks --------------------------------------------------------
// CTA = (32 v-dims, v-head): two groups of four warps.  A group owns 16 v-dims; its state slice
// Z [16][128] is split by k-dim quarter over the four warps (4 accumulator tiles each).  Per chunk:
//   1. every warp multiplies ITS k-dim quarter of Z into all 64 steps (split-K partials of
//      E = Z W^T and OQ = Z Q^T), the partials meet in shared memory;
//   2. warp w sums the four partials for ITS 16 steps, forms Delta^T = U^T - E there, and publishes
//      it (plain and scaled by e^{G_C-G_i}) as bf16;
//   3. every warp reads all of Delta^T as an A operand: O^T quarter += Delta^T P^T (its 16 steps),
//      Z quarter = e^{G_C} Z + (scaled Delta^T) K (its 32 k-dims).
// 56 MMAs per warp per chunk on the dependent chain instead of 224, at the price of two
// 128-thread named barriers.
constexpr uint32_t kScanThreads = 256;
constexpr uint32_t kStW = 0, kStQ = kStW + kWBytes, kStK = kStQ + kWBytes, kStP = kStK + kWBytes,
                   kStU = kStP + kPBytesC, kStG = kStU + 32u * kChunk * 2u, kStageScan = kStG + kGFloats * 4u;
constexpr uint32_t kPartStride = 72u, kDeltaStride = 72u;            // padded rows: no bank conflicts
constexpr uint32_t kPartFloats = 16u * kPartStride;                  // one [16][64] f32 partial
constexpr uint32_t kOffPart = 2u * kStageScan;                       // [group 2][warp 4][E|OQ][16][64] f32
constexpr uint32_t kOffDelta = kOffPart + 2u * 4u * 2u * kPartFloats * 4u;  // [group 2][plain|scaled][16][64] bf16
constexpr uint32_t kOffOut = kOffDelta + 2u * 2u * 16u * kDeltaStride * 2u; // [64 steps][32 v-dims] bf16
constexpr uint32_t kScanSmem = kOffOut + kChunk * 32u * 2u;

__device__ __forceinline__ void scan_issue(uint32_t stage, const uint8_t* chunk_scratch,
                                           const __nv_bfloat16* qk_rows, uint32_t live_rows, uint32_t qcol,
                                           uint32_t slice) {
    const uint32_t tid = threadIdx.x;
    for (uint32_t idx = tid; idx < kChunk * 16u; idx += kScanThreads) {      // W [64][128]
        const uint32_t r = idx >> 4, c = idx & 15u;
        cpa16(stage + kStW + swz<128>(r, c), chunk_scratch + idx * 16u);
    }
    for (uint32_t idx = tid; idx < 2u * kChunk * 16u; idx += kScanThreads) { // Q and K rows of the qk tensor
        const uint32_t which = idx >> 10, rem = idx & 1023u, r = rem >> 4, c = rem & 15u;
        const bool live = r < live_rows;
        const __nv_bfloat16* src = qk_rows + uint64_t(live ? r : 0u) * kGdnQk + (which ? kGdnKOff + qcol : qcol) + c * 8u;
        cpa16z(stage + (which ? kStK : kStQ) + swz<128>(r, c), src, live);
    }
    for (uint32_t idx = tid; idx < kChunk * 8u; idx += kScanThreads) {       // P [64][64]
        const uint32_t r = idx >> 3, c = idx & 7u;
        cpa16(stage + kStP + swz<64>(r, c), chunk_scratch + kWBytes + kUtBytes + idx * 16u);
    }
    for (uint32_t idx = tid; idx < 32u * 8u; idx += kScanThreads)            // U^T rows of this CTA's 32 v-dims
        cpa16(stage + kStU + idx * 16u, chunk_scratch + kWBytes + slice * (32u * kChunk * 2u) + idx * 16u);
    for (uint32_t idx = tid; idx < kGFloats / 4u; idx += kScanThreads)       // decay vectors
        cpa16(stage + kStG + idx * 16u, chunk_scratch + kWBytes + kUtBytes + kPBytesC + idx * 16u);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}

__global__ void __launch_bounds__(kScanThreads, 1)
gdn_chunk_scan_kernel(const __nv_bfloat16* __restrict__ qk, const uint8_t* __restrict__ scratch,
                      const float* __restrict__ state_in, __nv_bfloat16* __restrict__ y,
                      float* __restrict__ state_out, uint32_t rows, uint32_t nchunks) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t slice = blockIdx.x, head = blockIdx.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t group = warp >> 2, wq = warp & 3u;   // v-dim half of the CTA, quarter within the group
    const uint32_t g = lane >> 2, t = lane & 3u, j = lane >> 3, r8 = lane & 7u;
    const uint32_t qcol = (head >> 1) * kGdnDim;
    const uint32_t vrow = slice * 32u + group * 16u;     // first v-dim of this group
    const uint32_t sbase = sm_u32(smem);
    const uint32_t group_bar = 1u + group;
    float* part = reinterpret_cast<float*>(smem + kOffPart) + group * (4u * 2u * kPartFloats);
    __nv_bfloat16* delta = reinterpret_cast<__nv_bfloat16*>(smem + kOffDelta) + group * (2u * 16u * kDeltaStride);
    __nv_bfloat16* ost = reinterpret_cast<__nv_bfloat16*>(smem + kOffOut);

    // this warp's quarter of the state slice: Z[16 v-dims][k-dims 32*wq .. +31] as 4 accumulator tiles
    float z[4][4];
    {
        const float* src = state_in + (uint64_t(head) * kGdnDim + vrow) * kGdnDim + wq * 32u;
#pragma unroll
        for (uint32_t nt = 0; nt < 4; ++nt) {
            const float2 lo = *reinterpret_cast<const float2*>(src + uint64_t(g) * kGdnDim + nt * 8u + 2u * t);
            const float2 hi = *reinterpret_cast<const float2*>(src + uint64_t(g + 8u) * kGdnDim + nt * 8u + 2u * t);
            z[nt][0] = lo.x; z[nt][1] = lo.y; z[nt][2] = hi.x; z[nt][3] = hi.y;
        }
    }
    auto chunk_ptr = [&](uint32_t c) { return scratch + (uint64_t(c) * kGdnValueHeads + head) * kChunkScratch; };
    scan_issue(sbase, chunk_ptr(0), qk, min(kChunk, rows), qcol, slice);

    for (uint32_t c = 0; c < nchunks; ++c) {
        const uint32_t stage = sbase + (c & 1u) * kStageScan;
        const uint8_t* stage_ptr = smem + (c & 1u) * kStageScan;
        if (c + 1u < nchunks) {
            const uint32_t next_rows = min(kChunk, rows - (c + 1u) * kChunk);
            scan_issue(sbase + ((c + 1u) & 1u) * kStageScan, chunk_ptr(c + 1u),
                       qk + uint64_t(c + 1u) * kChunk * kGdnQk, next_rows, qcol, slice);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* gvec = reinterpret_cast<const float*>(stage_ptr + kStG);

        // ---- 1. split-K partials over this warp's 32 k-dims, all 64 steps
        uint32_t za[2][4];
#pragma unroll
        for (uint32_t ks = 0; ks < 2; ++ks) {
            za[ks][0] = pack2(z[2 * ks][0], z[2 * ks][1]);
            za[ks][1] = pack2(z[2 * ks][2], z[2 * ks][3]);
            za[ks][2] = pack2(z[2 * ks + 1][0], z[2 * ks + 1][1]);
            za[ks][3] = pack2(z[2 * ks + 1][2], z[2 * ks + 1][3]);
        }
        float e[8][4], o[8][4];
#pragma unroll
        for (uint32_t nt = 0; nt < 8; ++nt) {
            e[nt][0] = e[nt][1] = e[nt][2] = e[nt][3] = 0.0f;
            o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
        }
#pragma unroll
        for (uint32_t ks = 0; ks < 2; ++ks) {
#pragma unroll
            for (uint32_t np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                const uint32_t off = swz<128>(np * 16u + (j >> 1) * 8u + r8, (wq * 2u + ks) * 2u + (j & 1u));
                ldsm_x4(stage + kStW + off, b0, b1, b2, b3);
                mma16816(e[2 * np], za[ks][0], za[ks][1], za[ks][2], za[ks][3], b0, b1);
                mma16816(e[2 * np + 1], za[ks][0], za[ks][1], za[ks][2], za[ks][3], b2, b3);
                ldsm_x4(stage + kStQ + off, b0, b1, b2, b3);
                mma16816(o[2 * np], za[ks][0], za[ks][1], za[ks][2], za[ks][3], b0, b1);
                mma16816(o[2 * np + 1], za[ks][0], za[ks][1], za[ks][2], za[ks][3], b2, b3);
            }
        }
        {
            float* pe = part + (wq * 2u) * kPartFloats;
            float* po = pe + kPartFloats;
#pragma unroll
            for (uint32_t nt = 0; nt < 8; ++nt) {
                const uint32_t col = nt * 8u + 2u * t;
                *reinterpret_cast<float2*>(pe + g * kPartStride + col) = make_float2(e[nt][0], e[nt][1]);
                *reinterpret_cast<float2*>(pe + (g + 8u) * kPartStride + col) = make_float2(e[nt][2], e[nt][3]);
                *reinterpret_cast<float2*>(po + g * kPartStride + col) = make_float2(o[nt][0], o[nt][1]);
                *reinterpret_cast<float2*>(po + (g + 8u) * kPartStride + col) = make_float2(o[nt][2], o[nt][3]);
            }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");

        // ---- 2. this warp's 16 steps: sum the four partials (warp order), Delta^T, scaled OQ
        float oq[2][4];
        {
            const __nv_bfloat16* ut = reinterpret_cast<const __nv_bfloat16*>(stage_ptr + kStU) + (group * 16u) * kChunk;
#pragma unroll
            for (uint32_t nt = 0; nt < 2; ++nt) {
                const uint32_t col = wq * 16u + nt * 8u + 2u * t;
                float2 elo = make_float2(0.0f, 0.0f), ehi = elo, olo = elo, ohi = elo;
#pragma unroll
                for (uint32_t w = 0; w < 4; ++w) {
                    const float* pe = part + (w * 2u) * kPartFloats;
                    const float* po = pe + kPartFloats;
                    const float2 a = *reinterpret_cast<const float2*>(pe + g * kPartStride + col);
                    const float2 b = *reinterpret_cast<const float2*>(pe + (g + 8u) * kPartStride + col);
                    const float2 cc = *reinterpret_cast<const float2*>(po + g * kPartStride + col);
                    const float2 d = *reinterpret_cast<const float2*>(po + (g + 8u) * kPartStride + col);
                    elo.x += a.x; elo.y += a.y; ehi.x += b.x; ehi.y += b.y;
                    olo.x += cc.x; olo.y += cc.y; ohi.x += d.x; ohi.y += d.y;
                }
                const __nv_bfloat162 ulo = *reinterpret_cast<const __nv_bfloat162*>(ut + g * kChunk + col);
                const __nv_bfloat162 uhi = *reinterpret_cast<const __nv_bfloat162*>(ut + (g + 8u) * kChunk + col);
                const float d0 = bf2f(ulo.x) - elo.x, d1 = bf2f(ulo.y) - elo.y;
                const float d2 = bf2f(uhi.x) - ehi.x, d3 = bf2f(uhi.y) - ehi.y;
                const float gr0 = gvec[col], gr1 = gvec[col + 1u];
                const float gc0 = gvec[kChunk + col], gc1 = gvec[kChunk + col + 1u];
                oq[nt][0] = olo.x * gr0; oq[nt][1] = olo.y * gr1; oq[nt][2] = ohi.x * gr0; oq[nt][3] = ohi.y * gr1;
                *reinterpret_cast<uint32_t*>(delta + g * kDeltaStride + col) = pack2(d0, d1);
                *reinterpret_cast<uint32_t*>(delta + (g + 8u) * kDeltaStride + col) = pack2(d2, d3);
                *reinterpret_cast<uint32_t*>(delta + 16u * kDeltaStride + g * kDeltaStride + col) = pack2(d0 * gc0, d1 * gc1);
                *reinterpret_cast<uint32_t*>(delta + 16u * kDeltaStride + (g + 8u) * kDeltaStride + col) = pack2(d2 * gc0, d3 * gc1);
            }
        }
        asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");

        // ---- 3. all of Delta^T as A fragments; O^T quarter and Z quarter
        uint32_t da[4][4], ds[4][4];
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            const uint32_t col = ks * 16u + 2u * t;
            da[ks][0] = *reinterpret_cast<const uint32_t*>(delta + g * kDeltaStride + col);
            da[ks][1] = *reinterpret_cast<const uint32_t*>(delta + (g + 8u) * kDeltaStride + col);
            da[ks][2] = *reinterpret_cast<const uint32_t*>(delta + g * kDeltaStride + col + 8u);
            da[ks][3] = *reinterpret_cast<const uint32_t*>(delta + (g + 8u) * kDeltaStride + col + 8u);
            ds[ks][0] = *reinterpret_cast<const uint32_t*>(delta + 16u * kDeltaStride + g * kDeltaStride + col);
            ds[ks][1] = *reinterpret_cast<const uint32_t*>(delta + 16u * kDeltaStride + (g + 8u) * kDeltaStride + col);
            ds[ks][2] = *reinterpret_cast<const uint32_t*>(delta + 16u * kDeltaStride + g * kDeltaStride + col + 8u);
            ds[ks][3] = *reinterpret_cast<const uint32_t*>(delta + 16u * kDeltaStride + (g + 8u) * kDeltaStride + col + 8u);
        }
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(stage + kStP + swz<64>(wq * 16u + (j >> 1) * 8u + r8, ks * 2u + (j & 1u)), b0, b1, b2, b3);
            mma16816(oq[0], da[ks][0], da[ks][1], da[ks][2], da[ks][3], b0, b1);
            mma16816(oq[1], da[ks][0], da[ks][1], da[ks][2], da[ks][3], b2, b3);
        }
        const float gend = gvec[2u * kChunk];
#pragma unroll
        for (uint32_t nt = 0; nt < 4; ++nt) {
            z[nt][0] *= gend; z[nt][1] *= gend; z[nt][2] *= gend; z[nt][3] *= gend;
        }
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (uint32_t np = 0; np < 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(stage + kStK + swz<128>(ks * 16u + (j & 1u) * 8u + r8, (wq * 2u + np) * 2u + (j >> 1)), b0, b1, b2, b3);
                mma16816(z[2 * np], ds[ks][0], ds[ks][1], ds[ks][2], ds[ks][3], b0, b1);
                mma16816(z[2 * np + 1], ds[ks][0], ds[ks][1], ds[ks][2], ds[ks][3], b2, b3);
            }
        }
        // outputs: O^T [v-dim][step] -> staging [step][32 v-dims] -> y rows (64 bytes per row)
#pragma unroll
        for (uint32_t nt = 0; nt < 2; ++nt) {
            const uint32_t col = wq * 16u + nt * 8u + 2u * t;
            ost[col * 32u + group * 16u + g] = f2bf(oq[nt][0]);
            ost[(col + 1u) * 32u + group * 16u + g] = f2bf(oq[nt][1]);
            ost[col * 32u + group * 16u + g + 8u] = f2bf(oq[nt][2]);
            ost[(col + 1u) * 32u + group * 16u + g + 8u] = f2bf(oq[nt][3]);
        }
        __syncthreads();
        const uint32_t live_rows = min(kChunk, rows - c * kChunk);
        {
            const uint32_t r = threadIdx.x >> 2, q4 = threadIdx.x & 3u;   // 256 threads = 64 rows x 4 x 16 B
            if (r < live_rows)
                *reinterpret_cast<uint4*>(y + uint64_t(c * kChunk + r) * kGdnV + head * kGdnDim + slice * 32u + q4 * 8u) =
                    *reinterpret_cast<const uint4*>(smem + kOffOut + r * 64u + q4 * 16u);
        }
        __syncthreads(); // the other stage, the exchange buffers and the output staging are free again
    }
    float* dst = state_out + (uint64_t(head) * kGdnDim + vrow) * kGdnDim + wq * 32u;
#pragma unroll
    for (uint32_t nt = 0; nt < 4; ++nt) {
        *reinterpret_cast<float2*>(dst + uint64_t(g) * kGdnDim + nt * 8u + 2u * t) = make_float2(z[nt][0], z[nt][1]);
        *reinterpret_cast<float2*>(dst + uint64_t(g + 8u) * kGdnDim + nt * 8u + 2u * t) = make_float2(z[nt][2], z[nt][3]);
    }
}

uint64_t gdn_chunked_scratch_bytes(uint32_t rows) {
    const uint64_t nchunks = (uint64_t(rows) + kChunk - 1u) / kChunk;
    return nchunks * kGdnValueHeads * kChunkScratch;
}

static tatara_status launch_gdn_chunked_regs(tatara_ctx* ctx, cudaStream_t stream, const __nv_bfloat16* qk,
                                 const __nv_bfloat16* value, const float* decay, const float* beta,
                                 const float* state_in, __nv_bfloat16* y, float* state_out, uint32_t rows,
                                 void* scratch, uint64_t scratch_bytes) {
    if (scratch == nullptr || !aligned(scratch, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "gdn_prefill: the chunked form needs 16-byte aligned scratch");
    if (scratch_bytes < gdn_chunked_scratch_bytes(rows))
        return fail(ctx, TATARA_SCRATCH_TOO_SMALL, "gdn_prefill: scratch smaller than tatara_gdn_prefill_scratch_bytes(rows)");
    const uint32_t nchunks = (rows + kChunk - 1u) / kChunk;
    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem) != cudaSuccess)
            return check_launch(ctx, "gdn_prefill: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    gdn_chunk_prepare_kernel<<<dim3(nchunks, kGdnValueHeads), 256, kPrepSmem, stream>>>(
        qk, value, decay, beta, static_cast<uint8_t*>(scratch), rows);
    tatara_status st = check_launch(ctx, "gdn_prefill(prepare)");
    if (st != TATARA_OK) return st;
    gdn_chunk_scan_kernel<<<dim3(4, kGdnValueHeads), kScanThreads, kScanSmem, stream>>>(
        qk, static_cast<const uint8_t*>(scratch), state_in, y, state_out, rows, nchunks);
    return check_launch(ctx, "gdn_prefill(scan)");
}

uint64_t gdn_tc_scratch_bytes(uint32_t rows);
tatara_status launch_gdn_chunked_tc(tatara_ctx* ctx, cudaStream_t stream, const __nv_bfloat16* qk,
                                    const __nv_bfloat16* value, const float* decay, const float* beta,
                                    const float* state_in, __nv_bfloat16* y, float* state_out, uint32_t rows,
                                    void* scratch, uint64_t scratch_bytes);

// The chunked form has two implementations of the same algebra, chosen by TATARA_POLICY_GDN_CHUNK_FORM:
// 0 (default) the tensor-memory form of gdn_chunked_tc.cu as one launch, 2 the same as two launches,
// 1 the register-resident mma.sync form above.
tatara_status launch_gdn_chunked(tatara_ctx* ctx, cudaStream_t stream, const __nv_bfloat16* qk,
                                 const __nv_bfloat16* value, const float* decay, const float* beta,
                                 const float* state_in, __nv_bfloat16* y, float* state_out, uint32_t rows,
                                 void* scratch, uint64_t scratch_bytes) {
    if (ctx->gdn_chunk_form == 1u)
        return launch_gdn_chunked_regs(ctx, stream, qk, value, decay, beta, state_in, y, state_out, rows, scratch, scratch_bytes);
    return launch_gdn_chunked_tc(ctx, stream, qk, value, decay, beta, state_in, y, state_out, rows, scratch, scratch_bytes);
}

} // namespace tb

// Enough for either form of the chunked evaluation.
extern "C" uint64_t tatara_gdn_prefill_scratch_bytes(uint32_t rows) {
    const uint64_t a = tb::gdn_chunked_scratch_bytes(rows), b = tb::gdn_tc_scratch_bytes(rows);
    return a > b ? a : b;
}
