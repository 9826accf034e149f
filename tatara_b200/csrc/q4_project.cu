// Affine-Q4 (group 64) projections on either side of the attention / Gated DeltaNet layers:
// hidden row -> projection row (attn_project, gdn_project) and gated row -> hidden row
// (out_projection).  Two policies, as in the reference:
//
//   exact row   q4_project_kernel: the reference's per-row sequence (q4_dot.metal:9-42) on CUDA
//               cores, one warp per output column; lane l owns 16 consecutive inputs of each
//               512-column block, nibbles are used in place (mask, no shift) against inputs
//               pre-divided by the nibble's place value, fused multiply-add chains, one
//               adjacent-pairs tree at the end.  A row's bits are the same for any batch size.
//               Bound by the Q4 weight stream (0.5 B per weight) for a few rows, by FMA rate
//               beyond about four rows.
//   tensor unit q4_dequant_kernel once at load time (bf16(q*scale + bias), the staging step of
//               native_dense_qgemm.metal), then dense_project_kernel: a bf16 GEMM with f32
//               accumulation on tcgen05 -- TMA-fed 4-stage ring of 128x64 (input) and 256x64
//               (weight) swizzled tiles, 128x256 accumulators double-buffered in tensor memory so
//               that the epilogue of one tile overlaps the MMAs of the next, persistent CTAs.
#include "tc05.cuh"

namespace tb {

// =========================================================================================
// exact-row policy
// =========================================================================================
constexpr uint32_t kQ4MaxMats = 4;
constexpr uint32_t kQ4Warps = 8;

struct Q4Mat {
    const uint2* words;            // [rows][k/16] (8 bytes = one lane's 16 nibbles of a block)
    const __nv_bfloat16* scales;   // [rows][k/64]
    const __nv_bfloat16* biases;
    uint32_t col_begin, col_end;
};
struct Q4Params {
    const __nv_bfloat16* x;
    __nv_bfloat16* out;
    uint64_t x_stride, out_stride;
    uint32_t n_rows, k, n_cols, n_mats;
    uint32_t* status;   // the context's device status words (time-outs of the bulk-copy form)
    Q4Mat mat[kQ4MaxMats];
};

// float(v) for an integer 0 <= v < 2^23 without a conversion instruction
__device__ __forceinline__ float small_int_to_float(uint32_t v) {
    return __uint_as_float(v | 0x4B000000u) - 8388608.0f;
}

// R input rows and C output columns per warp pass.  A CTA stages its R input rows in shared
// memory once; each warp then walks a flat sequence of (column group, 512-column block) items
// in one rolled loop (a decode call runs a warp through a handful of items only, so a long
// unrolled body would spend the kernel fetching instructions) and requests the next item's
// words and affine constants two items ahead of the arithmetic, across group boundaries too.
template <int R, int C>
__global__ void __launch_bounds__(kQ4Warps * 32) q4_project_kernel(const __grid_constant__ Q4Params p) {
    extern __shared__ uint4 xs[];   // [R][k/8]: row r, 8 inputs per uint4
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row0 = blockIdx.y * R;
    const uint32_t blocks = p.k >> 9, wpr = p.k >> 4, gpr = p.k >> 6, xpr = p.k >> 3;
    // Launched as a programmatic dependent of its predecessor in the stream: the weights do not
    // depend on it, so the first two items are requested at once; the input rows (and the output)
    // are touched only after griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t n_groups = p.n_cols / C;
    const uint32_t nwarps = gridDim.x * kQ4Warps;
    uint32_t g = blockIdx.x * kQ4Warps + (threadIdx.x >> 5);   // group being computed

    // fetch cursor: one item ahead of the arithmetic
    const uint2* fw;
    const unsigned short *fs, *fb;
    uint32_t fg = g, fblock = 0;
    auto locate = [&](uint32_t group) {
        const uint32_t col0 = group * C;
        uint32_t m = 0;
        while (m + 1u < p.n_mats && col0 >= p.mat[m].col_end) ++m;
        const uint32_t local = col0 - p.mat[m].col_begin;
        fw = p.mat[m].words + uint64_t(local) * wpr + lane;
        fs = reinterpret_cast<const unsigned short*>(p.mat[m].scales) + uint64_t(local) * gpr + (lane >> 2);
        fb = reinterpret_cast<const unsigned short*>(p.mat[m].biases) + uint64_t(local) * gpr + (lane >> 2);
    };
    uint2 wd[C], wn[C], wf[C];                 // current item, next, the one after
    uint32_t sd[C], bd[C], sn[C], bn[C], sf[C], bf_[C];
    auto fetch = [&](uint2* w, uint32_t* s, uint32_t* b) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            w[c] = __ldg(fw + uint64_t(c) * wpr + fblock * 32u);
            s[c] = __ldg(fs + uint64_t(c) * gpr + fblock * 8u);
            b[c] = __ldg(fb + uint64_t(c) * gpr + fblock * 8u);
        }
        if (++fblock == blocks) {
            fblock = 0;
            fg += nwarps;
            if (fg < n_groups) locate(fg);
        }
    };
    if (g < n_groups) {
        locate(fg);
        fetch(wd, sd, bd);
        if (fg < n_groups) fetch(wn, sn, bn);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = threadIdx.x; i < R * xpr; i += kQ4Warps * 32u) {
        const uint32_t r = i / xpr, j = i - r * xpr;
        const uint32_t row = min(row0 + r, p.n_rows - 1u);
        xs[i] = *(reinterpret_cast<const uint4*>(p.x + uint64_t(row) * p.x_stride) + j);
    }
    __syncthreads();

    float result[R][C];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < C; ++c) result[r][c] = 0.0f;
    uint32_t b = 0;
#pragma unroll 1
    while (g < n_groups) {
        if (fg < n_groups) fetch(wf, sf, bf_);
        float xv[R][16], sum[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint4 v0 = xs[r * xpr + b * 64u + lane * 2u], v1 = xs[r * xpr + b * 64u + lane * 2u + 1u];
            const uint32_t raw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a0 = __uint_as_float(raw[2 * i] << 16), a1 = __uint_as_float(raw[2 * i] & 0xFFFF0000u);
                const float a2 = __uint_as_float(raw[2 * i + 1] << 16), a3 = __uint_as_float(raw[2 * i + 1] & 0xFFFF0000u);
                s = __fadd_rn(s, __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3));
                xv[r][4 * i] = a0;
                xv[r][4 * i + 1] = __fmul_rn(a1, 0.0625f);           // exact: a1 / 16
                xv[r][4 * i + 2] = __fmul_rn(a2, 0.00390625f);       // a2 / 256
                xv[r][4 * i + 3] = __fmul_rn(a3, 0.000244140625f);   // a3 / 4096
            }
            sum[r] = s;
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const uint32_t half[4] = {wd[c].x & 0xFFFFu, wd[c].x >> 16, wd[c].y & 0xFFFFu, wd[c].y >> 16};
            const float scale = __uint_as_float(sd[c] << 16), bias = __uint_as_float(bd[c] << 16);
            float wq[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                wq[4 * i] = small_int_to_float(half[i] & 0x000Fu);
                wq[4 * i + 1] = small_int_to_float(half[i] & 0x00F0u);
                wq[4 * i + 2] = small_int_to_float(half[i] & 0x0F00u);
                wq[4 * i + 3] = small_int_to_float(half[i] & 0xF000u);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float quant = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    quant = __fmaf_rn(xv[r][4 * i + 3], wq[4 * i + 3],
                                      __fmaf_rn(xv[r][4 * i + 2], wq[4 * i + 2],
                                                __fmaf_rn(xv[r][4 * i + 1], wq[4 * i + 1],
                                                          __fmaf_rn(xv[r][4 * i], wq[4 * i], quant))));
                result[r][c] = __fmaf_rn(sum[r], bias, __fmaf_rn(scale, quant, result[r][c]));
            }
        }
        if (++b == blocks) {
            // adjacent-pairs tree per (row, column); lane c keeps column c and stores it
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float keep = 0.0f;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const float total = warp_sum(result[r][c]);
                    if (lane == uint32_t(c)) keep = total;
                    result[r][c] = 0.0f;
                }
                if (lane < uint32_t(C) && row0 + uint32_t(r) < p.n_rows)
                    p.out[uint64_t(row0 + r) * p.out_stride + g * C + lane] = f2bf(keep);
            }
            b = 0;
            g += nwarps;
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
            wd[c] = wn[c];
            sd[c] = sn[c];
            bd[c] = bn[c];
            wn[c] = wf[c];
            sn[c] = sf[c];
            bn[c] = bf_[c];
        }
    }
}

// The same arithmetic with the weights brought in by the copy engine.  The rolled loop above keeps two
// items (one 512-input block of a column group) in flight per warp, so a warp that owns one column
// group of a 4096-input matrix walks its eight blocks at two blocks per trip to memory: 0.67 us per
// block, 5.4 us for the single-row out projection whose whole weight stream is 0.7 us of HBM time.
// Here lane 0 of each warp asks for the WHOLE column group at once -- C rows of words, of scales and
// of biases, each contiguous, three cp.async.bulk copies completing on one mbarrier -- and for the
// warp's next group into a second buffer, before the dependency wait: every byte of the matrix is
// in flight from the start.  The pre-divided inputs and the block sums are computed once per CTA into
// shared memory (the values and the order of the per-warp code above), and the block loop reads
// everything from shared memory.  Same chains, same trees: bit-identical to q4_project_kernel.
struct Q4BulkLayout {
    uint32_t x_bytes, group_bytes, words_bytes, affine_bytes, bars_off, total;
};
__host__ __device__ inline Q4BulkLayout q4_bulk_layout(uint32_t rows, uint32_t cols, uint32_t k) {
    Q4BulkLayout l;
    l.x_bytes = rows * (k * 4u + (k >> 9) * 128u);          // [R][blocks][4][32] float4, then [R][blocks][32] sums
    l.words_bytes = cols * (k >> 1);
    l.affine_bytes = cols * (k >> 5);                       // one of scales / biases
    l.group_bytes = l.words_bytes + 2u * l.affine_bytes;
    l.bars_off = l.x_bytes + kQ4Warps * 2u * l.group_bytes;
    l.total = l.bars_off + kQ4Warps * 16u + 16u;
    return l;
}
__device__ __forceinline__ void q4_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int R, int C>
__global__ void __launch_bounds__(kQ4Warps * 32) q4_project_bulk_kernel(const __grid_constant__ Q4Params p) {
    extern __shared__ __align__(128) uint8_t q4s[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row0 = blockIdx.y * R;
    const uint32_t blocks = p.k >> 9, wpr = p.k >> 4, gpr = p.k >> 6;
    const Q4BulkLayout lay = q4_bulk_layout(R, C, p.k);
    float4* xf = reinterpret_cast<float4*>(q4s);
    float* xsum = reinterpret_cast<float*>(q4s + R * p.k * 4u);
    uint8_t* wbuf = q4s + lay.x_bytes + warp * 2u * lay.group_bytes;
    const uint32_t bars = s2u(q4s + lay.bars_off) + warp * 16u;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(q4s + lay.bars_off + kQ4Warps * 16u);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t n_groups = p.n_cols / C;
    const uint32_t nwarps = gridDim.x * kQ4Warps;
    uint32_t g = blockIdx.x * kQ4Warps + warp;
    // lane 0: the three copies of one column group into buffer `buf`
    auto request = [&](uint32_t group, uint32_t buf) {
        const uint32_t col0 = group * C;
        uint32_t m = 0;
        while (m + 1u < p.n_mats && col0 >= p.mat[m].col_end) ++m;
        const uint32_t local = col0 - p.mat[m].col_begin;
        const uint32_t dst = s2u(wbuf + buf * lay.group_bytes), bar = bars + 8u * buf;
        mbar_expect_tx(bar, lay.group_bytes);
        q4_bulk_load(dst, p.mat[m].words + uint64_t(local) * wpr, lay.words_bytes, bar);
        q4_bulk_load(dst + lay.words_bytes, p.mat[m].scales + uint64_t(local) * gpr, lay.affine_bytes, bar);
        q4_bulk_load(dst + lay.words_bytes + lay.affine_bytes, p.mat[m].biases + uint64_t(local) * gpr,
                     lay.affine_bytes, bar);
    };
    if (threadIdx.x == 0) *abort_flag = 0u;   // read only after the barrier below
    if (lane == 0) {
        mbar_init(bars, 1);
        mbar_init(bars + 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (g < n_groups) request(g, 0);
        if (g + nwarps < n_groups) request(g + nwarps, 1);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // inputs: (row, block, lane) -> this lane's 16 values of the block, pre-divided, and their sum
    for (uint32_t i = threadIdx.x; i < R * blocks * 32u; i += kQ4Warps * 32u) {
        const uint32_t l = i & 31u, rb = i >> 5, r = rb / blocks, b = rb - r * blocks;
        const uint32_t row = min(row0 + r, p.n_rows - 1u);
        const uint4* src = reinterpret_cast<const uint4*>(p.x + uint64_t(row) * p.x_stride) + b * 64u + l * 2u;
        const uint4 v0 = src[0], v1 = src[1];
        const uint32_t raw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float s = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float a0 = __uint_as_float(raw[2 * q] << 16), a1 = __uint_as_float(raw[2 * q] & 0xFFFF0000u);
            const float a2 = __uint_as_float(raw[2 * q + 1] << 16), a3 = __uint_as_float(raw[2 * q + 1] & 0xFFFF0000u);
            s = __fadd_rn(s, __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3));
            xf[(rb * 4u + q) * 32u + l] = make_float4(a0, __fmul_rn(a1, 0.0625f), __fmul_rn(a2, 0.00390625f),
                                                      __fmul_rn(a3, 0.000244140625f));
        }
        xsum[rb * 32u + l] = s;
    }
    __syncthreads();

    bool ok = true;
    uint32_t buf = 0, phase = 0;   // bit b of `phase`: parity of buffer b's next completion
#pragma unroll 1
    while (g < n_groups) {
        __syncwarp();
        if (ok) ok = mbar_wait(bars + 8u * buf, (phase >> buf) & 1u, abort_flag);
        const uint8_t* gb = wbuf + buf * lay.group_bytes;
        const unsigned short* gs = reinterpret_cast<const unsigned short*>(gb + lay.words_bytes);
        const unsigned short* gbias = reinterpret_cast<const unsigned short*>(gb + lay.words_bytes + lay.affine_bytes);
        float result[R][C];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < C; ++c) result[r][c] = 0.0f;
#pragma unroll 1
        for (uint32_t b = 0; b < blocks; ++b) {
            float xv[R][16], sum[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 v = xf[((r * blocks + b) * 4u + q) * 32u + lane];
                    xv[r][4 * q] = v.x; xv[r][4 * q + 1] = v.y; xv[r][4 * q + 2] = v.z; xv[r][4 * q + 3] = v.w;
                }
                sum[r] = xsum[(r * blocks + b) * 32u + lane];
            }
            // Columns in PAIRS: every multiply-add of the chain is one packed fma.rn.f32x2 on {column c,
            // column c+1} against the same input (each component rounds as the scalar fma, so the bits
            // are those of the single-column chain), and the nibble -> float subtraction is packed too.
            const float2 magic = make_float2(-8388608.0f, -8388608.0f);
#pragma unroll
            for (int c = 0; c < C; c += 2) {
                const uint2 wa = *reinterpret_cast<const uint2*>(gb + uint32_t(c) * (p.k >> 1) + b * 256u + lane * 8u);
                const uint2 wb = *reinterpret_cast<const uint2*>(gb + uint32_t(c + 1) * (p.k >> 1) + b * 256u + lane * 8u);
                const uint32_t ha[4] = {wa.x & 0xFFFFu, wa.x >> 16, wa.y & 0xFFFFu, wa.y >> 16};
                const uint32_t hb[4] = {wb.x & 0xFFFFu, wb.x >> 16, wb.y & 0xFFFFu, wb.y >> 16};
                const uint32_t gi = b * 8u + (lane >> 2);
                const float2 scale = make_float2(__uint_as_float(uint32_t(gs[uint32_t(c) * gpr + gi]) << 16),
                                                 __uint_as_float(uint32_t(gs[uint32_t(c + 1) * gpr + gi]) << 16));
                const float2 bias = make_float2(__uint_as_float(uint32_t(gbias[uint32_t(c) * gpr + gi]) << 16),
                                                __uint_as_float(uint32_t(gbias[uint32_t(c + 1) * gpr + gi]) << 16));
                float2 quant[R];
#pragma unroll
                for (int r = 0; r < R; ++r) quant[r] = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 q0 = __fadd2_rn(make_float2(__uint_as_float((ha[i] & 0x000Fu) | 0x4B000000u),
                                                             __uint_as_float((hb[i] & 0x000Fu) | 0x4B000000u)), magic);
                    const float2 q1 = __fadd2_rn(make_float2(__uint_as_float((ha[i] & 0x00F0u) | 0x4B000000u),
                                                             __uint_as_float((hb[i] & 0x00F0u) | 0x4B000000u)), magic);
                    const float2 q2 = __fadd2_rn(make_float2(__uint_as_float((ha[i] & 0x0F00u) | 0x4B000000u),
                                                             __uint_as_float((hb[i] & 0x0F00u) | 0x4B000000u)), magic);
                    const float2 q3 = __fadd2_rn(make_float2(__uint_as_float((ha[i] & 0xF000u) | 0x4B000000u),
                                                             __uint_as_float((hb[i] & 0xF000u) | 0x4B000000u)), magic);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        quant[r] = __ffma2_rn(make_float2(xv[r][4 * i], xv[r][4 * i]), q0, quant[r]);
                        quant[r] = __ffma2_rn(make_float2(xv[r][4 * i + 1], xv[r][4 * i + 1]), q1, quant[r]);
                        quant[r] = __ffma2_rn(make_float2(xv[r][4 * i + 2], xv[r][4 * i + 2]), q2, quant[r]);
                        quant[r] = __ffma2_rn(make_float2(xv[r][4 * i + 3], xv[r][4 * i + 3]), q3, quant[r]);
                    }
                }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float2 acc = __ffma2_rn(make_float2(sum[r], sum[r]), bias,
                                                  __ffma2_rn(scale, quant[r], make_float2(result[r][c], result[r][c + 1])));
                    result[r][c] = acc.x;
                    result[r][c + 1] = acc.y;
                }
            }
        }
        // adjacent-pairs tree per (row, column); lane c keeps column c and stores it
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float keep = 0.0f;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const float total = warp_sum(result[r][c]);
                if (lane == uint32_t(c)) keep = total;
            }
            if (ok && lane < uint32_t(C) && row0 + uint32_t(r) < p.n_rows)
                p.out[uint64_t(row0 + r) * p.out_stride + g * C + lane] = f2bf(keep);
        }
        // the buffer is read: it takes the group two rounds ahead
        __syncwarp();
        if (lane == 0 && ok && g + 2u * nwarps < n_groups) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            request(g + 2u * nwarps, buf);
        }
        phase ^= 1u << buf;
        buf ^= 1u;
        g += nwarps;
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        atomicCAS(p.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
        p.status[kStatusDetail] = blockIdx.x;
        __nanosleep(200000);   // let copies still in flight land before the shared memory is released
    }
}

// The inputs of 2 * n_pairs rows as row pairs in shared memory: float4 (pair, block, i4, lane) =
// {x0[2 i4], x1[2 i4], x0[2 i4 + 1], x1[2 i4 + 1]} of the lane's 16 inputs of the block, each already divided by
// the weight of its nibble position inside the half-word (1, 16, 256, 4096: exact), and the sums of the 16 raw
// inputs per (pair, block, lane).  One item = both rows of a pair at one (block, lane): whole float4 stores
// (the two rows as separate items wrote every other word: four wavefronts per 32-bit store).
__device__ __forceinline__ void stage_row_pairs(const Q4Params& p, uint32_t row0, uint32_t n_pairs, uint32_t blocks,
                                                float4* xs4, float2* sum2, uint32_t tid, uint32_t n_threads) {
    for (uint32_t item = tid; item < n_pairs * blocks * 32u; item += n_threads) {
        const uint32_t l = item & 31u, b = (item >> 5) % blocks, rp = item / (32u * blocks);
        const uint32_t r0 = min(row0 + 2u * rp, p.n_rows - 1u), r1 = min(row0 + 2u * rp + 1u, p.n_rows - 1u);
        const uint4* xp0 = reinterpret_cast<const uint4*>(p.x + uint64_t(r0) * p.x_stride + b * 512u + l * 16u);
        const uint4* xp1 = reinterpret_cast<const uint4*>(p.x + uint64_t(r1) * p.x_stride + b * 512u + l * 16u);
        const uint4 u0 = xp0[0], u1 = xp0[1], v0 = xp1[0], v1 = xp1[1];
        const uint32_t raw0[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        const uint32_t raw1[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float4* dst = xs4 + (rp * blocks + b) * 256u + l;
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a0 = __uint_as_float(raw0[2 * i] << 16), a1 = __uint_as_float(raw0[2 * i] & 0xFFFF0000u);
            const float a2 = __uint_as_float(raw0[2 * i + 1] << 16), a3 = __uint_as_float(raw0[2 * i + 1] & 0xFFFF0000u);
            const float c0 = __uint_as_float(raw1[2 * i] << 16), c1 = __uint_as_float(raw1[2 * i] & 0xFFFF0000u);
            const float c2 = __uint_as_float(raw1[2 * i + 1] << 16), c3 = __uint_as_float(raw1[2 * i + 1] & 0xFFFF0000u);
            s0 = __fadd_rn(s0, __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3));
            s1 = __fadd_rn(s1, __fadd_rn(__fadd_rn(__fadd_rn(c0, c1), c2), c3));
            dst[(2 * i) * 32u] = make_float4(a0, c0, __fmul_rn(a1, 0.0625f), __fmul_rn(c1, 0.0625f));
            dst[(2 * i + 1) * 32u] = make_float4(__fmul_rn(a2, 0.00390625f), __fmul_rn(c2, 0.00390625f),
                                                 __fmul_rn(a3, 0.000244140625f), __fmul_rn(c3, 0.000244140625f));
        }
        sum2[(rp * blocks + b) * 32u + l] = make_float2(s0, s1);
    }
}

// Batched form for more than two rows: 2*RP rows per pass, rows taken in PAIRS so that every
// multiply-add of the chain is one packed fma.rn.f32x2 (sm_100): the pair {row 2p, row 2p+1}
// shares the decoded nibble and each component keeps the scalar kernel's exact sequence
// (per-component rounding of fma.rn.f32x2 is that of fma.rn.f32), so a row's bits are still
// those of the single-row chain.  The pre-divided inputs and their block sums are computed ONCE
// per CTA into shared memory as row pairs ([pair][block][i/2][lane] -> {x0[i], x1[i], x0[i+1],
// x1[i+1]}, one conflict-free LDS.128 per two inputs) instead of once per warp and block.
template <int RP, int C>
__global__ void __launch_bounds__(kQ4Warps * 32, 1) q4_project_pairs_kernel(const __grid_constant__ Q4Params p) {
    extern __shared__ float4 xs4[];   // [RP][blocks][8][32] float4, then the sums [RP][blocks][32] float2
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row0 = blockIdx.y * (2 * RP);
    const uint32_t blocks = p.k >> 9, wpr = p.k >> 4, gpr = p.k >> 6;
    float2* sum2 = reinterpret_cast<float2*>(xs4 + RP * blocks * 256u);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t n_groups = p.n_cols / C;
    const uint32_t nwarps = gridDim.x * kQ4Warps;
    uint32_t g = blockIdx.x * kQ4Warps + (threadIdx.x >> 5);

    const uint2* fw;
    const unsigned short *fs, *fb;
    uint32_t fg = g, fblock = 0;
    auto locate = [&](uint32_t group) {
        const uint32_t col0 = group * C;
        uint32_t m = 0;
        while (m + 1u < p.n_mats && col0 >= p.mat[m].col_end) ++m;
        const uint32_t local = col0 - p.mat[m].col_begin;
        fw = p.mat[m].words + uint64_t(local) * wpr + lane;
        fs = reinterpret_cast<const unsigned short*>(p.mat[m].scales) + uint64_t(local) * gpr + (lane >> 2);
        fb = reinterpret_cast<const unsigned short*>(p.mat[m].biases) + uint64_t(local) * gpr + (lane >> 2);
    };
    // three items of words and affine constants (scale bits << 16 | bias bits) in registers:
    // the one being used and the two behind it already requested
    uint2 wd[C], wn[C], wf[C];
    uint32_t ad[C], an[C], af[C];
    auto fetch = [&](uint2* w, uint32_t* a) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            w[c] = __ldg(fw + uint64_t(c) * wpr + fblock * 32u);
            a[c] = (uint32_t(__ldg(fs + uint64_t(c) * gpr + fblock * 8u)) << 16) |
                   uint32_t(__ldg(fb + uint64_t(c) * gpr + fblock * 8u));
        }
        if (++fblock == blocks) {
            fblock = 0;
            fg += nwarps;
            if (fg < n_groups) locate(fg);
        }
    };
    if (g < n_groups) {
        locate(fg);
        fetch(wd, ad);
        if (fg < n_groups) fetch(wn, an);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stage_row_pairs(p, row0, RP, blocks, xs4, sum2, threadIdx.x, kQ4Warps * 32u);
    __syncthreads();
    if (g >= n_groups) return;

    float2 result[RP][C];
#pragma unroll
    for (int rp = 0; rp < RP; ++rp)
#pragma unroll
        for (int c = 0; c < C; ++c) result[rp][c] = make_float2(0.0f, 0.0f);
    uint32_t b = 0;
    const float2 magic = make_float2(-8388608.0f, -8388608.0f);
#pragma unroll 1
    while (g < n_groups) {
        if (fg < n_groups) fetch(wf, af);
        float4 xv[RP][8];
        float2 sum[RP];
#pragma unroll
        for (int rp = 0; rp < RP; ++rp) {
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[rp][i] = xs4[((rp * blocks + b) * 8u + i) * 32u + lane];
            sum[rp] = sum2[(rp * blocks + b) * 32u + lane];
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const uint32_t half[4] = {wd[c].x & 0xFFFFu, wd[c].x >> 16, wd[c].y & 0xFFFFu, wd[c].y >> 16};
            const float scale = __uint_as_float(ad[c] & 0xFFFF0000u), bias = __uint_as_float(ad[c] << 16);
            float2 quant[RP];
#pragma unroll
            for (int rp = 0; rp < RP; ++rp) quant[rp] = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // the four nibbles of half-word i, each as {w, w}; inputs 4i .. 4i+3 are xv[.][2i].xy, .zw, xv[.][2i+1].xy, .zw
                const float w0 = __uint_as_float((half[i] & 0x000Fu) | 0x4B000000u), w1 = __uint_as_float((half[i] & 0x00F0u) | 0x4B000000u);
                const float w2 = __uint_as_float((half[i] & 0x0F00u) | 0x4B000000u), w3 = __uint_as_float((half[i] & 0xF000u) | 0x4B000000u);
                const float2 q0 = __fadd2_rn(make_float2(w0, w0), magic), q1 = __fadd2_rn(make_float2(w1, w1), magic);
                const float2 q2 = __fadd2_rn(make_float2(w2, w2), magic), q3 = __fadd2_rn(make_float2(w3, w3), magic);
#pragma unroll
                for (int rp = 0; rp < RP; ++rp) {
                    const float4 lo = xv[rp][2 * i], hi = xv[rp][2 * i + 1];
                    quant[rp] = __ffma2_rn(make_float2(lo.x, lo.y), q0, quant[rp]);
                    quant[rp] = __ffma2_rn(make_float2(lo.z, lo.w), q1, quant[rp]);
                    quant[rp] = __ffma2_rn(make_float2(hi.x, hi.y), q2, quant[rp]);
                    quant[rp] = __ffma2_rn(make_float2(hi.z, hi.w), q3, quant[rp]);
                }
            }
#pragma unroll
            for (int rp = 0; rp < RP; ++rp)
                result[rp][c] = __ffma2_rn(sum[rp], make_float2(bias, bias),
                                           __ffma2_rn(make_float2(scale, scale), quant[rp], result[rp][c]));
        }
        if (++b == blocks) {
#pragma unroll
            for (int rp = 0; rp < RP; ++rp) {
                float keep0 = 0.0f, keep1 = 0.0f;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const float t0 = warp_sum(result[rp][c].x), t1 = warp_sum(result[rp][c].y);
                    if (lane == uint32_t(c)) {
                        keep0 = t0;
                        keep1 = t1;
                    }
                    result[rp][c] = make_float2(0.0f, 0.0f);
                }
                const uint32_t r0 = row0 + 2u * rp;
                if (lane < uint32_t(C)) {
                    if (r0 < p.n_rows) p.out[uint64_t(r0) * p.out_stride + g * C + lane] = f2bf(keep0);
                    if (r0 + 1u < p.n_rows) p.out[uint64_t(r0 + 1u) * p.out_stride + g * C + lane] = f2bf(keep1);
                }
            }
            b = 0;
            g += nwarps;
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
            wd[c] = wn[c];
            ad[c] = an[c];
            wn[c] = wf[c];
            an[c] = af[c];
        }
    }
}

// The row-pair kernel with the weights brought in by the copy engine (whole column groups, two buffers per
// warp, asked for before the dependency wait: see q4_project_bulk_kernel); the arithmetic is the row-pair
// kernel's, so are the bits.
template <int RP, int C, int W, int NB>
__global__ void __launch_bounds__(W * 32, 1) q4_project_pairs_bulk_kernel(const __grid_constant__ Q4Params p) {
    extern __shared__ float4 xs4[];   // [RP][blocks][8][32] float4, the sums [RP][blocks][32] float2, then the weight buffers
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t row0 = blockIdx.y * (2 * RP);
    const uint32_t blocks = p.k >> 9, wpr = p.k >> 4, gpr = p.k >> 6;
    float2* sum2 = reinterpret_cast<float2*>(xs4 + RP * blocks * 256u);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t n_groups = p.n_cols / C;
    const uint32_t nwarps = gridDim.x * uint32_t(W);
    uint32_t g = blockIdx.x * uint32_t(W) + warp;

    const Q4BulkLayout lay = q4_bulk_layout(1, C, p.k);      // (group geometry only; the inputs are laid out below)
    const uint32_t x_bytes = RP * blocks * (256u * 16u + 32u * 8u);
    uint8_t* smem_bytes = reinterpret_cast<uint8_t*>(xs4);
    uint8_t* wbuf = smem_bytes + x_bytes + warp * uint32_t(NB) * lay.group_bytes;   // NB buffers per warp
    const uint32_t bars = s2u(smem_bytes + x_bytes + uint32_t(W) * uint32_t(NB) * lay.group_bytes) + warp * 16u;
    volatile uint32_t* abort_flag =
        reinterpret_cast<volatile uint32_t*>(smem_bytes + x_bytes + uint32_t(W) * uint32_t(NB) * lay.group_bytes + uint32_t(W) * 16u);
    // lane 0: the three copies of one column group into buffer `buf` (see q4_project_bulk_kernel)
    auto request = [&](uint32_t group, uint32_t buf) {
        const uint32_t col0 = group * C;
        uint32_t m = 0;
        while (m + 1u < p.n_mats && col0 >= p.mat[m].col_end) ++m;
        const uint32_t local = col0 - p.mat[m].col_begin;
        const uint32_t dst = s2u(wbuf + buf * lay.group_bytes), bar = bars + 8u * buf;
        mbar_expect_tx(bar, lay.group_bytes);
        q4_bulk_load(dst, p.mat[m].words + uint64_t(local) * wpr, lay.words_bytes, bar);
        q4_bulk_load(dst + lay.words_bytes, p.mat[m].scales + uint64_t(local) * gpr, lay.affine_bytes, bar);
        q4_bulk_load(dst + lay.words_bytes + lay.affine_bytes, p.mat[m].biases + uint64_t(local) * gpr,
                     lay.affine_bytes, bar);
    };
    if (threadIdx.x == 0) *abort_flag = 0u;   // read only after the barrier below
    if (lane == 0) {
        mbar_init(bars, 1);
        mbar_init(bars + 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (g < n_groups) request(g, 0);
        if (NB > 1 && g + nwarps < n_groups) request(g + nwarps, 1);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stage_row_pairs(p, row0, RP, blocks, xs4, sum2, threadIdx.x, uint32_t(W) * 32u);
    __syncthreads();

    float2 result[RP][C];
#pragma unroll
    for (int rp = 0; rp < RP; ++rp)
#pragma unroll
        for (int c = 0; c < C; ++c) result[rp][c] = make_float2(0.0f, 0.0f);
    const float2 magic = make_float2(-8388608.0f, -8388608.0f);
    bool ok = true;
    uint32_t buf = 0, phase = 0;
#pragma unroll 1
    while (g < n_groups) {
        __syncwarp();
        if (ok) ok = mbar_wait(bars + 8u * buf, (phase >> buf) & 1u, abort_flag);
        const uint8_t* gb = wbuf + buf * lay.group_bytes;
        const unsigned short* gs = reinterpret_cast<const unsigned short*>(gb + lay.words_bytes);
        const unsigned short* gbias = reinterpret_cast<const unsigned short*>(gb + lay.words_bytes + lay.affine_bytes);
#pragma unroll 2
      for (uint32_t b = 0; b < blocks; ++b) {
        // Half-word by half-word (four inputs of every row at a time) with the columns inside: only two
        // float4 of inputs per row pair are live instead of eight, and the RP x C chains of one step
        // are independent of one another (a chain still takes its inputs in order 0 .. 15).
        uint2 wdc[C];
        float2 quant[RP][C];
#pragma unroll
        for (int c = 0; c < C; ++c) {
            wdc[c] = *reinterpret_cast<const uint2*>(gb + uint32_t(c) * (p.k >> 1) + b * 256u + lane * 8u);
#pragma unroll
            for (int rp = 0; rp < RP; ++rp) quant[rp][c] = make_float2(0.0f, 0.0f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 lo[RP], hi[RP];
#pragma unroll
            for (int rp = 0; rp < RP; ++rp) {
                lo[rp] = xs4[((rp * blocks + b) * 8u + 2 * i) * 32u + lane];
                hi[rp] = xs4[((rp * blocks + b) * 8u + 2 * i + 1) * 32u + lane];
            }
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const uint32_t word = (i & 2) ? wdc[c].y : wdc[c].x;
                const uint32_t half = (i & 1) ? (word >> 16) : (word & 0xFFFFu);
                // the four nibbles of half-word i, each as {w, w}; inputs 4i .. 4i+3 are lo.xy, lo.zw, hi.xy, hi.zw
                const float w0 = __uint_as_float((half & 0x000Fu) | 0x4B000000u), w1 = __uint_as_float((half & 0x00F0u) | 0x4B000000u);
                const float w2 = __uint_as_float((half & 0x0F00u) | 0x4B000000u), w3 = __uint_as_float((half & 0xF000u) | 0x4B000000u);
                const float n0 = __fadd_rn(w0, magic.x), n1 = __fadd_rn(w1, magic.x);
                const float n2 = __fadd_rn(w2, magic.x), n3 = __fadd_rn(w3, magic.x);
                const float2 q0 = make_float2(n0, n0), q1 = make_float2(n1, n1), q2 = make_float2(n2, n2), q3 = make_float2(n3, n3);
#pragma unroll
                for (int rp = 0; rp < RP; ++rp) {
                    quant[rp][c] = __ffma2_rn(make_float2(lo[rp].x, lo[rp].y), q0, quant[rp][c]);
                    quant[rp][c] = __ffma2_rn(make_float2(lo[rp].z, lo[rp].w), q1, quant[rp][c]);
                    quant[rp][c] = __ffma2_rn(make_float2(hi[rp].x, hi[rp].y), q2, quant[rp][c]);
                    quant[rp][c] = __ffma2_rn(make_float2(hi[rp].z, hi[rp].w), q3, quant[rp][c]);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const float scale = __uint_as_float(uint32_t(gs[uint32_t(c) * gpr + b * 8u + (lane >> 2)]) << 16);
            const float bias = __uint_as_float(uint32_t(gbias[uint32_t(c) * gpr + b * 8u + (lane >> 2)]) << 16);
#pragma unroll
            for (int rp = 0; rp < RP; ++rp) {
                const float2 sum = sum2[(rp * blocks + b) * 32u + lane];
                result[rp][c] = __ffma2_rn(sum, make_float2(bias, bias),
                                           __ffma2_rn(make_float2(scale, scale), quant[rp][c], result[rp][c]));
            }
        }
      }
        {
#pragma unroll
            for (int rp = 0; rp < RP; ++rp) {
                float keep0 = 0.0f, keep1 = 0.0f;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    const float t0 = warp_sum(result[rp][c].x), t1 = warp_sum(result[rp][c].y);
                    if (lane == uint32_t(c)) {
                        keep0 = t0;
                        keep1 = t1;
                    }
                    result[rp][c] = make_float2(0.0f, 0.0f);
                }
                const uint32_t r0 = row0 + 2u * rp;
                if (ok && lane < uint32_t(C)) {
                    if (r0 < p.n_rows) p.out[uint64_t(r0) * p.out_stride + g * C + lane] = f2bf(keep0);
                    if (r0 + 1u < p.n_rows) p.out[uint64_t(r0 + 1u) * p.out_stride + g * C + lane] = f2bf(keep1);
                }
            }
        }
        // the buffer is read: it takes the group two rounds ahead
        __syncwarp();
        if (lane == 0 && ok && g + uint32_t(NB) * nwarps < n_groups) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            request(g + uint32_t(NB) * nwarps, buf);
        }
        phase ^= 1u << buf;
        if (NB > 1) buf ^= 1u;
        g += nwarps;
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        atomicCAS(p.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
        p.status[kStatusDetail] = blockIdx.x;
        __nanosleep(200000);   // let copies still in flight land before the shared memory is released
    }
}

template <int RP, int C>
static cudaError_t launch_q4_pairs(const Q4Params& p, uint32_t sm_count, int device, cudaStream_t stream) {
    const uint32_t groups = p.n_cols / C, blocks = p.k >> 9;
    const uint32_t ctas = min((groups + kQ4Warps - 1u) / kQ4Warps, sm_count);
    const uint32_t smem = RP * blocks * (256u * 16u + 32u * 8u);
    static bool configured[64] = {false};   // the attribute is per device
    if (!configured[device & 63]) {
        const cudaError_t err = cudaFuncSetAttribute(q4_project_pairs_kernel<RP, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, 212992);
        if (err != cudaSuccess) return err;
        configured[device & 63] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, (p.n_rows + 2 * RP - 1) / (2 * RP));
    cfg.blockDim = dim3(kQ4Warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, q4_project_pairs_kernel<RP, C>, p);
}

template <int RP, int C, int W, int NB>
static cudaError_t launch_q4_pairs_bulk(const Q4Params& p, uint32_t sm_count, int device, cudaStream_t stream) {
    const uint32_t groups = p.n_cols / C, blocks = p.k >> 9;
    const uint32_t ctas = min((groups + uint32_t(W) - 1u) / uint32_t(W), sm_count);
    const uint32_t smem = RP * blocks * (256u * 16u + 32u * 8u) + uint32_t(W) * uint32_t(NB) * q4_bulk_layout(1, C, p.k).group_bytes +
                          uint32_t(W) * 16u + 16u;
    static bool configured[64] = {false};   // the attribute is per device
    if (!configured[device & 63]) {
        const cudaError_t err = cudaFuncSetAttribute(q4_project_pairs_bulk_kernel<RP, C, W, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 221184);
        if (err != cudaSuccess) return err;
        configured[device & 63] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, (p.n_rows + 2 * RP - 1) / (2 * RP));
    cfg.blockDim = dim3(uint32_t(W) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, q4_project_pairs_bulk_kernel<RP, C, W, NB>, p);
}

// The bulk-copy form of the exact-row kernel (rows <= 4).
template <int R, int C>
static cudaError_t launch_q4_bulk(const Q4Params& p, uint32_t sm_count, int device, cudaStream_t stream) {
    const uint32_t groups = p.n_cols / C;
    const Q4BulkLayout lay = q4_bulk_layout(R, C, p.k);
    // as many CTAs per SM as the shared memory holds (at most three): more warps to hide the latencies
    // of the block loop, and more of the matrix asked for at once
    const uint32_t per_sm = max(1u, min(3u, 232448u / (lay.total + 1024u)));
    const uint32_t ctas = min((groups + kQ4Warps - 1u) / kQ4Warps, sm_count * per_sm);
    static bool configured[64] = {false};   // the attribute is per device
    if (!configured[device & 63]) {
        const cudaError_t err = cudaFuncSetAttribute(q4_project_bulk_kernel<R, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, 221184);
        if (err != cudaSuccess) return err;
        configured[device & 63] = true;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, (p.n_rows + R - 1) / R);
    cfg.blockDim = dim3(kQ4Warps * 32);
    cfg.dynamicSmemBytes = lay.total;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, q4_project_bulk_kernel<R, C>, p);
}

// Up to 4 rows per warp pass (more rows run as further row tiles that re-read the weights from L2).
template <int R, int C>
static void launch_q4(const Q4Params& p, uint32_t sm_count, uint32_t ctas_per_sm, cudaStream_t stream) {
    const uint32_t groups = p.n_cols / C;
    const uint32_t ctas = min((groups + kQ4Warps - 1u) / kQ4Warps, sm_count * ctas_per_sm);
    const uint32_t smem = R * (p.k >> 3) * 16u;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, (p.n_rows + R - 1) / R);
    cfg.blockDim = dim3(kQ4Warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, q4_project_kernel<R, C>, p);
}

// =========================================================================================
// tensor-unit policy: dequantise once ...
// =========================================================================================
__global__ void __launch_bounds__(256) q4_dequant_kernel(const uint32_t* __restrict__ words,
                                                         const __nv_bfloat16* __restrict__ scales,
                                                         const __nv_bfloat16* __restrict__ biases,
                                                         __nv_bfloat16* __restrict__ weights, uint64_t n_words) {
    for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < n_words; i += uint64_t(gridDim.x) * 256ull) {
        const uint32_t word = __ldg(words + i);
        const float scale = bf2f(scales[i >> 3]), bias = bf2f(biases[i >> 3]);
        __nv_bfloat16 res[8];
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) res[j] = f2bf(__fmaf_rn(float((word >> (4u * j)) & 15u), scale, bias));
        *reinterpret_cast<uint4*>(weights + i * 8ull) = *reinterpret_cast<const uint4*>(res);
    }
}

// ... then out[M][N] = x[M][K] . w[N][K]^T on the tensor cores.
constexpr uint32_t kGM = 128, kGN = 256, kGK = 64, kGStages = 4, kGAccs = 2;
constexpr uint32_t kGABytes = kGM * 128, kGBBytes = kGN * 128, kGStageBytes = kGABytes + kGBBytes;
constexpr uint32_t kGOffBar = kGStages * kGStageBytes;
constexpr uint32_t kGemmSmem = kGOffBar + 256;
constexpr uint32_t kGemmThreads = 192;  // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue (one TMEM lane quarter each)
enum : uint32_t { kGBarFull = 0, kGBarEmpty = kGBarFull + kGStages, kGBarAccFull = kGBarEmpty + kGStages,
                  kGBarAccEmpty = kGBarAccFull + kGAccs, kGBarCount = kGBarAccEmpty + kGAccs };
static_assert(8 * kGBarCount + 16 <= 256, "barrier block");

struct GemmParams {
    __nv_bfloat16* out;
    uint32_t* status;
    uint64_t out_stride;
    uint32_t m, n, k, m_tiles, n_tiles;
};

__global__ void __launch_bounds__(kGemmThreads, 1)
dense_project_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t base = s2u(smem), bars = base + kGOffBar;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kGOffBar + 8 * kGBarCount);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kGOffBar + 8 * kGBarCount + 8);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };
    const uint32_t n_tiles_total = p.m_tiles * p.n_tiles, kblocks = p.k / kGK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kGStages; ++s) {
            mbar_init(bar(kGBarFull + s), 1);
            mbar_init(bar(kGBarEmpty + s), 1);
        }
        for (uint32_t a = 0; a < kGAccs; ++a) {
            mbar_init(bar(kGBarAccFull + a), 1);
            mbar_init(bar(kGBarAccEmpty + a), 128);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)),
                     "r"(kGAccs * kGN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // Tile order: the weight tiles of one band of input rows are adjacent, so the CTAs running
    // at the same time share a few input tiles and walk the (L2-resident) weight matrix.
    if (warp == 0) {
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x) {
                const int m0 = int((t / p.n_tiles) * kGM), n0 = int((t % p.n_tiles) * kGN);
                for (uint32_t kb = 0; kb < kblocks; ++kb, ++n) {
                    const uint32_t s = n % kGStages, use = n / kGStages;
                    if (use > 0 && !mbar_wait(bar(kGBarEmpty + s), (use - 1u) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(bar(kGBarFull + s), kGStageBytes);
                    tma_load_2d(base + s * kGStageBytes, &map_x, bar(kGBarFull + s), int(kb * kGK), m0);
                    tma_load_2d(base + s * kGStageBytes + kGABytes, &map_w, bar(kGBarFull + s), int(kb * kGK), n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(kGM, kGN, false);
            uint32_t n = 0, it = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < n_tiles_total; t += gridDim.x, ++it) {
                const uint32_t ab = it % kGAccs, ause = it / kGAccs;
                if (ause > 0 && !mbar_wait(bar(kGBarAccEmpty + ab), (ause - 1u) & 1u, abort_flag)) break;
                tc_fence_after();
                for (uint32_t kb = 0; kb < kblocks; ++kb, ++n) {
                    const uint32_t s = n % kGStages;
                    if (!mbar_wait(bar(kGBarFull + s), (n / kGStages) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ++ks) {
                        const uint64_t ad = smem_desc(base + s * kGStageBytes + ks * 32u, 16, 1024);
                        const uint64_t bd = smem_desc(base + s * kGStageBytes + kGABytes + ks * 32u, 16, 1024);
                        tc_mma(tmem + ab * kGN, ad, bd, idesc, (kb | ks) ? 1u : 0u);
                    }
                    tc_commit(bar(kGBarEmpty + s));
                }
                if (ok) tc_commit(bar(kGBarAccFull + ab));
            }
        }
    } else {
        // epilogue: thread = one output row of the tile (its TMEM lane), 32 columns at a time
        const uint32_t quarter = warp & 3u, row_in_tile = quarter * 32u + lane;
        const uint32_t tlane = (quarter * 32u) << 16;
        uint32_t it = 0;
        for (uint32_t t = blockIdx.x; t < n_tiles_total; t += gridDim.x, ++it) {
            const uint32_t ab = it % kGAccs;
            if (!mbar_wait(bar(kGBarAccFull + ab), (it / kGAccs) & 1u, abort_flag)) break;
            tc_fence_after();
            const uint32_t row = (t / p.n_tiles) * kGM + row_in_tile, n0 = (t % p.n_tiles) * kGN;
            __nv_bfloat16* orow = p.out + uint64_t(row) * p.out_stride + n0;
#pragma unroll 2
            for (uint32_t ch = 0; ch < kGN / 32u; ++ch) {
                float v[32];
                tmem_ld32(tmem + tlane + ab * kGN + ch * 32u, v);
                tmem_wait_ld();
                if (row < p.m && n0 + ch * 32u < p.n) {
#pragma unroll
                    for (uint32_t q = 0; q < 4; ++q) {
                        __nv_bfloat162 h[4];
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                        *reinterpret_cast<uint4*>(orow + ch * 32u + q * 8u) = *reinterpret_cast<const uint4*>(h);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar(kGBarAccEmpty + ab));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicCAS(p.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
            p.status[kStatusDetail] = blockIdx.x;
        }
        __nanosleep(200000); // let copies still in flight land before the shared memory is released
        __syncthreads();
    }
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGAccs * kGN) : "memory");
    }
}

// ---- CTA-pair form: two SMs on one 256 x 256 output tile (tcgen05 cta_group::2) -------------
// A cluster of two CTAs; CTA r owns rows [128r, 128r+128) of the tile (its own 128 TMEM lanes)
// and loads, per 128-wide k step, its 128 input rows and HALF of the 256 weight rows (32 KiB
// each): the pair's tensor cores exchange the weight halves, so every SM pulls 64 KiB per 128 of k
// from L2 instead of 96 KiB and reads 8 KiB instead of 12 KiB of shared memory per MMA.  The even
// CTA (leader) issues the M256 N256 K16 MMAs for both; both CTAs run a TMA producer and an
// epilogue.  Barriers: `full` lives in the leader (the leader's producer arrives expecting the
// bytes of both CTAs; both CTAs' copies complete on it), `empty` and `acc_full` live in each CTA
// and are signalled by one tcgen05.commit of the leader that arrives in both CTAs, `acc_empty`
// lives in the leader and counts one arrival per epilogue warp of both CTAs.
constexpr uint32_t kPK = 128, kPStages = 3, kPStageBytes = 65536, kPABytes = 32768, kPAtomBytes = 16384;
constexpr uint32_t kPOffBar = kPStages * kPStageBytes;
constexpr uint32_t kPairSmem = kPOffBar + 256;
enum : uint32_t { kPBarFull = 0, kPBarEmpty = kPBarFull + kPStages, kPBarAccFull = kPBarEmpty + kPStages,
                  kPBarAccEmpty = kPBarAccFull + kGAccs, kPBarCount = kPBarAccEmpty + kGAccs };
static_assert(8 * kPBarCount + 16 <= 256, "barrier block");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
dense_project_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                          const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t base = s2u(smem), bars = base + kPOffBar;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kPOffBar + 8 * kPBarCount);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kPOffBar + 8 * kPBarCount + 8);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0u;
    const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t n_tiles_total = p.m_tiles * p.n_tiles, kblocks = p.k / kPK;   // tiles of 256 x 256

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kPStages; ++s) {
            mbar_init(bar(kPBarFull + s), 1);    // the leader arrives, expecting the bytes of both CTAs
            mbar_init(bar(kPBarEmpty + s), 1);
        }
        for (uint32_t a = 0; a < kGAccs; ++a) {
            mbar_init(bar(kPBarAccFull + a), 1);
            mbar_init(bar(kPBarAccEmpty + a), 8);   // 4 epilogue warps x 2 CTAs
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs allocates the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)),
                     "r"(kGAccs * kGN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs are initialised before any remote arrival
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < n_tiles_total; t += n_pairs) {
                const int m0 = int((t / p.n_tiles) * 256u + rank * 128u), n0 = int((t % p.n_tiles) * 256u + rank * 128u);
                for (uint32_t kb = 0; kb < kblocks; ++kb, ++n) {
                    const uint32_t s = n % kPStages, use = n / kPStages;
                    if (use > 0 && !mbar_wait(bar(kPBarEmpty + s), (use - 1u) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    // Both CTAs' copies complete on the leader's barrier; the leader alone arrives on it,
                    // expecting the bytes of both (a remote arrive.expect_tx with cluster-scope release
                    // cost the producers 1200 cycles per stage: measured with cycle counters).
                    const uint32_t full = map_to_cta(bar(kPBarFull + s), 0u);
                    if (leader) mbar_expect_tx(bar(kPBarFull + s), 2u * kPStageBytes);
#pragma unroll
                    for (uint32_t a = 0; a < 2; ++a) {   // two 64-wide swizzle atoms per operand
                        tma_load_2d_pair(base + s * kPStageBytes + a * kPAtomBytes, &map_x, full, int(kb * kPK + a * 64u), m0);
                        tma_load_2d_pair(base + s * kPStageBytes + kPABytes + a * kPAtomBytes, &map_w, full, int(kb * kPK + a * 64u), n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = instr_desc(256, kGN, false);
            uint32_t n = 0, it = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < n_tiles_total; t += n_pairs, ++it) {
                const uint32_t ab = it % kGAccs, ause = it / kGAccs;
                if (ause > 0 && !mbar_wait(bar(kPBarAccEmpty + ab), (ause - 1u) & 1u, abort_flag)) break;
                tc_fence_after();
                for (uint32_t kb = 0; kb < kblocks; ++kb, ++n) {
                    const uint32_t s = n % kPStages;
                    if (!mbar_wait(bar(kPBarFull + s), (n / kPStages) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks) {
                        const uint32_t off = (ks >> 2) * kPAtomBytes + (ks & 3u) * 32u;
                        const uint64_t ad = smem_desc(base + s * kPStageBytes + off, 16, 1024);
                        const uint64_t bd = smem_desc(base + s * kPStageBytes + kPABytes + off, 16, 1024);
                        tc_mma_pair(tmem + ab * kGN, ad, bd, idesc, (kb | ks) ? 1u : 0u);
                    }
                    tc_commit_both(bar(kPBarEmpty + s));
                }
                if (ok) {
                    tc_commit_both(bar(kPBarAccFull + ab));
                }
            }
        }
    } else {
        const uint32_t quarter = warp & 3u, row_in_tile = quarter * 32u + lane;
        const uint32_t tlane = (quarter * 32u) << 16;
        uint32_t it = 0;
        for (uint32_t t = pair; t < n_tiles_total; t += n_pairs, ++it) {
            const uint32_t ab = it % kGAccs;
            if (!mbar_wait(bar(kPBarAccFull + ab), (it / kGAccs) & 1u, abort_flag)) break;
            tc_fence_after();
            const uint32_t row = (t / p.n_tiles) * 256u + rank * 128u + row_in_tile, n0 = (t % p.n_tiles) * 256u;
            __nv_bfloat16* orow = p.out + uint64_t(row) * p.out_stride + n0;
#pragma unroll 2
            for (uint32_t ch = 0; ch < kGN / 32u; ++ch) {
                float v[32];
                tmem_ld32(tmem + tlane + ab * kGN + ch * 32u, v);
                tmem_wait_ld();
                if (row < p.m && n0 + ch * 32u < p.n) {
#pragma unroll
                    for (uint32_t q = 0; q < 4; ++q) {
                        __nv_bfloat162 h[4];
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                        *reinterpret_cast<uint4*>(orow + ch * 32u + q * 8u) = *reinterpret_cast<const uint4*>(h);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(bar(kPBarAccEmpty + ab), 0u));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicCAS(p.status + kStatusCode, 0u, uint32_t(TATARA_DEVICE_WAIT_TIMEOUT));
            p.status[kStatusDetail] = blockIdx.x;
        }
        __nanosleep(200000); // let copies still in flight land before the shared memory is released
    }
    // neither CTA leaves (or frees tensor memory) while its peer may still arrive on its barriers
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGAccs * kGN) : "memory");
    }
}

// 2-D bf16 tensor map {k, rows} with a {64, box_rows} box and the 128-byte swizzle.
static bool make_map_2d(CUtensorMap* map, const void* ptr, uint64_t k, uint64_t rows, uint64_t stride_bytes,
                        uint32_t box_rows) {
    EncodeTiled fn = encode_tiled_entry();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {stride_bytes};
    const cuuint32_t box[2] = {kGK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static tatara_status check_matrices(tatara_ctx* ctx, const tatara_q4_matrix* matrices, uint32_t n_matrices,
                                    uint32_t k, uint32_t k_multiple, const char* what, uint32_t* total) {
    if (matrices == nullptr || n_matrices == 0 || n_matrices > kQ4MaxMats)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, what);
    if (k == 0 || k % k_multiple != 0) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, what);
    uint32_t cols = 0;
    for (uint32_t i = 0; i < n_matrices; ++i) {
        const tatara_q4_matrix& m = matrices[i];
        if (!m.words || !m.scales || !m.biases) return fail(ctx, TATARA_INVALID_BUFFER, what);
        if (!aligned(m.words, 16) || !aligned(m.scales, 2) || !aligned(m.biases, 2))
            return fail(ctx, TATARA_INVALID_BUFFER, what);
        if (m.rows == 0 || m.rows % 16u != 0) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, what);
        cols += m.rows;
    }
    *total = cols;
    return TATARA_OK;
}

} // namespace tb

using namespace tb;

extern "C" tatara_status tatara_q4_project(tatara_ctx* ctx, void* stream, const void* input,
                                           uint64_t input_stride, uint32_t n_rows,
                                           const tatara_q4_matrix* matrices, uint32_t n_matrices,
                                           uint32_t k, void* out, uint64_t out_stride) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!input || !out) return fail(ctx, TATARA_INVALID_BUFFER, "q4_project: null buffer");
    if (!aligned(input, 16) || !aligned(out, 2))
        return fail(ctx, TATARA_INVALID_BUFFER, "q4_project: misaligned buffer");
    uint32_t cols = 0;
    const tatara_status st = check_matrices(ctx, matrices, n_matrices, k, 512, "q4_project: matrices", &cols);
    if (st != TATARA_OK) return st;
    if (n_rows == 0 || input_stride < k || input_stride % 8u != 0 || out_stride < cols)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "q4_project: rows or strides");
    Q4Params p{};
    p.x = static_cast<const __nv_bfloat16*>(input);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.x_stride = input_stride;
    p.out_stride = out_stride;
    p.n_rows = n_rows;
    p.k = k;
    p.n_cols = cols;
    p.n_mats = n_matrices;
    uint32_t at = 0;
    for (uint32_t i = 0; i < n_matrices; ++i) {
        p.mat[i].words = static_cast<const uint2*>(matrices[i].words);
        p.mat[i].scales = static_cast<const __nv_bfloat16*>(matrices[i].scales);
        p.mat[i].biases = static_cast<const __nv_bfloat16*>(matrices[i].biases);
        p.mat[i].col_begin = at;
        at += matrices[i].rows;
        p.mat[i].col_end = at;
    }
    auto s = static_cast<cudaStream_t>(stream);
    const uint32_t sms = uint32_t(ctx->sm_count);
    if (k > 6144u) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "q4_project: k above 6144");
    p.status = ctx->device_status;
    // The bulk-copy form needs 16-byte aligned rows of scales and biases (k / 32 bytes each, from a
    // 16-byte aligned base) and a column count that splits into whole groups.
    bool aligned16 = ctx->q4_row_form == 0u && k % 512u == 0u;
    for (uint32_t i = 0; i < n_matrices && aligned16; ++i)
        aligned16 = aligned(matrices[i].scales, 16) && aligned(matrices[i].biases, 16);
    const bool bulk = aligned16 && n_rows <= 4u && q4_bulk_layout(n_rows <= 2u ? n_rows : 4u, 4u, k).total <= 221184u;
    // more than four rows: the row-pair kernel, its weights by bulk copies when the inputs of eight rows
    // and the buffers fit the shared memory (four columns per warp up to 2048 inputs, two up to 4096)
    const uint32_t pairs_x = 4u * (k >> 9) * (256u * 16u + 32u * 8u);
    auto pairs_fit = [&](uint32_t cols_per_warp, uint32_t warps, uint32_t buffers) {
        return pairs_x + warps * buffers * q4_bulk_layout(1, cols_per_warp, k).group_bytes + warps * 16u + 16u <= 221184u;
    };
    auto rounds = [&](uint32_t cols_per_warp, uint32_t warps) {
        const uint32_t groups = cols / cols_per_warp;
        return (groups + sms * warps - 1u) / (sms * warps);
    };
    // (two columns per warp re-read the inputs twice as often: measured 15.1 -> 10.4 us at 8 rows of the
    // out projection but 15.1 -> 20.3 us at 16, where two row tiles share the SMs)
    const bool pairs_bulk4 = aligned16 && n_rows > 4u && pairs_fit(4, 8, 2);
    const bool pairs_bulk2 = aligned16 && n_rows > 4u && n_rows <= 8u && !pairs_bulk4 && pairs_fit(2, 8, 2);
    // EIGHT columns per warp halve the shared-memory traffic per multiply-add (the inputs of a block are read
    // once per eight columns): taken when every warp then has exactly one column group, which also needs one
    // buffer per warp only.
    const bool pairs_bulk8 = pairs_bulk4 && cols % 8u == 0u && rounds(8, 8) == 1u && pairs_fit(8, 8, 1);
    // Eight, eleven or twelve warps per SM (157 registers): more warps hide more latency, but what matters first is how
    // evenly the column groups divide over the warps (2304 groups of attn_project on 8 / 12 warps: two rounds
    // either way, 14.3 / 18.3 us; 3088 groups of gdn_project: three rounds of 8 or two of 12, 19.7 / 18.9 us).
    auto slots = [&](uint32_t groups, uint32_t warps) { return ((groups + sms * warps - 1u) / (sms * warps)) * warps; };
    auto best_warps = [&](uint32_t cols_per_warp) {
        uint32_t best = 8;
        for (uint32_t w : {11u, 12u})
            if (pairs_fit(cols_per_warp, w, 2) && slots(cols / cols_per_warp, w) <= slots(cols / cols_per_warp, best)) best = w;
        // seven warps when they still take every group in ONE round (2048 columns in pairs: 147 CTAs of 7 warps on
        // 148 SMs instead of 128 CTAs of 8; with several rounds fewer warps hide less: gdn_project 17.6 -> 18.3 us)
        if (cols / cols_per_warp <= sms * 7u && slots(cols / cols_per_warp, 7) < slots(cols / cols_per_warp, best)) best = 7;
        return best;
    };
    if (pairs_bulk8) {
        (void)launch_q4_pairs_bulk<4, 8, 8, 1>(p, sms, ctx->device, s);
    } else if (pairs_bulk4) {
        const uint32_t w = best_warps(4);
        if (w == 12) (void)launch_q4_pairs_bulk<4, 4, 12, 2>(p, sms, ctx->device, s);
        else if (w == 11) (void)launch_q4_pairs_bulk<4, 4, 11, 2>(p, sms, ctx->device, s);
        else if (w == 7) (void)launch_q4_pairs_bulk<4, 4, 7, 2>(p, sms, ctx->device, s);
        else (void)launch_q4_pairs_bulk<4, 4, 8, 2>(p, sms, ctx->device, s);
    } else if (pairs_bulk2) {
        const uint32_t w = best_warps(2);
        if (w == 12) (void)launch_q4_pairs_bulk<4, 2, 12, 2>(p, sms, ctx->device, s);
        else if (w == 11) (void)launch_q4_pairs_bulk<4, 2, 11, 2>(p, sms, ctx->device, s);
        else if (w == 7) (void)launch_q4_pairs_bulk<4, 2, 7, 2>(p, sms, ctx->device, s);
        else (void)launch_q4_pairs_bulk<4, 2, 8, 2>(p, sms, ctx->device, s);
    } else if (bulk) {
        // narrow matrices take two columns per warp so that every warp of the grid has a group
        const bool narrow = cols / 4u < sms * kQ4Warps;
        cudaError_t err;
        if (n_rows == 1) err = narrow ? launch_q4_bulk<1, 2>(p, sms, ctx->device, s) : launch_q4_bulk<1, 4>(p, sms, ctx->device, s);
        else if (n_rows == 2) err = narrow ? launch_q4_bulk<2, 2>(p, sms, ctx->device, s) : launch_q4_bulk<2, 4>(p, sms, ctx->device, s);
        else err = narrow ? launch_q4_bulk<4, 2>(p, sms, ctx->device, s) : launch_q4_bulk<4, 4>(p, sms, ctx->device, s);
        (void)err;
    } else if (n_rows == 1) {
        // few warps with many bytes in flight each; narrow matrices get narrower groups (more warps)
        if (cols >= 8192u) launch_q4<1, 8>(p, sms, 1, s);
        else launch_q4<1, 4>(p, sms, 1, s);
    } else if (n_rows == 2) {
        launch_q4<2, 4>(p, sms, 1, s);
    } else if (n_rows <= 4) {
        launch_q4<4, 4>(p, sms, 1, s);
    } else {
        (void)launch_q4_pairs<4, 4>(p, sms, ctx->device, s);   // 8 rows per pass; more rows run as further row tiles
    }
    return check_launch(ctx, "q4_project");
}

extern "C" tatara_status tatara_q4_dequantize(tatara_ctx* ctx, void* stream,
                                              const tatara_q4_matrix* matrices, uint32_t n_matrices,
                                              uint32_t k, void* weights) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!weights || !aligned(weights, 16)) return fail(ctx, TATARA_INVALID_BUFFER, "q4_dequantize: weights");
    uint32_t cols = 0;
    const tatara_status st = check_matrices(ctx, matrices, n_matrices, k, 64, "q4_dequantize: matrices", &cols);
    if (st != TATARA_OK) return st;
    auto* w = static_cast<__nv_bfloat16*>(weights);
    for (uint32_t i = 0; i < n_matrices; ++i) {
        const uint64_t n_words = uint64_t(matrices[i].rows) * (k / 8u);
        const uint64_t want = (n_words + 255u) / 256u, cap = uint64_t(ctx->sm_count) * 16u;
        const uint32_t grid = uint32_t(want < cap ? want : cap);
        q4_dequant_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint32_t*>(matrices[i].words), static_cast<const __nv_bfloat16*>(matrices[i].scales),
            static_cast<const __nv_bfloat16*>(matrices[i].biases), w, n_words);
        const tatara_status ls = check_launch(ctx, "q4_dequantize");
        if (ls != TATARA_OK) return ls;
        w += uint64_t(matrices[i].rows) * k;
    }
    return TATARA_OK;
}

extern "C" tatara_status tatara_project_dense(tatara_ctx* ctx, void* stream, const void* input,
                                              uint64_t input_stride, uint32_t n_rows,
                                              const void* weights, uint32_t n, uint32_t k, void* out,
                                              uint64_t out_stride) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!input || !weights || !out) return fail(ctx, TATARA_INVALID_BUFFER, "project_dense: null buffer");
    if (!aligned(input, 16) || !aligned(weights, 16) || !aligned(out, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "project_dense: buffers must be 16-byte aligned");
    if (n_rows == 0 || n == 0 || n % 32u != 0 || k == 0 || k % kGK != 0 || input_stride < k ||
        input_stride % 8u != 0 || out_stride < n || out_stride % 8u != 0)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "project_dense: extents");
    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(dense_project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) !=
                cudaSuccess ||
            cudaFuncSetAttribute(dense_project_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) !=
                cudaSuccess)
            return check_launch(ctx, "project_dense: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    GemmParams gp{};
    gp.out = static_cast<__nv_bfloat16*>(out);
    gp.status = ctx->device_status;
    gp.out_stride = out_stride;
    gp.m = n_rows;
    gp.n = n;
    gp.k = k;
    CUtensorMap map_x, map_w;
    // Blocks of at least 256 rows run on CTA pairs (256 x 256 tiles, half a weight tile per CTA).
    if (n_rows >= 256u && n >= 256u && k % kPK == 0 && ctx->sm_count >= 2) {
        if (!make_map_2d(&map_x, input, k, n_rows, input_stride * 2ull, 128) ||
            !make_map_2d(&map_w, weights, k, n, uint64_t(k) * 2ull, 128))
            return fail(ctx, TATARA_CUDA_ERROR, "project_dense: tensor map encoding failed");
        gp.m_tiles = (n_rows + 255u) / 256u;
        gp.n_tiles = (n + 255u) / 256u;
        const uint32_t tiles = gp.m_tiles * gp.n_tiles, pairs = uint32_t(ctx->sm_count) / 2u;
        const uint32_t grid = 2u * (tiles < pairs ? tiles : pairs);
        dense_project_pair_kernel<<<grid, kGemmThreads, kPairSmem, static_cast<cudaStream_t>(stream)>>>(map_x, map_w, gp);
        return check_launch(ctx, "project_dense(pair)");
    }
    if (!make_map_2d(&map_x, input, k, n_rows, input_stride * 2ull, kGM) ||
        !make_map_2d(&map_w, weights, k, n, uint64_t(k) * 2ull, kGN))
        return fail(ctx, TATARA_CUDA_ERROR, "project_dense: tensor map encoding failed");
    gp.m_tiles = (n_rows + kGM - 1u) / kGM;
    gp.n_tiles = (n + kGN - 1u) / kGN;
    const uint32_t tiles = gp.m_tiles * gp.n_tiles;
    const uint32_t grid = tiles < uint32_t(ctx->sm_count) ? tiles : uint32_t(ctx->sm_count);
    dense_project_kernel<<<grid, kGemmThreads, kGemmSmem, static_cast<cudaStream_t>(stream)>>>(map_x, map_w, gp);
    return check_launch(ctx, "project_dense");
}
