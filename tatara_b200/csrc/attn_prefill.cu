// Causal block prefill of the gated GQA attention layers on the 5th-generation tensor cores
// (reference semantics: attention_partial_blk + attention_combine_blk,
// prefill_attention.metal:97-254; shipped pair of GEMMs + softmax + gate, host
// src/runtime/prefill_step.cpp:1467-1819).
//
// One CTA owns 128 query rows of one head and streams the visible keys in tiles of 128:
//     S = Q K^T      tcgen05.mma  M128 N128 K256   (A = Q, B = K tile, both K-major swizzled smem)
//     P = exp2(S*c - m)  in registers, one thread per query row (tcgen05.ld of its TMEM lane)
//     O += P V       tcgen05.mma  M128 N256 K128   (A = P, K-major swizzled smem; B = V tile, MN-major smem)
// An M128 MMA costs about 64 cycles whatever its N up to 128 (measured: N = 64 tiles ran the
// tensor pipe at half rate), so the score tile is 128 keys wide.  K and V stream through rings of
// 32 KiB slots that are released and refilled INSIDE a tile: a K slot holds 128 of the 256 dims
// (the operand of eight consecutive k-steps), a V slot holds 64 of the 128 keys (four k-steps);
// a tcgen05.commit after each slot's MMAs hands the slot back to the TMA producer.
// TMEM map (512 columns): S buffer 0 at 0..127, buffer 1 at 128..255, O at 256..511.  P goes
// through SHARED memory (bf16, written by the softmax threads under the 128-byte swizzle as the
// K-major A operand), not through the S buffer: an S buffer is released the moment its scores are
// in registers, so the score MMAs run two tiles ahead and the softmax of a tile (about 1750
// cycles) is no longer the latency between two MMAs on one TMEM buffer.  Shared memory: Q 64 KiB,
// K ring 2 x 32 KiB, V ring 2 x 32 KiB, P 32 KiB.  Warp roles: warp 0 TMA producer, warp 1 MMA
// issuer, warps 2..9 softmax + epilogue (two warps per 32-row TMEM lane quarter, each owning one
// 64-key half of the score tile; the halves exchange their row maxima through shared memory).
// The running maximum is updated lazily (O and l are rescaled only when the maximum grows by more
// than 2^8), which keeps the TMEM round trip of O off the steady-state path.
// Every mbarrier wait is bounded; on a timeout the CTA latches TATARA_DEVICE_WAIT_TIMEOUT in the
// context's status word, frees its TMEM and returns.
// Two kernels share the softmax rows: attn_prefill_kernel (one CTA per tile and head, described
// above) and attn_prefill_pair_kernel (two CTAs on two heads of a KV group, described at its
// definition), selected by TATARA_POLICY_ATTN_PREFILL_FORM; their outputs are bit-identical.
#include "tc05.cuh"

namespace tb {

constexpr uint32_t kBM = 128, kBN = 128, kKSlots = 2, kVSlots = 2, kSBufs = 2;
constexpr uint32_t kAtomBytesQ = kBM * 128;          // one 64-dim swizzle atom of the Q tile
constexpr uint32_t kQBytes = 4 * kAtomBytesQ;        // 64 KiB
constexpr uint32_t kSlotBytes = 32768;               // K slot: 128 keys x 128 dims; V slot: 64 keys x 256 d
constexpr uint32_t kKAtomBytes = 128 * 128;          // one 64-dim atom of a K slot (128 keys x 128 B)
constexpr uint32_t kVAtomBytes = 64 * 128;           // one 64-d atom of a V slot (64 keys x 128 B)
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + kQBytes;
constexpr uint32_t kOffV = kOffK + kKSlots * kSlotBytes;
constexpr uint32_t kOffP = kOffV + kVSlots * kSlotBytes;   // P tile [128 rows x 128 keys] bf16, K-major, two 64-key atoms
constexpr uint32_t kPAtomBytes = kBM * 128, kPBytes = 2 * kPAtomBytes;
constexpr uint32_t kOffBar = kOffP + kPBytes;
constexpr uint32_t kPrefillSmem = kOffBar + 256 + 2 * 256 * 4;  // + row-max exchange (2 phases)
static_assert(kPrefillSmem <= 232448, "shared memory budget");
constexpr uint32_t kPrefillThreads = 320;   // TMA warp, MMA warp, 8 softmax warps
constexpr uint32_t kSoftmaxThreads = 256;
constexpr uint32_t kTmemCols = 512, kColS = 0, kColO = 256;

// barrier slots
enum : uint32_t { kBarQ = 0, kBarKFull = 1, kBarKEmpty = kBarKFull + kKSlots, kBarVFull = kBarKEmpty + kKSlots,
                  kBarVEmpty = kBarVFull + kVSlots, kBarSFull = kBarVEmpty + kVSlots, kBarSFree = kBarSFull + kSBufs,
                  kBarPFull = kBarSFree + kSBufs, kBarPvDone = kBarPFull + 1, kBarCount = kBarPvDone + 1 };
static_assert(8 * kBarCount + 16 <= 256, "barrier block");
constexpr uint32_t kOffPair = kOffBar + 256;       // [2 halves][128 rows] f32 exchange between the two warps of a row


struct PrefillParams {
    const __nv_bfloat16* gate;
    __nv_bfloat16* out;
    uint32_t* status;
    uint32_t context_base, rows, n_qtiles;
};

// What the softmax rows need to know of a kernel form: where Q, P and the row-max exchange live in
// shared memory, how many P buffers there are, and the slots of the barriers they touch.
struct SingleForm {
    static constexpr uint32_t kOffQ = tb::kOffQ, kOffP = tb::kOffP, kOffPair = tb::kOffPair, kPBufs = 1;
    static constexpr bool kArriveAtLeader = false;
    static constexpr uint32_t kBarSFull = tb::kBarSFull, kBarSFree = tb::kBarSFree, kBarPFull = tb::kBarPFull,
                              kBarPvDone = tb::kBarPvDone;
};

// ---------------- softmax + epilogue: two threads per query row (warps 2..9 of a CTA) ----------------
// How the softmax rows signal the MMA issuer.  One CTA: every thread arrives on its CTA's barrier.
// CTA pair: the issuer sits in the leader CTA, so each warp of BOTH CTAs arrives once, through one
// lane, on the leader's barrier (after __syncwarp, which orders the other lanes' tensor-memory loads
// and shared-memory stores before it).  The arrive has CTA-scope release semantics: a cluster-scope
// release on this path held the arriving thread for about 800 ns (timeline of a temporary build).
template <class Form>
__device__ __forceinline__ void rows_arrive(uint32_t bar_addr, uint32_t lane) {
    if constexpr (Form::kArriveAtLeader) {
        __syncwarp();
        if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(map_to_cta(bar_addr, 0u)) : "memory");
    } else {
        mbar_arrive(bar_addr);
    }
}

template <class Form>
__device__ __forceinline__ void softmax_rows(uint8_t* smem, uint32_t bars, uint32_t tmem, const PrefillParams& p,
                                             uint32_t warp, uint32_t lane, uint32_t head, uint32_t r0,
                                             uint32_t rows_here, uint32_t ntiles, volatile uint32_t* abort_flag) {
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };
    const uint32_t quarter = warp & 3u;            // TMEM lanes 32*quarter .. +31
    const uint32_t half = (warp - 2u) >> 2;        // which 64 keys of the tile / 128 dims of O
    const uint32_t row = quarter * 32u + lane;
    const uint32_t tlane = (quarter * 32u) << 16;
    const uint32_t pos = p.context_base + r0 + row; // keys 0..pos are visible to this row
    const float c = kAttnScale * 1.4426950408889634f;
    float* pair_x = reinterpret_cast<float*>(smem + Form::kOffPair);
    const uint32_t pair_bar = 1u + quarter;        // named barrier of the two warps of this quarter
    float m_used = -INFINITY, l = 0.0f;
    bool ok = true;
    for (uint32_t j = 0; j < ntiles; ++j) {
        const uint32_t s = j % kSBufs, par = (j / kSBufs) & 1u;
        // After a failed wait a thread keeps walking the tiles without waiting again (what it computes
        // and stores from then on is never used: the CTA reports the time-out and writes no output),
        // so every warp-wide instruction, the pair barrier and the arrivals stay convergent.
        if (ok && !mbar_wait(bar(Form::kBarSFull + s), par, abort_flag)) ok = false;
        tc_fence_after();
        float sv[64];
        tmem_ld32(tmem + tlane + kColS + s * kBN + half * 64u, sv);
        tmem_ld32(tmem + tlane + kColS + s * kBN + half * 64u + 32u, sv + 32);
        tmem_wait_ld();
        tc_fence_before();
        rows_arrive<Form>(bar(Form::kBarSFree + s), lane);   // the scores are in registers: the buffer may take tile j+2
        const uint32_t key0 = j * kBN + half * 64u;
        if (j * kBN + kBN - 1u > p.context_base + r0) { // the tile crosses this CTA's diagonal
#pragma unroll
            for (uint32_t i = 0; i < 64; ++i) sv[i] = key0 + i <= pos ? sv[i] : -INFINITY;
        }
        // row maximum of the raw scores (c > 0), four independent chains
        float m0 = fmaxf(sv[0], sv[1]), m1 = fmaxf(sv[2], sv[3]), m2 = fmaxf(sv[4], sv[5]), m3 = fmaxf(sv[6], sv[7]);
#pragma unroll
        for (uint32_t i = 8; i < 64; i += 8) {
            m0 = fmaxf(m0, fmaxf(sv[i], sv[i + 1]));
            m1 = fmaxf(m1, fmaxf(sv[i + 2], sv[i + 3]));
            m2 = fmaxf(m2, fmaxf(sv[i + 4], sv[i + 5]));
            m3 = fmaxf(m3, fmaxf(sv[i + 6], sv[i + 7]));
        }
        float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * c;
        // both halves of the row must agree on the maximum: exchange through shared memory
        pair_x[(j & 1u) * 256u + half * 128u + row] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        mx = fmaxf(mx, pair_x[(j & 1u) * 256u + (half ^ 1u) * 128u + row]);
        if (j == 0) {
            m_used = mx; // key 0 is visible to every row, so this is finite
        } else {
            const bool grow = mx > m_used + 8.0f;
            if (__any_sync(0xffffffffu, grow)) {
                // O holds P.V of tiles < j: wait for tile j-1, then rescale this row's half of O
                const uint32_t jp = j - 1u;
                if (ok && !mbar_wait(bar(Form::kBarPvDone + jp % Form::kPBufs), (jp / Form::kPBufs) & 1u, abort_flag))
                    ok = false;
                tc_fence_after();
                const float f = grow ? ex2(m_used - mx) : 1.0f;
                for (uint32_t ch = 0; ch < 4; ++ch) {
                    float ov[32];
                    tmem_ld32(tmem + tlane + kColO + half * 128u + ch * 32u, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) ov[i] *= f;
                    tmem_st32(tmem + tlane + kColO + half * 128u + ch * 32u, ov);
                }
                tmem_wait_st();
                l *= f;
                if (grow) m_used = mx;
            }
        }
        // p = 2^(s*c - m): one FFMA + one MUFU per score; four independent sums
        const float neg_m = -m_used;
        float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 64; i += 4) {
            sv[i] = ex2(fmaf(sv[i], c, neg_m));
            sv[i + 1] = ex2(fmaf(sv[i + 1], c, neg_m));
            sv[i + 2] = ex2(fmaf(sv[i + 2], c, neg_m));
            sv[i + 3] = ex2(fmaf(sv[i + 3], c, neg_m));
            s0 += sv[i]; s1 += sv[i + 1]; s2 += sv[i + 2]; s3 += sv[i + 3];
        }
        l += (s0 + s1) + (s2 + s3);
        // P goes to shared memory as the K-major A operand of P.V: this thread's 64 keys are one
        // 128-byte row of atom `half`, eight 16-byte chunks under the 128-byte swizzle.  The single
        // P tile is free once P.V of the tile that used it before (j - kPBufs) has completed.
        const uint32_t pb = j % Form::kPBufs;
        if (ok && j >= Form::kPBufs &&
            !mbar_wait(bar(Form::kBarPvDone + pb), (j / Form::kPBufs - 1u) & 1u, abort_flag))
            ok = false;
        {
            uint8_t* prow = smem + Form::kOffP + pb * kPBytes + half * kPAtomBytes + row * 128u;
#pragma unroll
            for (uint32_t ch = 0; ch < 8; ++ch) {
                uint32_t w[4];
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(sv[ch * 8 + 2 * i], sv[ch * 8 + 2 * i + 1]);
                    w[i] = *reinterpret_cast<const uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7u)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        if (j + 1u == ntiles) {   // the partner reads this half's row sum after the last P.V completes
            reinterpret_cast<float*>(smem + Form::kOffQ)[half * 128u + row] = l; // Q is dead: every S MMA has completed
            __threadfence_block();
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> the MMA's async proxy
        rows_arrive<Form>(bar(Form::kBarPFull + pb), lane);
    }
    if (ok) {
        const uint32_t jl = ntiles - 1u;
        ok = mbar_wait(bar(Form::kBarPvDone + jl % Form::kPBufs), (jl / Form::kPBufs) & 1u, abort_flag);
    }
    if (__all_sync(0xffffffffu, ok)) {   // warp-uniform: the tensor-memory loads below are warp-wide
        tc_fence_after();
        l += reinterpret_cast<const float*>(smem + Form::kOffQ)[(half ^ 1u) * 128u + row]; // + the partner's half
        const float inv_l = 1.0f / l;
        const bool live = row < rows_here;
        const uint64_t at = (uint64_t(r0 + row) * kQHeads + head) * kHeadDim + half * 128u;
        for (uint32_t ch = 0; ch < 4; ++ch) {
            float ov[32];
            tmem_ld32(tmem + tlane + kColO + half * 128u + ch * 32u, ov);
            tmem_wait_ld();
            if (live) {
#pragma unroll
                for (uint32_t q4 = 0; q4 < 4; ++q4) {
                    const uint4 graw = *reinterpret_cast<const uint4*>(p.gate + at + ch * 32u + q4 * 8u);
                    const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&graw);
                    __nv_bfloat16 res[8];
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        const float gate = bf2f(g[i]);
                        res[i] = f2bf((ov[q4 * 8 + i] * inv_l) * (1.0f / (1.0f + __expf(-gate))));
                    }
                    *reinterpret_cast<uint4*>(p.out + at + ch * 32u + q4 * 8u) = *reinterpret_cast<const uint4*>(res);
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kPrefillThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t base = s2u(smem);
    const uint32_t bars = base + kOffBar;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kOffBar + 8 * kBarCount);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + 8 * kBarCount + 8);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };

    // longest tiles first; the 16 heads of one query tile are adjacent (K/V stay hot in L2)
    const uint32_t qt = p.n_qtiles - 1u - (blockIdx.x >> 4);
    const uint32_t head = blockIdx.x & 15u, kv = head >> 3;
    const uint32_t r0 = qt * kBM;
    const uint32_t rows_here = min(kBM, p.rows - r0);
    const uint32_t visible = p.context_base + r0 + rows_here; // keys [0, visible)
    const uint32_t ntiles = (visible + kBN - 1u) / kBN;

    if (threadIdx.x == 0) {
        mbar_init(bar(kBarQ), 1);
        for (uint32_t s = 0; s < kKSlots; ++s) {
            mbar_init(bar(kBarKFull + s), 1);
            mbar_init(bar(kBarKEmpty + s), 1);
        }
        for (uint32_t s = 0; s < kVSlots; ++s) {
            mbar_init(bar(kBarVFull + s), 1);
            mbar_init(bar(kBarVEmpty + s), 1);
        }
        for (uint32_t s = 0; s < kSBufs; ++s) {
            mbar_init(bar(kBarSFull + s), 1);
            mbar_init(bar(kBarSFree + s), kSoftmaxThreads);
        }
        mbar_init(bar(kBarPFull), kSoftmaxThreads);
        mbar_init(bar(kBarPvDone), 1);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_expect_tx(bar(kBarQ), kQBytes);
            for (uint32_t a = 0; a < 4; ++a)
                tma_load_3d(base + kOffQ + a * kAtomBytesQ, &map_q, bar(kBarQ), int(a * 64), int(head), int(r0));
            // consumption order of the MMA thread: S_0, S_1, P.V_0, S_2, P.V_1, ...
            auto load_k = [&](uint32_t j) {                 // two 128-dim halves of key tile j
                for (uint32_t h = 0; h < 2; ++h) {
                    const uint32_t n = j * 2u + h, slot = n % kKSlots, use = n / kKSlots;
                    if (use > 0 && !mbar_wait(bar(kBarKEmpty + slot), (use - 1u) & 1u, abort_flag)) return false;
                    mbar_expect_tx(bar(kBarKFull + slot), kSlotBytes);
                    for (uint32_t a = 0; a < 2; ++a)
                        tma_load_3d(base + kOffK + slot * kSlotBytes + a * kKAtomBytes, &map_k, bar(kBarKFull + slot),
                                    int((h * 2u + a) * 64u), int(j * kBN), int(kv));
                }
                return true;
            };
            auto load_v = [&](uint32_t j) {                 // two 64-key halves of key tile j
                for (uint32_t g = 0; g < 2; ++g) {
                    const uint32_t n = j * 2u + g, slot = n % kVSlots, use = n / kVSlots;
                    if (use > 0 && !mbar_wait(bar(kBarVEmpty + slot), (use - 1u) & 1u, abort_flag)) return false;
                    mbar_expect_tx(bar(kBarVFull + slot), kSlotBytes);
                    for (uint32_t a = 0; a < 4; ++a)
                        tma_load_3d(base + kOffV + slot * kSlotBytes + a * kVAtomBytes, &map_v, bar(kBarVFull + slot),
                                    int(a * 64), int(j * kBN + g * 64u), int(kv));
                }
                return true;
            };
            bool ok = load_k(0);
            for (uint32_t j = 0; ok && j < ntiles; ++j) {
                if (j + 1u < ntiles) ok = load_k(j + 1u);
                if (ok) ok = load_v(j);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(kBM, kBN, false);
            constexpr uint32_t idesc_pv = instr_desc(kBM, kHeadDim, true);
            bool ok = mbar_wait(bar(kBarQ), 0, abort_flag);
            auto issue_s = [&](uint32_t j) {
                const uint32_t b = j % kSBufs;
                // S buffer b is free once the softmax threads have read tile j-2 out of it
                if (j >= kSBufs && !mbar_wait(bar(kBarSFree + b), (j / kSBufs - 1u) & 1u, abort_flag)) return false;
                tc_fence_after();
                for (uint32_t h = 0; h < 2; ++h) {
                    const uint32_t n = j * 2u + h, slot = n % kKSlots;
                    if (!mbar_wait(bar(kBarKFull + slot), (n / kKSlots) & 1u, abort_flag)) return false;
                    tc_fence_after();
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks) {
                        const uint32_t atom = ks >> 2, inner = (ks & 3u) * 32u;
                        const uint64_t ad = smem_desc(base + kOffQ + (h * 2u + atom) * kAtomBytesQ + inner, 16, 1024);
                        const uint64_t bd = smem_desc(base + kOffK + slot * kSlotBytes + atom * kKAtomBytes + inner, 16, 1024);
                        tc_mma(tmem + kColS + b * kBN, ad, bd, idesc_s, (h | ks) ? 1u : 0u);
                    }
                    tc_commit(bar(kBarKEmpty + slot));
                }
                tc_commit(bar(kBarSFull + b));
                return true;
            };
            auto issue_pv = [&](uint32_t i) {
                if (!mbar_wait(bar(kBarPFull), i & 1u, abort_flag)) return false;
                for (uint32_t g = 0; g < 2; ++g) {
                    const uint32_t n = i * 2u + g, slot = n % kVSlots;
                    if (!mbar_wait(bar(kBarVFull + slot), (n / kVSlots) & 1u, abort_flag)) return false;
                    tc_fence_after();
#pragma unroll
                    for (uint32_t h = 0; h < 4; ++h) {
                        // A = P [128 x 128] bf16 in shared memory, K-major: atom g holds keys 64g..64g+63,
                        // 32 bytes per 16-key step.
                        // B = V slot [64 keys x 256 d] MN-major: atoms of 64 d are kVAtomBytes apart
                        // (leading offset), groups of 8 keys 1024 B apart (stride offset); 16 keys = 2048 B
                        const uint64_t ad = smem_desc(base + kOffP + g * kPAtomBytes + h * 32u, 16, 1024);
                        const uint64_t bd = smem_desc(base + kOffV + slot * kSlotBytes + h * 2048u, kVAtomBytes, 1024);
                        tc_mma(tmem + kColO, ad, bd, idesc_pv, (i | g | h) ? 1u : 0u);
                    }
                    tc_commit(bar(kBarVEmpty + slot));
                }
                tc_commit(bar(kBarPvDone));
                return true;
            };
            // The score MMAs run up to two tiles ahead of the softmax (their buffer is released as soon
            // as it has been read); P.V of a tile follows as soon as its P is in shared memory.
            if (ok) ok = issue_s(0);
            if (ok && ntiles > 1u) ok = issue_s(1);
            for (uint32_t j = 0; ok && j < ntiles; ++j) {
                ok = issue_pv(j);
                if (ok && j + 2u < ntiles) ok = issue_s(j + 2u);
            }
        }
    } else {
        softmax_rows<SingleForm>(smem, bars, tmem, p, warp, lane, head, r0, rows_here, ntiles, abort_flag);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- CTA-pair form (cluster of two, tcgen05 cta_group::2) ------------------------------------
// The two CTAs of a pair own the same 128 query rows of two heads of one KV group (heads 2g and
// 2g+1), so every K and V tile serves 256 MMA rows: CTA r loads keys [64r, 64r+64) of each K tile
// and dims [128r, 128r+128) of each V tile (32 KiB instead of 64 KiB per tile and SM from L2), and
// the pair's tensor cores read the other half from the peer's shared memory.  The leader (rank 0)
// issues every MMA (M256: N128 for the scores, N256 for P.V); each CTA keeps its own Q, P, S and O.
// With the rings at half size there is room for TWO P buffers, which is what makes the form pay:
// P ready -> P.V done -> P buffer free is a chain through the leader, and with one buffer that
// chain was the tile period.  Hand-offs: `full` barriers live in the leader (its producer arrives
// expecting the bytes of both CTAs; both CTAs' copies complete on them); `empty`, `S full` and
// `P.V done` are one tcgen05.commit that arrives in both CTAs; `S free` and `P full` live in the
// leader and count one arrival per softmax warp of both CTAs.
constexpr uint32_t kPpKSlots = 3, kPpVSlots = 3, kPpPBufs = 2;
constexpr uint32_t kPvWarp = 10, kPpThreads = 352;   // TMA warp, score-MMA warp, 8 softmax warps, P.V-MMA warp
constexpr uint32_t kPpSlotBytes = 16384;   // K slot: 64 keys x 128 dims; V slot: 64 keys x 128 d
constexpr uint32_t kPpAtomBytes = 8192;    // one 64-wide swizzle atom of a slot (64 keys x 128 B)
constexpr uint32_t kPpOffQ = 0;
constexpr uint32_t kPpOffK = kPpOffQ + kQBytes;
constexpr uint32_t kPpOffV = kPpOffK + kPpKSlots * kPpSlotBytes;
constexpr uint32_t kPpOffP = kPpOffV + kPpVSlots * kPpSlotBytes;
constexpr uint32_t kPpOffBar = kPpOffP + kPpPBufs * kPBytes;
constexpr uint32_t kPpOffPair = kPpOffBar + 256;
constexpr uint32_t kPpSmem = kPpOffPair + 2 * 256 * 4;
static_assert(kPpSmem <= 232448, "shared memory budget");
enum : uint32_t { kPpBarQ = 0, kPpBarKFull = 1, kPpBarKEmpty = kPpBarKFull + kPpKSlots,
                  kPpBarVFull = kPpBarKEmpty + kPpKSlots, kPpBarVEmpty = kPpBarVFull + kPpVSlots,
                  kPpBarSFull = kPpBarVEmpty + kPpVSlots, kPpBarSFree = kPpBarSFull + kSBufs,
                  kPpBarPFull = kPpBarSFree + kSBufs, kPpBarPvDone = kPpBarPFull + kPpPBufs,
                  kPpBarCount = kPpBarPvDone + kPpPBufs };
static_assert(8 * kPpBarCount + 16 <= 256, "barrier block");

struct PairForm {
    static constexpr uint32_t kOffQ = kPpOffQ, kOffP = kPpOffP, kOffPair = kPpOffPair, kPBufs = kPpPBufs;
    static constexpr bool kArriveAtLeader = true;
    static constexpr uint32_t kBarSFull = kPpBarSFull, kBarSFree = kPpBarSFree, kBarPFull = kPpBarPFull,
                              kBarPvDone = kPpBarPvDone;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPpThreads, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t base = s2u(smem);
    const uint32_t bars = base + kPpOffBar;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kPpOffBar + 8 * kPpBarCount);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kPpOffBar + 8 * kPpBarCount + 8);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0u;

    // blockIdx.x = 16 * tile + head: the pair (2g, 2g+1) is one cluster, both of KV group head >> 3
    const uint32_t qt = p.n_qtiles - 1u - (blockIdx.x >> 4);
    const uint32_t head = blockIdx.x & 15u, kv = head >> 3;
    const uint32_t r0 = qt * kBM;
    const uint32_t rows_here = min(kBM, p.rows - r0);
    const uint32_t visible = p.context_base + r0 + rows_here;
    const uint32_t ntiles = (visible + kBN - 1u) / kBN;

    if (threadIdx.x == 0) {
        mbar_init(bar(kPpBarQ), 1);
        for (uint32_t s = 0; s < kPpKSlots; ++s) {
            mbar_init(bar(kPpBarKFull + s), 1);
            mbar_init(bar(kPpBarKEmpty + s), 1);
        }
        for (uint32_t s = 0; s < kPpVSlots; ++s) {
            mbar_init(bar(kPpBarVFull + s), 1);
            mbar_init(bar(kPpBarVEmpty + s), 1);
        }
        for (uint32_t s = 0; s < kSBufs; ++s) {
            mbar_init(bar(kPpBarSFull + s), 1);
            mbar_init(bar(kPpBarSFree + s), 2u * kSoftmaxThreads / 32u);   // one arrival per softmax warp of both CTAs
        }
        for (uint32_t s = 0; s < kPpPBufs; ++s) {
            mbar_init(bar(kPpBarPFull + s), 2u * kSoftmaxThreads / 32u);
            mbar_init(bar(kPpBarPvDone + s), 1);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {   // the same warp of both CTAs allocates the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s2u(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs are initialised before any remote arrival
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (one per CTA; every copy completes on the leader's barrier) ----------------
        if (lane == 0) {
            if (leader) mbar_expect_tx(bar(kPpBarQ), 2u * kQBytes);
            const uint32_t qfull = map_to_cta(bar(kPpBarQ), 0u);
            for (uint32_t a = 0; a < 4; ++a)
                tma_load_3d_pair(base + kPpOffQ + a * kAtomBytesQ, &map_q, qfull, int(a * 64), int(head), int(r0));
            auto load_k = [&](uint32_t j) {                 // this CTA's 64 keys of tile j, two 128-dim halves
                for (uint32_t h = 0; h < 2; ++h) {
                    const uint32_t n = j * 2u + h, slot = n % kPpKSlots, use = n / kPpKSlots;
                    if (use > 0 && !mbar_wait(bar(kPpBarKEmpty + slot), (use - 1u) & 1u, abort_flag)) return false;
                    if (leader) mbar_expect_tx(bar(kPpBarKFull + slot), 2u * kPpSlotBytes);
                    const uint32_t full = map_to_cta(bar(kPpBarKFull + slot), 0u);
                    for (uint32_t a = 0; a < 2; ++a)
                        tma_load_3d_pair(base + kPpOffK + slot * kPpSlotBytes + a * kPpAtomBytes, &map_k, full,
                                         int((h * 2u + a) * 64u), int(j * kBN + rank * 64u), int(kv));
                }
                return true;
            };
            auto load_v = [&](uint32_t j) {                 // this CTA's 128 dims of tile j, two 64-key halves
                for (uint32_t g = 0; g < 2; ++g) {
                    const uint32_t n = j * 2u + g, slot = n % kPpVSlots, use = n / kPpVSlots;
                    if (use > 0 && !mbar_wait(bar(kPpBarVEmpty + slot), (use - 1u) & 1u, abort_flag)) return false;
                    if (leader) mbar_expect_tx(bar(kPpBarVFull + slot), 2u * kPpSlotBytes);
                    const uint32_t full = map_to_cta(bar(kPpBarVFull + slot), 0u);
                    for (uint32_t a = 0; a < 2; ++a)
                        tma_load_3d_pair(base + kPpOffV + slot * kPpSlotBytes + a * kPpAtomBytes, &map_v, full,
                                         int(rank * 128u + a * 64u), int(j * kBN + g * 64u), int(kv));
                }
                return true;
            };
            // in the order the leader's MMAs use them: S_0, S_1, S_2, P.V_0, S_3, P.V_1, ...
            bool ok = load_k(0);
            if (ok && ntiles > 1u) ok = load_k(1);
            if (ok && ntiles > 2u) ok = load_k(2);
            for (uint32_t j = 0; ok && j < ntiles; ++j) {
                ok = load_v(j);
                if (ok && j + 3u < ntiles) ok = load_k(j + 3u);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---------------- score MMAs of the pair ----------------
            constexpr uint32_t idesc_s = instr_desc(2u * kBM, kBN, false);
            bool ok = mbar_wait_cluster(bar(kPpBarQ), 0, abort_flag);
            // S_j goes out as soon as the softmax rows have taken S_{j-2} into registers (the start of
            // their tile j-2): the score MMAs stay a full softmax tile ahead of the P.V chain.
            for (uint32_t j = 0; ok && j < ntiles; ++j) {
                const uint32_t b = j % kSBufs;
                // S buffer b of BOTH CTAs is free once their softmax threads have read tile j-2 out of it
                if (j >= kSBufs && !mbar_wait_cluster(bar(kPpBarSFree + b), (j / kSBufs - 1u) & 1u, abort_flag)) break;
                tc_fence_after();
                for (uint32_t h = 0; ok && h < 2; ++h) {
                    const uint32_t n = j * 2u + h, slot = n % kPpKSlots;
                    if (!mbar_wait_cluster(bar(kPpBarKFull + slot), (n / kPpKSlots) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks) {
                        const uint32_t atom = ks >> 2, inner = (ks & 3u) * 32u;
                        const uint64_t ad = smem_desc(base + kPpOffQ + (h * 2u + atom) * kAtomBytesQ + inner, 16, 1024);
                        const uint64_t bd = smem_desc(base + kPpOffK + slot * kPpSlotBytes + atom * kPpAtomBytes + inner, 16, 1024);
                        tc_mma_pair(tmem + kColS + b * kBN, ad, bd, idesc_s, (h | ks) ? 1u : 0u);
                    }
                    tc_commit_both(bar(kPpBarKEmpty + slot));
                }
                if (ok) tc_commit_both(bar(kPpBarSFull + b));
            }
        }
    } else if (warp == kPvWarp) {
        if (lane == 0 && leader) {
            // ---------------- P.V MMAs of the pair: a second issuing thread, so that the tensor pipe is fed
            // by one thread while the other waits on a barrier or commits ----------------
            constexpr uint32_t idesc_pv = instr_desc(2u * kBM, kHeadDim, true);
            bool ok = true;
            for (uint32_t i = 0; ok && i < ntiles; ++i) {
                const uint32_t pb = i % kPpPBufs;
                if (!mbar_wait_cluster(bar(kPpBarPFull + pb), (i / kPpPBufs) & 1u, abort_flag)) break;
                for (uint32_t g = 0; g < 2; ++g) {
                    const uint32_t n = i * 2u + g, slot = n % kPpVSlots;
                    if (!mbar_wait_cluster(bar(kPpBarVFull + slot), (n / kPpVSlots) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t h = 0; h < 4; ++h) {
                        // A = each CTA's own P buffer (K-major, atom g = keys 64g..64g+63, 32 bytes per
                        // 16-key step); B = V slot [64 keys x 128 d] MN-major: atoms of 64 d are
                        // kPpAtomBytes apart (leading offset), groups of 8 keys 1024 B apart; 16 keys = 2048 B
                        const uint64_t ad = smem_desc(base + kPpOffP + pb * kPBytes + g * kPAtomBytes + h * 32u, 16, 1024);
                        const uint64_t bd = smem_desc(base + kPpOffV + slot * kPpSlotBytes + h * 2048u, kPpAtomBytes, 1024);
                        tc_mma_pair(tmem + kColO, ad, bd, idesc_pv, (i | g | h) ? 1u : 0u);
                    }
                    tc_commit_both(bar(kPpBarVEmpty + slot));
                }
                if (ok) tc_commit_both(bar(kPpBarPvDone + pb));
            }
        }
    } else {
        softmax_rows<PairForm>(smem, bars, tmem, p, warp, lane, head, r0, rows_here, ntiles, abort_flag);
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
    // or read its K/V halves
    cluster_sync_all();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------
// 3-D bf16 tensor map {256 dims, d1, d2} with a {64, box1, 1} box and the 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* ptr, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                     uint64_t stride2_bytes, uint32_t box1, uint32_t box2) {
    EncodeTiled fn = encode_tiled_entry();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {kHeadDim, d1, d2};
    const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    const cuuint32_t box[3] = {64, box1, box2};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace tb

using namespace tb;

extern "C" tatara_status tatara_attn_prefill(tatara_ctx* ctx, void* stream, const void* query,
                                             const void* gate, const void* keys, const void* values,
                                             uint32_t context_base, uint32_t rows, uint32_t capacity,
                                             void* out) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (!query || !gate || !keys || !values || !out)
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_prefill: null buffer");
    if (!aligned(query, 16) || !aligned(gate, 16) || !aligned(keys, 16) || !aligned(values, 16) || !aligned(out, 16))
        return fail(ctx, TATARA_INVALID_BUFFER, "attn_prefill: buffers must be 16-byte aligned");
    if (rows == 0) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_prefill: rows");
    if (capacity == 0 || uint64_t(context_base) + rows > capacity)
        return fail(ctx, TATARA_CONTEXT_OUT_OF_RANGE, "attn_prefill: rows past capacity");
    const uint32_t visible = context_base + rows;
    const bool pair = ctx->attn_prefill_form == 0u;
    CUtensorMap map_q, map_k, map_v;
    // Q [rows][16 heads][256]: box = 64 dims x 1 head x 128 rows
    if (!make_map(&map_q, query, kQHeads, rows, kHeadDim * 2ull, uint64_t(kQHeads) * kHeadDim * 2ull, 1, kBM) ||
        // K, V [2][capacity][256], extent clipped to the visible keys so the tail reads as zero; a CTA of
        // the pair form takes 64 keys of a K tile per copy, the single-CTA form all 128
        !make_map(&map_k, keys, visible, kKvHeads, kHeadDim * 2ull, uint64_t(capacity) * kHeadDim * 2ull,
                  pair ? 64 : kBN, 1) ||
        !make_map(&map_v, values, visible, kKvHeads, kHeadDim * 2ull, uint64_t(capacity) * kHeadDim * 2ull, 64, 1))
        return fail(ctx, TATARA_CUDA_ERROR, "attn_prefill: tensor map encoding failed");
    static bool configured[64] = {false};
    if (!configured[ctx->device & 63]) {
        if (cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kPrefillSmem) != cudaSuccess ||
            cudaFuncSetAttribute(attn_prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kPpSmem) != cudaSuccess)
            return check_launch(ctx, "attn_prefill: shared memory attribute");
        configured[ctx->device & 63] = true;
    }
    PrefillParams pp{};
    pp.gate = static_cast<const __nv_bfloat16*>(gate);
    pp.out = static_cast<__nv_bfloat16*>(out);
    pp.status = ctx->device_status;
    pp.context_base = context_base;
    pp.rows = rows;
    pp.n_qtiles = (rows + kBM - 1u) / kBM;
    if (pair)
        attn_prefill_pair_kernel<<<pp.n_qtiles * kQHeads, kPpThreads, kPpSmem, static_cast<cudaStream_t>(stream)>>>(
            map_q, map_k, map_v, pp);
    else
        attn_prefill_kernel<<<pp.n_qtiles * kQHeads, kPrefillThreads, kPrefillSmem, static_cast<cudaStream_t>(stream)>>>(
            map_q, map_k, map_v, pp);
    return check_launch(ctx, "attn_prefill");
}
