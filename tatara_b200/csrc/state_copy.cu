// Segment gather / scatter for state snapshots: one launch copies a whole list of
// (source, destination, bytes) segments device to device at copy bandwidth.
//
// The reference moves a request's state between its decode slot and a prefix-cache arena as a
// list of blit copies, one per segment (60 gated-delta + 40 attention segments for the 40-layer
// schedule; src/runtime/prefix_state_transfer.cpp:236-262, backend::metal::copy_buffer).  Here the
// list is a kernel argument: the segments are cut into 32 KiB chunks and the chunks are dealt
// round-robin over a grid that fills every SM, so that short segments (48 KiB of conv state)
// and long ones (128 MiB of keys) stream together.
#include "common.cuh"

namespace tb {

constexpr uint32_t kCopyMaxSegments = 120;
constexpr uint32_t kCopyThreads = 256, kCopyChunkBytes = 32768, kCopyPerThread = kCopyChunkBytes / (kCopyThreads * 16);

struct CopyParams {
    const uint8_t* src[kCopyMaxSegments];
    uint8_t* dst[kCopyMaxSegments];
    uint64_t bytes[kCopyMaxSegments];
    uint32_t first_chunk[kCopyMaxSegments + 1];   // running chunk count
    uint32_t n;
};
static_assert(sizeof(CopyParams) <= 4000, "kernel parameter space");

__global__ void __launch_bounds__(kCopyThreads) state_copy_kernel(const __grid_constant__ CopyParams p) {
    __shared__ uint32_t first_chunk[kCopyMaxSegments + 1];
    for (uint32_t i = threadIdx.x; i <= p.n; i += kCopyThreads) first_chunk[i] = p.first_chunk[i];
    __syncthreads();
    const uint32_t total = first_chunk[p.n];
    for (uint32_t chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
        uint32_t lo = 0, hi = p.n;   // last segment with first_chunk <= chunk
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (first_chunk[mid] <= chunk) lo = mid; else hi = mid;
        }
        const uint64_t offset = uint64_t(chunk - first_chunk[lo]) * kCopyChunkBytes;
        const uint64_t left = p.bytes[lo] - offset;
        const uint32_t vecs = uint32_t(left < kCopyChunkBytes ? left : kCopyChunkBytes) >> 4;
        const uint4* s = reinterpret_cast<const uint4*>(p.src[lo] + offset);
        uint4* d = reinterpret_cast<uint4*>(p.dst[lo] + offset);
        uint4 v[kCopyPerThread];
#pragma unroll
        for (uint32_t i = 0; i < kCopyPerThread; ++i) {
            const uint32_t at = i * kCopyThreads + threadIdx.x;
            if (at < vecs) v[i] = __ldcs(s + at);
        }
#pragma unroll
        for (uint32_t i = 0; i < kCopyPerThread; ++i) {
            const uint32_t at = i * kCopyThreads + threadIdx.x;
            if (at < vecs) __stcs(d + at, v[i]);
        }
    }
}

} // namespace tb

using namespace tb;

extern "C" tatara_status tatara_state_copy(tatara_ctx* ctx, void* stream, const tatara_copy_segment* segments,
                                           uint32_t n_segments) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    if (segments == nullptr || n_segments == 0)
        return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "state_copy: no segments");
    // validate the whole list before the first launch
    for (uint32_t i = 0; i < n_segments; ++i) {
        const tatara_copy_segment& s = segments[i];
        if (!s.src || !s.dst || !aligned(s.src, 16) || !aligned(s.dst, 16))
            return fail(ctx, TATARA_INVALID_BUFFER, "state_copy: null or misaligned segment");
        if (s.bytes == 0 || s.bytes % 16u != 0 || s.bytes > (uint64_t(1) << 40))
            return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "state_copy: segment length");
    }
    for (uint32_t base = 0; base < n_segments; base += kCopyMaxSegments) {
        CopyParams p{};
        p.n = n_segments - base < kCopyMaxSegments ? n_segments - base : kCopyMaxSegments;
        uint64_t chunks = 0;
        for (uint32_t i = 0; i < p.n; ++i) {
            const tatara_copy_segment& s = segments[base + i];
            p.src[i] = static_cast<const uint8_t*>(s.src);
            p.dst[i] = static_cast<uint8_t*>(s.dst);
            p.bytes[i] = s.bytes;
            p.first_chunk[i] = uint32_t(chunks);
            chunks += (s.bytes + kCopyChunkBytes - 1) / kCopyChunkBytes;
            if (chunks > 0xFFFFFFFFull) return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "state_copy: too many chunks");
        }
        p.first_chunk[p.n] = uint32_t(chunks);
        const uint64_t cap = uint64_t(ctx->sm_count) * 8u;
        const uint32_t grid = uint32_t(chunks < cap ? chunks : cap);
        state_copy_kernel<<<grid, kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
        const tatara_status st = check_launch(ctx, "state_copy");
        if (st != TATARA_OK) return st;
    }
    return TATARA_OK;
}
