// Causal block prefill attention (tcgen05 / TMEM / TMA).
#include "common.cuh"

using namespace tb;

extern "C" tatara_status tatara_attn_prefill(tatara_ctx* ctx, void*, const void*, const void*,
                                             const void*, const void*, uint32_t, uint32_t, uint32_t,
                                             void*) {
    if (ctx == nullptr) return TATARA_INVALID_BUFFER;
    return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "attn_prefill: kernel not built in this revision");
}
