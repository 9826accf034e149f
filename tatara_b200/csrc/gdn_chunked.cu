// Chunk-64 (WY / UT transform) evaluation of the Gated DeltaNet recurrence.
#include "common.cuh"

namespace tb {

tatara_status launch_gdn_chunked(tatara_ctx* ctx, cudaStream_t, const __nv_bfloat16*,
                                 const __nv_bfloat16*, const float*, const float*, const float*,
                                 __nv_bfloat16*, float*, uint32_t) {
    return fail(ctx, TATARA_INVALID_DISPATCH_EXTENT, "gdn_prefill: chunked kernel not built in this revision");
}

} // namespace tb
