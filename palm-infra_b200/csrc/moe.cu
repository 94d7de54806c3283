#include "b200w4_internal.cuh"
extern "C" {
int b2w4_moe_forward(b2w4_ctx* ctx, const float*, int, int, int, const void*, int, int, int,
                     const b2w4_weight*, const b2w4_weight*, float*, int, float*, int32_t*,
                     float*) {
    return b2w4_fail(ctx, B2W4_E_INVALID, "moe: not built yet");
}
int b2w4_moe_select_routes(b2w4_ctx* ctx, const float*, int, int, int, int32_t*, float*) {
    return b2w4_fail(ctx, B2W4_E_INVALID, "moe: not built yet");
}
}
