// Mixture-of-experts layer. Placeholder until the kernels land.
#include "jl_internal.cuh"

JL_EXPORT int jl_moe(jl_ctx *ctx, float *, const void *, int, const float *, int, const jl_moe_desc *,
                     int32_t *, float *) {
    return jl_set_err(ctx, JL_DECLINED, "mixture layer not built");
}
JL_EXPORT int jl_moe_dev(jl_ctx *ctx, float *, const void *, int, const float *, int, const jl_moe_desc *,
                         int32_t *, float *, void *) {
    return jl_set_err(ctx, JL_DECLINED, "mixture layer not built");
}
