// Prefill kernels (tcgen05). Placeholder until the kernel lands: reports "not
// supported" so selection falls through to the decode family.
#include "jl_internal.cuh"

int jl_gemm_tc5_supported(uint32_t, int, int, int) { return 0; }
int jl_gemm_tc5_choice(jl_ctx *ctx, uint32_t, int, int, int, jl_choice *) {
    return jl_set_err(ctx, JL_DECLINED, "tcgen05 family not built");
}
int jl_launch_gemm_tc5(jl_ctx *ctx, void *, int, const jl_weight *, int, const void *, int, int, cudaStream_t) {
    return jl_set_err(ctx, JL_DECLINED, "tcgen05 family not built");
}
