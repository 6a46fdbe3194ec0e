// MXFP4 decode (1..8 tokens) on the f16 tensor-core path (mma.sync.m16n8k16, f32 accumulate).
//
// An e2m1 code s|e1 e0|m is, bit for bit, the top of an f16 whose exponent field is e1 e0 and whose first
// mantissa bit is m: the half-word (s<<15 | (e1 e0 m)<<9) reads as value * 2^-14, subnormals included (0 and
// 0.5). So the A fragments are made from the packed nibbles with shifts and masks only -- no table, no
// conversion instruction -- and the block's scale 2^(e-127) * 2^14 is applied in f32 to the sum of the
// block's two MMAs. Which element sits in which k-slot of an MMA is free as long as A and B agree: lane t
// of a quad takes bytes 4t..4t+3 of the block's 16 (elements 4t..4t+3 in the low nibbles, 16+4t..16+4t+3
// in the high ones), so its B fragments are two aligned 8-byte pieces of the activation row.
//
// Activations are prepared once per matvec: every 64-element span of a token is scaled by its own power of
// two and split x = hi + lo into two f16 rows, one MMA column each, so ~22 bits of every activation take
// part; the 8 columns serve four tokens; 1 / scale of the span folds in with the block scales. Warps of a
// CTA take different spans of the same 16 rows and meet in shared memory in fixed order (bit-stable).
#include "jl_internal.cuh"
#include <cuda_fp16.h>

// scratch: f16 rows [2 * ntok][k] (hi, lo of each token), then f32 [ntok][k / 64] (1 / scale of each span)
size_t jl_gemv_mxfp4_scratch_bytes(int k, int ntok) {
    return (((size_t)2 * ntok * k * 2 + 255) & ~(size_t)255) + (((size_t)ntok * (k / 64) * 4 + 255) & ~(size_t)255);
}

// One warp per (64-element span, token): x * 2^s = hi + lo in f16, s chosen so the span's amax sits in
// [2^14, 2^15) (f16 neither overflows nor flushes); 1 / 2^s goes to the span's slot of inv_scale.
__global__ void __launch_bounds__(128) mx_xprep_kernel(const float *__restrict__ X, __half *__restrict__ xh,
                                                       float *__restrict__ inv_scale, int k) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31, sp = blockIdx.x * 4 + (threadIdx.x >> 5), tok = blockIdx.y, nspan = k / 64;
    if (sp >= nspan) return;
    const float2 v = __ldg(reinterpret_cast<const float2 *>(X + (size_t)tok * k + (size_t)sp * 64) + lane);
    float amax = fmaxf(fabsf(v.x), fabsf(v.y));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    int sh = 14 - ((int)((__float_as_uint(amax) >> 23) & 0xFF) - 127);
    if (amax == 0.f || !(amax < __int_as_float(0x7f800000))) sh = 0;
    sh = max(-100, min(100, sh));
    const float scale = __uint_as_float((uint32_t)(127 + sh) << 23);
    const float a = v.x * scale, b = v.y * scale;
    const __half2 hh = __floats2half2_rn(a, b);
    const float2 back = __half22float2(hh);
    const __half2 ll = __floats2half2_rn(a - back.x, b - back.y);
    __half2 *hi = reinterpret_cast<__half2 *>(xh + (size_t)(2 * tok) * k + (size_t)sp * 64);
    hi[lane] = hh;
    reinterpret_cast<__half2 *>(xh + (size_t)(2 * tok + 1) * k + (size_t)sp * 64)[lane] = ll;
    if (lane == 0) inv_scale[(size_t)tok * nspan + sp] = __uint_as_float((uint32_t)(127 - sh) << 23);
}

__device__ __forceinline__ void mx_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// four codes in the HIGH nibbles of v's bytes -> the high bytes of their f16 images
__device__ __forceinline__ uint32_t mx_hbytes(uint32_t v) { return ((v & 0x70707070u) >> 3) | (v & 0x80808080u); }

// grid (row groups of 16, token groups of 4); WARPS warps split the row's 64-element spans.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) gemv_mxfp4_mma_kernel(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ eplane,
                                                                    int e_stride, const __half *__restrict__ xh,
                                                                    const float *__restrict__ inv_scale, float *__restrict__ Y,
                                                                    int nrows, int k, int ntok) {
    __shared__ float red[WARPS][16][4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row_a = min((int)blockIdx.x * 16 + g, nrows - 1), row_b = min((int)blockIdx.x * 16 + g + 8, nrows - 1);
    const int tok0 = blockIdx.y * 4;
    const int nspan = k / 64, nblk = k / 32;
    const uint8_t *ca = codes + (size_t)row_a * nblk * 16 + t * 4, *cb = codes + (size_t)row_b * nblk * 16 + t * 4;
    const uint8_t *ea = eplane + (size_t)row_a * e_stride, *eb = eplane + (size_t)row_b * e_stride;
    // this lane's B column g: row 2 * tok0 + g of the f16 activations (token tok0 + g/2, part hi/lo)
    const bool blive = 2 * tok0 + g < 2 * ntok;
    const __half *xb = xh + (size_t)(blive ? 2 * tok0 + g : 0) * k + 4 * t;

    // A warp's unit of work is MX_U consecutive spans (64 elements each): all of a unit's loads are issued
    // before the first is used, and the next unit's weights fly while this one is multiplied.
    constexpr int MX_U = 4;
    const int nunit = (nspan + MX_U - 1) / MX_U;
    const int mytok = tok0 + t;
    const float *isc = inv_scale + (size_t)(mytok < ntok ? mytok : 0) * nspan;
    uint32_t wa[MX_U][2], wb[MX_U][2], sea[MX_U], seb[MX_U];
    auto load_w = [&](int unit) {
#pragma unroll
        for (int u = 0; u < MX_U; u++) {
            const int sp = unit * MX_U + u;
            const bool in = sp < nspan;
            wa[u][0] = in ? __ldg(reinterpret_cast<const uint32_t *>(ca + (size_t)sp * 32)) : 0u;
            wa[u][1] = in ? __ldg(reinterpret_cast<const uint32_t *>(ca + (size_t)sp * 32 + 16)) : 0u;
            wb[u][0] = in ? __ldg(reinterpret_cast<const uint32_t *>(cb + (size_t)sp * 32)) : 0u;
            wb[u][1] = in ? __ldg(reinterpret_cast<const uint32_t *>(cb + (size_t)sp * 32 + 16)) : 0u;
            sea[u] = in ? *reinterpret_cast<const uint16_t *>(ea + 2 * sp) : 0u;
            seb[u] = in ? *reinterpret_cast<const uint16_t *>(eb + 2 * sp) : 0u;
        }
    };
    int unit = warp;
    if (unit < nunit) load_w(unit);                      // weights first: they do not depend on the kernel in front
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the f16 activation rows come from the kernel in front

    float acc_a = 0.f, acc_b = 0.f;
    for (; unit < nunit; unit += WARPS) {
        uint2 x0[MX_U][2], x1[MX_U][2];
        float is[MX_U];
        uint32_t ua[MX_U][2], ub[MX_U][2], ce_a[MX_U], ce_b[MX_U];
#pragma unroll
        for (int u = 0; u < MX_U; u++) {
            const int sp = unit * MX_U + u;
            const bool in = blive && sp < nspan;
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const __half *xp = xb + (size_t)sp * 64 + b * 32;
                x0[u][b] = in ? *reinterpret_cast<const uint2 *>(xp) : make_uint2(0u, 0u);          // elements 4t..4t+3
                x1[u][b] = in ? *reinterpret_cast<const uint2 *>(xp + 16) : make_uint2(0u, 0u);     // elements 16+4t..16+4t+3
            }
            is[u] = (mytok < ntok && sp < nspan) ? isc[sp] : 0.f;
            ua[u][0] = wa[u][0]; ua[u][1] = wa[u][1]; ub[u][0] = wb[u][0]; ub[u][1] = wb[u][1];
            ce_a[u] = sea[u]; ce_b[u] = seb[u];
        }
        if (unit + WARPS < nunit) load_w(unit + WARPS);
#pragma unroll
        for (int u = 0; u < MX_U; u++) {
            float sa = 0.f, sb = 0.f;
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const uint32_t hla = mx_hbytes(ua[u][b] << 4), hha = mx_hbytes(ua[u][b]);     // low / high nibbles of row g
                const uint32_t hlb = mx_hbytes(ub[u][b] << 4), hhb = mx_hbytes(ub[u][b]);     // ... of row g + 8
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                // k-slots (2t, 2t+1 | 2t+8, 2t+9) = elements (4t, 4t+1 | 4t+2, 4t+3), then the same + 16
                mx_mma(c, __byte_perm(hla, 0u, 0x1404), __byte_perm(hlb, 0u, 0x1404), __byte_perm(hla, 0u, 0x3424),
                       __byte_perm(hlb, 0u, 0x3424), x0[u][b].x, x0[u][b].y);
                mx_mma(c, __byte_perm(hha, 0u, 0x1404), __byte_perm(hhb, 0u, 0x1404), __byte_perm(hha, 0u, 0x3424),
                       __byte_perm(hhb, 0u, 0x3424), x1[u][b].x, x1[u][b].y);
                // 2^(e - 127) * 2^14 as an f32 (an all-zero block may carry any byte: keep the exponent field legal)
                const uint32_t e_a = min((ce_a[u] >> (8 * b)) & 0xFFu, 240u), e_b = min((ce_b[u] >> (8 * b)) & 0xFFu, 240u);
                sa = fmaf(c[0] + c[1], __uint_as_float((e_a + 14u) << 23), sa);     // hi + lo columns of token t
                sb = fmaf(c[2] + c[3], __uint_as_float((e_b + 14u) << 23), sb);
            }
            acc_a = fmaf(sa, is[u], acc_a);
            acc_b = fmaf(sb, is[u], acc_b);
        }
    }
    red[warp][g][t] = acc_a;
    red[warp][g + 8][t] = acc_b;
    __syncthreads();
    for (int i = tid; i < 64; i += WARPS * 32) {
        const int r = i >> 2, j = i & 3;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) sum += red[w][r][j];      // fixed order
        const int row = blockIdx.x * 16 + r, tok = tok0 + j;
        if (row < nrows && tok < ntok) Y[(size_t)tok * nrows + row] = sum;
    }
}

int jl_launch_gemv_mxfp4(jl_ctx *ctx, float *out_dev, const uint8_t *codes, const uint8_t *eplane, int e_stride,
                         const float *x_dev, int nrows, int k, int ntok, cudaStream_t s) {
    const size_t need = jl_gemv_mxfp4_scratch_bytes(k, ntok);
    if (ctx->scratch_cap < need)
        return jl_set_err(ctx, JL_ENOMEM, "decode scratch holds %zu bytes, %d x %d token(s) need %zu (jl_reserve sizes it)",
                          ctx->scratch_cap, k, ntok, need);
    __half *xh = (__half *)ctx->scratch;
    float *inv_scale = (float *)((uint8_t *)ctx->scratch + (((size_t)2 * ntok * k * 2 + 255) & ~(size_t)255));
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    const int nattr = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((k / 64 + 3) / 4, ntok); cfg.blockDim = dim3(128); cfg.stream = s; cfg.attrs = at; cfg.numAttrs = nattr;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, mx_xprep_kernel, x_dev, xh, inv_scale, k));
    ctx->st.launches++;
    const int nspan = k / 64;
    const int warps = nspan >= 32 ? 8 : (nspan >= 16 ? 4 : (nspan >= 8 ? 2 : 1));
    cfg.gridDim = dim3((nrows + 15) / 16, (ntok + 3) / 4); cfg.blockDim = dim3(warps * 32);
    const __half *xhc = xh;
    const float *isc = inv_scale;
    if (warps == 8) JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_mxfp4_mma_kernel<8>, codes, eplane, e_stride, xhc, isc, out_dev, nrows, k, ntok));
    else if (warps == 4) JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_mxfp4_mma_kernel<4>, codes, eplane, e_stride, xhc, isc, out_dev, nrows, k, ntok));
    else if (warps == 2) JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_mxfp4_mma_kernel<2>, codes, eplane, e_stride, xhc, isc, out_dev, nrows, k, ntok));
    else JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_mxfp4_mma_kernel<1>, codes, eplane, e_stride, xhc, isc, out_dev, nrows, k, ntok));
    ctx->st.launches++;
    return JL_OK;
}
