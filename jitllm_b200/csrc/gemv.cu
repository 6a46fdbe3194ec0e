// Decode kernels: out[tok][row] = dot(dequant(W[row]), x[tok]).
//
// Two families (jl_kernel):
//   JL_K_SIMT  one warp per row, weights decoded exactly as quant.Dequant32
//              does (format/quant/dequant.go:148-174,367-397), f32 FMA, warp
//              shuffle reduction. Serves every shape; the in-library check.
//   JL_K_MMA   the HBM-bound decode kernel. B200 moves ~12e12 4-bit weights a
//              second against ~36e12 lane-instructions, so a SIMT decode
//              (>= 3 instructions a weight) cannot keep up with HBM3e; the
//              multiply-accumulate goes to the tensor cores instead:
//                - a warp owns 16 rows x one 256-element super-block; each lane
//                  pulls whole 16-byte chunks of the raw 144-byte block with
//                  128-bit loads (the header chunk + two code chunks per row);
//                - nibbles become exact f16 integers sc*q with one LOP3 (OR into
//                  the mantissa of 1024.0) and one HFMA2 per two weights;
//                - activations are split x = hi + lo into two f16 (22 bits) and
//                  pre-arranged in shared memory in mma.sync B-fragment order;
//                - mma.sync.m16n8k16 accumulates sum(sc*q*x) over the super-block
//                  in f32; d, dmin and the sub-block minimums (a second tiny MMA
//                  against per-sub-block activation sums) are applied in f32;
//                - warps of a CTA cover different super-blocks of the same 16
//                  rows and meet through shared memory in fixed order, so the
//                  result is run-to-run bit-stable.
#include "jl_internal.cuh"

#include <stdio.h>

// ------------------------------------------------------------------ helpers

__device__ __forceinline__ uint4 ldg16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t u) {
    return __half2float(__ushort_as_half(u));
}

// e2m1 doubled, format/quant/dequant.go:266-268.
__device__ __constant__ float k_mxfp4_f[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f,
                                               0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};

__host__ __device__ static inline int q8_span_pos(int kk) {
    int blk = kk >> 5, within = kk & 31;
    int half = within >> 4, r16 = within & 15;
    int t = r16 >> 2, byte = r16 & 3;
    return t * 16 + (blk * 2 + half) * 4 + byte;
}

// --------------------------------------------------------------- SIMT family

// One warp per (row, token). Each lane walks 32-element sub-blocks.
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) gemv_simt_kernel(const uint8_t *__restrict__ data,
                                                        const uint8_t *__restrict__ scales, int scale_stride,
                                                        const float *__restrict__ X, float *__restrict__ Y,
                                                        int nrows, int k, int ntok) {
    int warp = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5);
    int lane = threadIdx.x & 31;
    int tok = blockIdx.y;
    if (warp >= nrows || tok >= ntok) return;
    int row = warp;
    const float *x = X + (size_t)tok * k;
    int nsub = k / 32;
    float acc = 0.f;
    for (int si = lane; si < nsub; si += 32) {
        const float *xs = x + si * 32;
        if (TYPE == JL_TYPE_Q4_K) {
            const uint8_t *blk = data + ((size_t)row * (nsub / 8) + (si >> 3)) * 144;
            int s = si & 7;
            float d = half_bits_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
            float dmin = half_bits_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
            const uint8_t *q = blk + 4;
            uint8_t sc, m;
            if (s < 4) { sc = q[s] & 63; m = q[s + 4] & 63; }
            else { sc = (uint8_t)((q[s + 4] & 0xF) | ((q[s - 4] >> 6) << 4)); m = (uint8_t)((q[s + 4] >> 4) | ((q[s] >> 6) << 4)); }
            float d1 = __fmul_rn(d, (float)sc), mn = __fmul_rn(dmin, (float)m);
            const uint8_t *grp = blk + 16 + (s >> 1) * 32;
            for (int l = 0; l < 32; l++) {
                int code = (s & 1) ? (grp[l] >> 4) : (grp[l] & 0xF);
                float w = __fsub_rn(__fmul_rn(d1, (float)code), mn);
                acc = fmaf(w, xs[l], acc);
            }
        } else if (TYPE == JL_TYPE_Q8_0) {
            const uint8_t *span = data + (size_t)row * k + (size_t)(si >> 1) * 64;
            float d = half_bits_to_float(((const uint16_t *)scales)[(size_t)row * scale_stride + si]);
            for (int l = 0; l < 32; l++) {
                float w = __fmul_rn(d, (float)(int8_t)span[q8_span_pos((si & 1) * 32 + l)]);
                acc = fmaf(w, xs[l], acc);
            }
        } else {  // MXFP4
            const uint8_t *c = data + ((size_t)row * nsub + si) * 16;
            int e = scales[(size_t)row * scale_stride + si];
            float d = __int_as_float(e >= 2 ? ((e - 1) << 23) : (e == 1 ? 0x00400000 : 0x00200000));  // 2^(e-128)
            for (int l = 0; l < 16; l++) {
                acc = fmaf(k_mxfp4_f[c[l] & 0xF] * d, xs[l], acc);
                acc = fmaf(k_mxfp4_f[c[l] >> 4] * d, xs[l + 16], acc);
            }
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) Y[(size_t)tok * nrows + row] = acc;
}

// ---------------------------------------------------------------- MMA family

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// Shared-memory geometry of the Q4_K decode kernel, per super-block:
//   xfrag  4 lanes x 17 slots x 16 B (16 used; the 17th staggers the banks):
//          slot (t, hl*8 + c) = {hi(x0,x2), hi(x1,x3), lo(x0,x2), lo(x1,x3)} of the
//          four activations e0..e0+3, e0 = 256 sb + 64 t + 32 hl + 4 c -- what the
//          lane holding code word c of group t multiplies against.
//   sxfrag 4 lanes x 8 B: {hi(S[2t], S[2t+1]), lo(...)}, S = sub-block sums / 64.
#define Q4K_XF_SB_BYTES (4 * 17 * 16)
#define Q4K_SX_SB_BYTES (4 * 8)

// Per-lane constants of one row's super-block: multipliers that turn the
// "nibble OR 1024.0" patterns into sc*q, and the minimum pair as f16.
struct q4k_rowk {
    uint32_t me, ae, mo, ao;  // half2 broadcast: even sub-block (low nibbles), odd (high nibbles)
    uint32_t hm;              // half2 (m[2t], m[2t+1])
    float d, dmin;
};

__device__ __forceinline__ q4k_rowk q4k_prepare(const uint4 &h, int t) {
    // h.x = d | dmin << 16; h.y, h.z, h.w = the twelve scale bytes q[0..11].
    // Sub-blocks 2t and 2t+1 (format/quant/dequant.go:360-365):
    //   j < 4 : sc = q[j] & 63,                      m = q[j+4] & 63
    //   j >= 4: sc = (q[j+4] & 15) | (q[j-4] >> 6) << 4,  m = (q[j+4] >> 4) | (q[j] >> 6) << 4
    int sh = (t & 1) * 16;
    uint32_t a = h.y >> sh, b = h.z >> sh, c = h.w >> sh;
    uint32_t scp, mp;
    if (t < 2) {
        scp = a & 0x3F3Fu;
        mp = b & 0x3F3Fu;
    } else {
        scp = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u);
        mp = ((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
    }
    const uint32_t k1024 = 0x64006400u;          // half2(1024, 1024)
    const uint32_t kscl = 0x2C003C00u;           // half2(1, 1/16)
    const uint32_t kneg = 0xE400E400u;           // half2(-1024, -1024)
    uint32_t hs = hsub2u(__byte_perm(scp, 0x64646464u, 0x4140), k1024);  // (sc_e, sc_o)
    hs = hmul2u(hs, kscl);                                                // (sc_e, sc_o / 16)
    q4k_rowk r;
    r.me = __byte_perm(hs, hs, 0x1010);
    r.mo = __byte_perm(hs, hs, 0x3232);
    r.ae = hmul2u(r.me, kneg);
    r.ao = hmul2u(r.mo, kneg);
    r.hm = hsub2u(__byte_perm(mp, 0x64646464u, 0x4140), k1024);
    __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    float2 f = __half22float2(dd);
    r.d = f.x;
    r.dmin = f.y;
    return r;
}

// Power-of-two scale that brings amax into [2^14, 2^15): the f16 hi/lo split
// then keeps ~22 bits relative to the largest activation, whatever its range.
__device__ __forceinline__ float pow2_scale_for(float amax, float *inv) {
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;  // floor(log2 amax)
    int s = 14 - e;
    if (amax == 0.f || amax != amax) s = 0;
    s = max(-100, min(100, s));
    *inv = __uint_as_float((uint32_t)(127 - s) << 23);
    return __uint_as_float((uint32_t)(127 + s) << 23);
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gemv_q4k_mma_kernel(const uint8_t *__restrict__ W, const float *__restrict__ X, float *__restrict__ Y,
                    int nrows, int nsb, int ntok) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *xfrag = smem;
    uint8_t *sxfrag = smem + (size_t)nsb * Q4K_XF_SB_BYTES;
    float *red = reinterpret_cast<float *>(sxfrag + (size_t)nsb * Q4K_SX_SB_BYTES);  // [WARPS][16]
    float *bcast = red + WARPS * 16;                                                // [WARPS] amax partials

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rg = blockIdx.x, tok = blockIdx.y;
    const int k = nsb * 256;
    const size_t row_bytes = (size_t)nsb * 144;
    const int rowA = min(rg * 16 + g, nrows - 1), rowB = min(rg * 16 + g + 8, nrows - 1);
    const uint8_t *pA = W + (size_t)rowA * row_bytes, *pB = W + (size_t)rowB * row_bytes;

    // 1. Put this warp's first super-block in flight before anything else: the
    //    weights do not depend on the activations.
    int sb = warp;
    uint4 hA, qA0, qA1, hB, qB0, qB1;
    if (sb < nsb) {
        const uint8_t *a = pA + (size_t)sb * 144, *b = pB + (size_t)sb * 144;
        hA = ldg16(a); qA0 = ldg16(a + 16 + 32 * t); qA1 = ldg16(a + 32 + 32 * t);
        hB = ldg16(b); qB0 = ldg16(b + 16 + 32 * t); qB1 = ldg16(b + 32 + 32 * t);
    }

    // 2. Activations: amax -> power-of-two scale -> f16 hi/lo fragments + sub-block sums.
    const float4 *x4 = reinterpret_cast<const float4 *>(X + (size_t)tok * k);
    const int nquad = k / 4;
    float amax = 0.f;
    for (int q = tid; q < nquad; q += WARPS * 32) {
        float4 v = __ldg(x4 + q);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) bcast[warp] = amax;
    __syncthreads();
    amax = bcast[0];
#pragma unroll
    for (int w = 1; w < WARPS; w++) amax = fmaxf(amax, bcast[w]);
    float inv_scale;
    const float scale = pow2_scale_for(amax, &inv_scale);

    for (int q = tid; q < nquad; q += WARPS * 32) {  // nquad is a multiple of 64: whole warps stay together
        float4 v = __ldg(x4 + q);
        v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
        __half2 h02 = __floats2half2_rn(v.x, v.z), h13 = __floats2half2_rn(v.y, v.w);
        float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
        uint4 slot;
        slot.x = *reinterpret_cast<uint32_t *>(&h02);
        slot.y = *reinterpret_cast<uint32_t *>(&h13);
        slot.z = pack_h2(v.x - f02.x, v.z - f02.y);
        slot.w = pack_h2(v.y - f13.x, v.w - f13.y);
        // q = 64 sb + 16 t + 8 hl + c
        int qsb = q >> 6, qt = (q >> 4) & 3, qi = q & 15;
        *reinterpret_cast<uint4 *>(xfrag + (size_t)qsb * Q4K_XF_SB_BYTES + (qt * 17 + qi) * 16) = slot;
        // sub-block sum: the 8 lanes that share (sb, t, hl).
        float s = (v.x + v.y) + (v.z + v.w);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        float so = __shfl_xor_sync(0xffffffffu, s, 8);  // the other nibble half's sub-block
        if ((q & 15) == 0) {                           // hl == 0, c == 0: s = S[2t], so = S[2t+1]
            float s0 = s * 0.015625f, s1 = so * 0.015625f;
            __half2 hh = __floats2half2_rn(s0, s1);
            float2 fh = __half22float2(hh);
            uint2 sx;
            sx.x = *reinterpret_cast<uint32_t *>(&hh);
            sx.y = pack_h2(s0 - fh.x, s1 - fh.y);
            *reinterpret_cast<uint2 *>(sxfrag + (size_t)qsb * Q4K_SX_SB_BYTES + qt * 8) = sx;
        }
    }
    __syncthreads();

    // 3. This warp's super-blocks.
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool bcol = (g == 0);  // lanes that hold B-fragment column 0 (the one token)
    while (sb < nsb) {
        uint4 nhA, nqA0, nqA1, nhB, nqB0, nqB1;
        const int nsbi = sb + WARPS;
        if (nsbi < nsb) {  // next super-block in flight while this one is consumed
            const uint8_t *a = pA + (size_t)nsbi * 144, *b = pB + (size_t)nsbi * 144;
            nhA = ldg16(a); nqA0 = ldg16(a + 16 + 32 * t); nqA1 = ldg16(a + 32 + 32 * t);
            nhB = ldg16(b); nqB0 = ldg16(b + 16 + 32 * t); nqB1 = ldg16(b + 32 + 32 * t);
        }
        const q4k_rowk ka = q4k_prepare(hA, t), kb = q4k_prepare(hB, t);
        const uint32_t wa[8] = {qA0.x, qA0.y, qA0.z, qA0.w, qA1.x, qA1.y, qA1.z, qA1.w};
        const uint32_t wb[8] = {qB0.x, qB0.y, qB0.z, qB0.w, qB1.x, qB1.y, qB1.z, qB1.w};
        const uint8_t *xf = xfrag + (size_t)sb * Q4K_XF_SB_BYTES + t * 17 * 16;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t k1024 = 0x64006400u;
#pragma unroll
        for (int cw = 0; cw < 8; cw++) {
            const uint32_t a = wa[cw], b = wb[cw];
            const uint32_t a8 = a >> 8, b8 = b >> 8;
            uint4 fl = make_uint4(0, 0, 0, 0), fh = make_uint4(0, 0, 0, 0);
            if (bcol) {
                fl = *reinterpret_cast<const uint4 *>(xf + cw * 16);
                fh = *reinterpret_cast<const uint4 *>(xf + (8 + cw) * 16);
            }
            // low nibbles: sub-block 2t
            uint32_t r0 = hfma2u((a & 0x000F000Fu) | k1024, ka.me, ka.ae);
            uint32_t r2 = hfma2u((a8 & 0x000F000Fu) | k1024, ka.me, ka.ae);
            uint32_t r1 = hfma2u((b & 0x000F000Fu) | k1024, kb.me, kb.ae);
            uint32_t r3 = hfma2u((b8 & 0x000F000Fu) | k1024, kb.me, kb.ae);
            mma16816(c, r0, r1, r2, r3, fl.x, fl.y);
            mma16816(c, r0, r1, r2, r3, fl.z, fl.w);
            // high nibbles: sub-block 2t+1 (pattern is 1024 + 16 q)
            r0 = hfma2u((a & 0x00F000F0u) | k1024, ka.mo, ka.ao);
            r2 = hfma2u((a8 & 0x00F000F0u) | k1024, ka.mo, ka.ao);
            r1 = hfma2u((b & 0x00F000F0u) | k1024, kb.mo, kb.ao);
            r3 = hfma2u((b8 & 0x00F000F0u) | k1024, kb.mo, kb.ao);
            mma16816(c, r0, r1, r2, r3, fh.x, fh.y);
            mma16816(c, r0, r1, r2, r3, fh.z, fh.w);
        }
        // minimums: sum_g m_g * S_g through one more MMA pair (k slots 2t, 2t+1).
        float c2[4] = {0.f, 0.f, 0.f, 0.f};
        uint2 sx = make_uint2(0, 0);
        if (bcol) sx = *reinterpret_cast<const uint2 *>(sxfrag + (size_t)sb * Q4K_SX_SB_BYTES + t * 8);
        mma16816(c2, ka.hm, kb.hm, 0u, 0u, sx.x, 0u);
        mma16816(c2, ka.hm, kb.hm, 0u, 0u, sx.y, 0u);
        acc[0] += ka.d * c[0] - ka.dmin * 64.f * c2[0];
        acc[1] += ka.d * c[1] - ka.dmin * 64.f * c2[1];
        acc[2] += kb.d * c[2] - kb.dmin * 64.f * c2[2];
        acc[3] += kb.d * c[3] - kb.dmin * 64.f * c2[3];
        sb = nsbi;
        if (sb < nsb) { hA = nhA; qA0 = nqA0; qA1 = nqA1; hB = nhB; qB0 = nqB0; qB1 = nqB1; }
    }

    // 4. Column 0 lives in lanes t == 0: c[0] = row g, c[2] = row g + 8.
    if (t == 0) {
        red[warp * 16 + g] = acc[0];
        red[warp * 16 + g + 8] = acc[2];
    }
    __syncthreads();
    if (tid < 16) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) s += red[w * 16 + tid];
        int row = rg * 16 + tid;
        if (row < nrows) Y[(size_t)tok * nrows + row] = s * inv_scale;
    }
}

static size_t q4k_mma_smem(int nsb, int warps) {
    return (size_t)nsb * (Q4K_XF_SB_BYTES + Q4K_SX_SB_BYTES) + (size_t)warps * 16 * 4 + (size_t)warps * 4;
}

// ------------------------------------------------------------------ dispatch

// Which decode kernel serves a shape. The reference decides per (quant, rows, k,
// ntok) (jit/gpu/tier/layer.go:10953-11016); here the tensor-core kernel takes
// every Q4_K shape whose activation fragments fit shared memory, the SIMT
// kernel takes the rest.
int jl_gemv_choice(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out) {
    jl_choice c = {};
    int pin = ctx ? ctx->opts.pin_kernel : JL_K_AUTO;
    int warps = ctx && ctx->opts.pin_warps > 0 ? ctx->opts.pin_warps : 8;
    if (warps != 4 && warps != 8 && warps != 16) warps = 8;
    bool mma_ok = type == JL_TYPE_Q4_K && k % 256 == 0 && q4k_mma_smem(k / 256, warps) <= 200 * 1024;
    if (pin == JL_K_SIMT || !mma_ok) {
        if (pin == JL_K_MMA || pin == JL_K_TC5) return JL_DECLINED;
        c.kernel = JL_K_SIMT; c.warps = 8; c.rows_per_cta = 8; c.split_k = 1;
        c.grid = (nrows + 7) / 8 * ntok;
    } else {
        c.kernel = JL_K_MMA; c.warps = warps; c.rows_per_cta = 16;
        c.split_k = warps < k / 256 ? warps : k / 256;
        c.tile_m = 16; c.tile_n = 8; c.tile_k = 16;
        c.grid = (nrows + 15) / 16 * ntok;
    }
    *out = c;
    return JL_OK;
}

int jl_launch_gemv(jl_ctx *ctx, float *out_dev, const jl_weight *w, int expert, const float *x_dev,
                   int ntok, int kernel, int warps, cudaStream_t s) {
    const int nrows = w->nrows, k = w->k;
    size_t rows_off = (size_t)expert * nrows;
    const uint8_t *data = w->data;
    const uint8_t *scales = w->scales;
    if (w->type == JL_TYPE_Q4_K) data += rows_off * jl_row_bytes(w->type, k);
    else if (w->type == JL_TYPE_Q8_0) { data += rows_off * (size_t)k; scales += rows_off * (size_t)w->scale_stride * 2; }
    else { data += rows_off * (size_t)(k / 32) * 16; scales += rows_off * (size_t)w->scale_stride; }

    if (kernel == JL_K_MMA && w->type == JL_TYPE_Q4_K) {
        int nsb = k / 256;
        size_t smem = q4k_mma_smem(nsb, warps);
        dim3 grid((nrows + 15) / 16, ntok);
#define LAUNCH_Q4K(WP)                                                                                  \
    do {                                                                                                \
        if (smem > 48 * 1024)                                                                           \
            JL_CUDA(ctx, cudaFuncSetAttribute(gemv_q4k_mma_kernel<WP>,                                  \
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        gemv_q4k_mma_kernel<WP><<<grid, WP * 32, smem, s>>>(data, x_dev, out_dev, nrows, nsb, ntok);    \
    } while (0)
        if (warps == 4) LAUNCH_Q4K(4);
        else if (warps == 16) LAUNCH_Q4K(16);
        else LAUNCH_Q4K(8);
#undef LAUNCH_Q4K
    } else {
        dim3 grid((nrows + 7) / 8, ntok);
        if (w->type == JL_TYPE_Q4_K)
            gemv_simt_kernel<JL_TYPE_Q4_K><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
        else if (w->type == JL_TYPE_Q8_0)
            gemv_simt_kernel<JL_TYPE_Q8_0><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
        else
            gemv_simt_kernel<JL_TYPE_MXFP4><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
    }
    ctx->st.launches++;
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}
