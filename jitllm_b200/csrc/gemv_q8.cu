// Q8_0 decode (1..8 tokens) and small batches (9..32 tokens) on the int8 tensor-core path.
//
// Q8_0 weights ARE int8, so they feed mma.sync.m16n8k32.s32.s8.s8 unconverted: one MMA covers 16 rows
// x one 32-element block, whose f16 scale d is applied to the integer sum afterwards. Activations are
// prepared once per matvec as two int8 digits per value (x * s ~ 256 q1 + q2 with s = 32512 / amax of the
// value's 32-element block, error <= 1.5e-5 of that amax, 3.1e-5 when the second digit saturates); the 8 MMA columns are (token j, digit) pairs, so one
// instruction serves up to four tokens and a lane ends up holding exactly the two digit sums of "its"
// token: y[row][tok] += d[row][blk] * (1/s)[tok][blk] * (256 * C1 + C2).
//
// The resident code plane is stored in 64-element spans whose 16-byte piece t holds what lane t of a quad
// feeds to the two MMAs of the span (formats.cu: q8_span_pos), so a lane's A fragments for two blocks are
// ONE 16-byte load per row. A warp's unit of work is 16 rows x 256 elements (4 KB of codes): all of its
// loads are issued before the first is used; warps of a CTA take different 256-element groups of the same
// 16 rows and meet in shared memory in fixed order (bit-stable).
#include "jl_internal.cuh"

#include <stdlib.h>

// Prepared activation operand of one token: k/64 spans x [digit 2][t 4] x 16 B, then k/32 f32 (1/s of each block).
static inline size_t q8_xp_token_bytes(int k) { return (size_t)k * 2 + (size_t)(k / 32) * 4; }
size_t jl_gemv_q8_scratch_bytes(int k, int ntok) { return ((q8_xp_token_bytes(k) + 255) & ~(size_t)255) * ntok; }

// One warp per (256-element group, token).
__global__ void __launch_bounds__(128) q8_xprep_kernel(const float *__restrict__ X, uint8_t *__restrict__ scratch, int k,
                                                       size_t tok_stride) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31, grp = blockIdx.x * 4 + (threadIdx.x >> 5), tok = blockIdx.y;
    if (grp >= k / 256) return;
    // lane = (span s of the group, quad lane t, block hb of the span): k offsets 4t..4t+3 and 16+4t..16+4t+3
    const int s = lane >> 3, t = (lane >> 1) & 3, hb = lane & 1;
    const float *x = X + (size_t)tok * k + (size_t)grp * 256 + s * 64 + hb * 32;
    const float4 v0 = __ldg(reinterpret_cast<const float4 *>(x + 4 * t));
    const float4 v1 = __ldg(reinterpret_cast<const float4 *>(x + 16 + 4 * t));
    float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                       fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    // the scale is per 32-element BLOCK (the four lanes that differ in t): the weights' own block structure costs
    // nothing extra in the kernel, and an outlier only coarsens its own block
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const bool live = amax > 0.f && amax < __int_as_float(0x7f800000);
    const float scale = live ? 32512.f / amax : 0.f;
    const float xs[8] = {v0.x * scale, v0.y * scale, v0.z * scale, v0.w * scale,
                         v1.x * scale, v1.y * scale, v1.z * scale, v1.w * scale};
    uint32_t d1[2] = {0, 0}, d2[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float q1f = rintf(xs[j] * (1.f / 256.f));
        const int q1 = (int)q1f;
        int q2 = (int)rintf(xs[j] - 256.f * q1f);
        q2 = max(-127, min(127, q2));
        d1[j >> 2] |= (uint32_t)(q1 & 0xFF) << (8 * (j & 3));
        d2[j >> 2] |= (uint32_t)(q2 & 0xFF) << (8 * (j & 3));
    }
    uint8_t *base = scratch + (size_t)tok * tok_stride;
    uint8_t *span = base + ((size_t)grp * 4 + s) * 128;
    *reinterpret_cast<uint2 *>(span + t * 16 + hb * 8) = make_uint2(d1[0], d1[1]);        // digit 1
    *reinterpret_cast<uint2 *>(span + 64 + t * 16 + hb * 8) = make_uint2(d2[0], d2[1]);   // digit 2
    if (t == 0) reinterpret_cast<float *>(base + (size_t)k * 2)[(grp * 4 + s) * 2 + hb] = live ? amax / 32512.f : 0.f;
}

__device__ __forceinline__ void q8_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

__device__ __forceinline__ uint4 q8_ldg16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// grid (row groups of 16, sets of NTG token groups of 4); WARPS warps split the 256-element groups of the row.
// NTG > 1 (batches of 5..32 tokens): the A fragments of a unit stay in registers while the CTA walks its token
// groups, so the weights are read once per 4 * NTG tokens.
template <int WARPS, int NTG>
__global__ void __launch_bounds__(WARPS * 32) gemv_q8_mma_kernel(const uint8_t *__restrict__ codes, const uint16_t *__restrict__ dplane,
                                                                 int d_stride, const uint8_t *__restrict__ xop, size_t tok_stride,
                                                                 float *__restrict__ Y, int nrows, int k, int ntok) {
    __shared__ float red[WARPS][NTG][16][4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row_a = min((int)blockIdx.x * 16 + g, nrows - 1), row_b = min((int)blockIdx.x * 16 + g + 8, nrows - 1);
    const int tok0 = blockIdx.y * 4 * NTG;
    const int ngrp = k / 256;
    const uint8_t *ca = codes + (size_t)row_a * k + t * 16, *cb = codes + (size_t)row_b * k + t * 16;
    const uint8_t *da = reinterpret_cast<const uint8_t *>(dplane + (size_t)row_a * d_stride);
    const uint8_t *db = reinterpret_cast<const uint8_t *>(dplane + (size_t)row_b * d_stride);
    // this lane's B column in token group tg: token tok0 + 4 tg + (g >> 1), digit g & 1; its accumulators: token
    // tok0 + 4 tg + t
    const size_t lane_xofs = (size_t)(g & 1) * 64 + t * 16;
    // weights first: they do not depend on the kernel in front
    uint4 wa[4], wb[4], dda, ddb;
    int grp = warp;
    if (grp < ngrp) {
#pragma unroll
        for (int s = 0; s < 4; s++) {
            wa[s] = q8_ldg16(ca + (size_t)grp * 256 + s * 64);
            wb[s] = q8_ldg16(cb + (size_t)grp * 256 + s * 64);
        }
        dda = q8_ldg16(da + (size_t)grp * 16);
        ddb = q8_ldg16(db + (size_t)grp * 16);
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the prepared activations come from the kernel in front

    float acc_a[NTG], acc_b[NTG];
#pragma unroll
    for (int tg = 0; tg < NTG; tg++) acc_a[tg] = acc_b[tg] = 0.f;
    for (; grp < ngrp; grp += WARPS) {
        const uint4 ua[4] = {wa[0], wa[1], wa[2], wa[3]}, ub[4] = {wb[0], wb[1], wb[2], wb[3]};
        const uint32_t dwa[4] = {dda.x, dda.y, dda.z, dda.w}, dwb[4] = {ddb.x, ddb.y, ddb.z, ddb.w};
        const int nx = grp + WARPS;
        if (nx < ngrp) {                                   // the next unit's loads fly while this one is multiplied
#pragma unroll
            for (int s = 0; s < 4; s++) {
                wa[s] = q8_ldg16(ca + (size_t)nx * 256 + s * 64);
                wb[s] = q8_ldg16(cb + (size_t)nx * 256 + s * 64);
            }
            dda = q8_ldg16(da + (size_t)nx * 16);
            ddb = q8_ldg16(db + (size_t)nx * 16);
        }
        float2 fa[4], fb[4];
#pragma unroll
        for (int s = 0; s < 4; s++) {
            fa[s] = __half22float2(*reinterpret_cast<const __half2 *>(&dwa[s]));
            fb[s] = __half22float2(*reinterpret_cast<const __half2 *>(&dwb[s]));
        }
#pragma unroll
        for (int tg = 0; tg < NTG; tg++) {
            const int btok = tok0 + 4 * tg + (g >> 1), mytok = tok0 + 4 * tg + t;
            const bool blive = btok < ntok;
            const uint8_t *xb = xop + (size_t)(blive ? btok : 0) * tok_stride + lane_xofs;
            uint4 xv[4];
#pragma unroll
            for (int s = 0; s < 4; s++)
                xv[s] = blive ? *reinterpret_cast<const uint4 *>(xb + ((size_t)grp * 4 + s) * 128) : make_uint4(0, 0, 0, 0);
            float4 isA = make_float4(0.f, 0.f, 0.f, 0.f), isB = isA;           // 1/s of the group's eight blocks
            if (mytok < ntok) {
                const float4 *ip = reinterpret_cast<const float4 *>(xop + (size_t)mytok * tok_stride + (size_t)k * 2) + grp * 2;
                isA = ip[0]; isB = ip[1];
            }
            const float isb[8] = {isA.x, isA.y, isA.z, isA.w, isB.x, isB.y, isB.z, isB.w};
            float ga = 0.f, gb = 0.f;
#pragma unroll
            for (int s = 0; s < 4; s++) {
                int c0[4], c1[4];
                q8_mma(c0, ua[s].x, ub[s].x, ua[s].y, ub[s].y, xv[s].x, xv[s].y);     // block 2s
                q8_mma(c1, ua[s].z, ub[s].z, ua[s].w, ub[s].w, xv[s].z, xv[s].w);     // block 2s + 1
                ga = fmaf(fa[s].x * isb[2 * s], (float)(256 * c0[0] + c0[1]), ga);
                gb = fmaf(fb[s].x * isb[2 * s], (float)(256 * c0[2] + c0[3]), gb);
                ga = fmaf(fa[s].y * isb[2 * s + 1], (float)(256 * c1[0] + c1[1]), ga);
                gb = fmaf(fb[s].y * isb[2 * s + 1], (float)(256 * c1[2] + c1[3]), gb);
            }
            acc_a[tg] += ga;
            acc_b[tg] += gb;
        }
    }
#pragma unroll
    for (int tg = 0; tg < NTG; tg++) {
        red[warp][tg][g][t] = acc_a[tg];
        red[warp][tg][g + 8][t] = acc_b[tg];
    }
    __syncthreads();
    for (int i = tid; i < 64 * NTG; i += WARPS * 32) {
        const int tg = i >> 6, r = (i >> 2) & 15, j = i & 3;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) sum += red[w][tg][r][j];      // fixed order
        const int row = blockIdx.x * 16 + r, tok = tok0 + 4 * tg + j;
        if (row < nrows && tok < ntok) Y[(size_t)tok * nrows + row] = sum;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Batches of 9..32 tokens: one pass over the weights for all tokens.
//
// A CTA of WARPS warps covers 16 * WARPS rows (a row group of 16 per warp) and a slice of the row's 256-element
// groups; all of its warps work on the same group at a time, so the group's prepared activations of all tokens
// (32 x 544 bytes) are staged ONCE per CTA in shared memory (cp.async, two stages) and every warp takes its MMA B
// fragments from there. The weights go straight from global memory into registers, one group ahead, and are used
// by up to eight token groups of four. The k-slices of a row tile are the CTAs of one thread-block cluster: each
// leaves its partial tile in its own shared memory, and after a cluster barrier CTA r sums slice r of the tile
// over the ranks in rank order through distributed shared memory (bit-stable; no partial planes in global memory,
// no second launch, no flag that one CTA would spin on).
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define Q8B_TOK 32
#define Q8B_TOK_BYTES 544          // 4 spans x 128 B of digits + 8 x f32 (1/s of the group's blocks)

__device__ __forceinline__ void q8b_cp16(void *smem, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(g) : "memory");
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemv_q8_batch_kernel(const uint8_t *__restrict__ codes, const uint16_t *__restrict__ dplane, int d_stride,
                     const uint8_t *__restrict__ xop, size_t tok_stride, float *__restrict__ Y, int nrows, int k, int ntok,
                     int groups_per_cta) {
    constexpr int ROWS = WARPS * 16, RED_STRIDE = ROWS + 4;
    constexpr int STAGE = Q8B_TOK * Q8B_TOK_BYTES;
    static_assert(Q8B_TOK * RED_STRIDE * 4 <= 2 * STAGE, "the partial tile reuses the activation stages");
    __shared__ __align__(16) uint8_t smem[2 * STAGE];
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * ROWS + warp * 16;
    const int row_a = min(row0 + g, nrows - 1), row_b = min(row0 + g + 8, nrows - 1);
    const int grp0 = blockIdx.y * groups_per_cta;
    const int ntg = (ntok + 3) >> 2;
    const uint8_t *ca = codes + (size_t)row_a * k + t * 16, *cb = codes + (size_t)row_b * k + t * 16;
    const uint8_t *da = reinterpret_cast<const uint8_t *>(dplane + (size_t)row_a * d_stride);
    const uint8_t *db = reinterpret_cast<const uint8_t *>(dplane + (size_t)row_b * d_stride);

    // weights of the first group: they do not depend on the kernel in front
    uint4 wa[4], wb[4], dda, ddb;
#pragma unroll
    for (int s = 0; s < 4; s++) {
        wa[s] = q8_ldg16(ca + (size_t)grp0 * 256 + s * 64);
        wb[s] = q8_ldg16(cb + (size_t)grp0 * 256 + s * 64);
    }
    dda = q8_ldg16(da + (size_t)grp0 * 16);
    ddb = q8_ldg16(db + (size_t)grp0 * 16);
    // tokens beyond ntok multiply zeros
    for (int i = tid; i < 2 * STAGE / 16; i += WARPS * 32) reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the prepared activations come from the kernel in front

    auto stage_in = [&](int st, int grp) {
        uint8_t *dst = smem + st * STAGE;
        for (int i = tid; i < ntok * 34; i += WARPS * 32) {
            const int tok = (int)(((unsigned)i * 1928u) >> 16), c = i - tok * 34;   // i / 34 for i < 32 * 34
            const uint8_t *src = xop + (size_t)tok * tok_stride + (c < 32 ? (size_t)grp * 512 + c * 16 : (size_t)k * 2 + (size_t)grp * 32 + (c - 32) * 16);
            q8b_cp16(dst + tok * Q8B_TOK_BYTES + c * 16, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage_in(0, grp0);

    float acc_a[8], acc_b[8];
#pragma unroll
    for (int tg = 0; tg < 8; tg++) acc_a[tg] = acc_b[tg] = 0.f;
    const int lane_xofs = (g >> 1) * Q8B_TOK_BYTES + (g & 1) * 64 + t * 16;   // B column: token 4 tg + (g >> 1), digit g & 1
    const int lane_iofs = t * Q8B_TOK_BYTES + 512;                            // accumulators: token 4 tg + t

    for (int i = 0; i < groups_per_cta; i++) {
        const int grp = grp0 + i;
        const uint4 ua[4] = {wa[0], wa[1], wa[2], wa[3]}, ub[4] = {wb[0], wb[1], wb[2], wb[3]};
        const uint32_t dwa[4] = {dda.x, dda.y, dda.z, dda.w}, dwb[4] = {ddb.x, ddb.y, ddb.z, ddb.w};
        if (i + 1 < groups_per_cta) {
#pragma unroll
            for (int s = 0; s < 4; s++) {
                wa[s] = q8_ldg16(ca + (size_t)(grp + 1) * 256 + s * 64);
                wb[s] = q8_ldg16(cb + (size_t)(grp + 1) * 256 + s * 64);
            }
            dda = q8_ldg16(da + (size_t)(grp + 1) * 16);
            ddb = q8_ldg16(db + (size_t)(grp + 1) * 16);
            stage_in((i + 1) & 1, grp + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint8_t *xs = smem + (i & 1) * STAGE;
        float2 fa[4], fb[4];
#pragma unroll
        for (int s = 0; s < 4; s++) {
            fa[s] = __half22float2(*reinterpret_cast<const __half2 *>(&dwa[s]));
            fb[s] = __half22float2(*reinterpret_cast<const __half2 *>(&dwb[s]));
        }
#pragma unroll
        for (int tg = 0; tg < 8; tg++) {
            if (tg < ntg) {
                const uint8_t *xb = xs + tg * 4 * Q8B_TOK_BYTES;
                uint4 xv[4];
#pragma unroll
                for (int s = 0; s < 4; s++) xv[s] = *reinterpret_cast<const uint4 *>(xb + lane_xofs + s * 128);
                const float4 isA = *reinterpret_cast<const float4 *>(xb + lane_iofs);
                const float4 isB = *reinterpret_cast<const float4 *>(xb + lane_iofs + 16);
                const float isb[8] = {isA.x, isA.y, isA.z, isA.w, isB.x, isB.y, isB.z, isB.w};
                float ga = 0.f, gb = 0.f;
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    int c0[4], c1[4];
                    q8_mma(c0, ua[s].x, ub[s].x, ua[s].y, ub[s].y, xv[s].x, xv[s].y);     // block 2s
                    q8_mma(c1, ua[s].z, ub[s].z, ua[s].w, ub[s].w, xv[s].z, xv[s].w);     // block 2s + 1
                    ga = fmaf(fa[s].x * isb[2 * s], (float)(256 * c0[0] + c0[1]), ga);
                    gb = fmaf(fb[s].x * isb[2 * s], (float)(256 * c0[2] + c0[3]), gb);
                    ga = fmaf(fa[s].y * isb[2 * s + 1], (float)(256 * c1[0] + c1[1]), ga);
                    gb = fmaf(fb[s].y * isb[2 * s + 1], (float)(256 * c1[2] + c1[3]), gb);
                }
                acc_a[tg] += ga;
                acc_b[tg] += gb;
            }
        }
        __syncthreads();   // the stage is refilled two iterations on
    }

    // partial tile [token][row] into this CTA's shared memory, then the cluster's ranks sum it slice by slice
    float *red = reinterpret_cast<float *>(smem);
#pragma unroll
    for (int tg = 0; tg < 8; tg++) {
        red[(4 * tg + t) * RED_STRIDE + warp * 16 + g] = acc_a[tg];
        red[(4 * tg + t) * RED_STRIDE + warp * 16 + g + 8] = acc_b[tg];
    }
    cluster.sync();
    const int ks = gridDim.y, rank = blockIdx.y;      // the cluster spans the whole y dimension
    // four consecutive rows of one token per thread; the ranks' values are fetched together (independent loads over
    // distributed shared memory: one after the other they cost a round trip each), then added in rank order
    const float4 *peer[8];
#pragma unroll
    for (int q = 0; q < 8; q++) peer[q] = reinterpret_cast<const float4 *>(cluster.map_shared_rank(red, q < ks ? q : 0));
    const int nvec = ntok * (ROWS / 4), per = (nvec + ks - 1) / ks;
    const int e1 = min(nvec, (rank + 1) * per);
    for (int e = rank * per + tid; e < e1; e += WARPS * 32) {
        const int tok = e / (ROWS / 4), r4 = e - tok * (ROWS / 4);
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; q++)
            if (q < ks) v[q] = peer[q][(tok * RED_STRIDE) / 4 + r4];
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 8; q++)
            if (q < ks) { sum.x += v[q].x; sum.y += v[q].y; sum.z += v[q].z; sum.w += v[q].w; }
        const int row = blockIdx.x * ROWS + 4 * r4;
        float *y = Y + (size_t)tok * nrows + row;
        if (row + 3 < nrows && (nrows & 3) == 0) {
            *reinterpret_cast<float4 *>(y) = sum;
        } else {
            if (row < nrows) y[0] = sum.x;
            if (row + 1 < nrows) y[1] = sum.y;
            if (row + 2 < nrows) y[2] = sum.z;
            if (row + 3 < nrows) y[3] = sum.w;
        }
    }
    cluster.sync();    // nobody leaves while a peer still reads its tile
}

// Row tile (warps) and k-slices of the batch kernel for a shape: the fewest slices that give every SM a CTA.
void jl_gemv_q8_batch_plan(int nrows, int k, int *warps, int *slices) {
    const int ngrp = k / 256;
    const int w = nrows >= 2048 ? 8 : 4;
    const int tiles = (nrows + 16 * w - 1) / (16 * w);
    int ks = 1;
    while (ks < 8 && tiles * ks < 148 && ngrp % (ks * 2) == 0) ks *= 2;
#ifdef JL_EXPERIMENT_ENV
    if (const char *e = getenv("Q8B_KS")) { const int v = atoi(e); if (v >= 1 && v <= 8 && ngrp % v == 0) ks = v; }
#endif
    *warps = w;
    *slices = ks;
}

static int launch_q8_batch(jl_ctx *ctx, float *out_dev, const uint8_t *codes, const uint16_t *dpl, int d_stride,
                           const uint8_t *xop, size_t tok_stride, int nrows, int k, int ntok, cudaStream_t s) {
    int warps, ks;
    jl_gemv_q8_batch_plan(nrows, k, &warps, &ks);
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = ks; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((nrows + 16 * warps - 1) / (16 * warps), ks); cfg.blockDim = dim3(warps * 32); cfg.stream = s;
    cfg.attrs = at; cfg.numAttrs = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 1 : 2;
    const int gpc = k / 256 / ks;
    if (warps == 8)
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_q8_batch_kernel<8>, codes, dpl, d_stride, xop, tok_stride, out_dev, nrows, k, ntok, gpc));
    else
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_q8_batch_kernel<4>, codes, dpl, d_stride, xop, tok_stride, out_dev, nrows, k, ntok, gpc));
    ctx->st.launches++;
    return JL_OK;
}

int jl_launch_gemv_q8(jl_ctx *ctx, float *out_dev, const uint8_t *codes, const uint8_t *scales, int d_stride,
                      const float *x_dev, int nrows, int k, int ntok, cudaStream_t s) {
    const size_t tok_stride = (q8_xp_token_bytes(k) + 255) & ~(size_t)255;
    const size_t need = tok_stride * ntok;
    if (ctx->scratch_cap < need)
        return jl_set_err(ctx, JL_ENOMEM, "decode scratch holds %zu bytes, %d x %d token(s) need %zu (jl_reserve sizes it)",
                          ctx->scratch_cap, k, ntok, need);
    uint8_t *scratch = (uint8_t *)ctx->scratch;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    const int nattr = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((k / 256 + 3) / 4, ntok); cfg.blockDim = dim3(128); cfg.stream = s; cfg.attrs = at; cfg.numAttrs = nattr;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, q8_xprep_kernel, x_dev, scratch, k, tok_stride));
    ctx->st.launches++;
    if (ntok > 8 && ntok <= Q8B_TOK)
        return launch_q8_batch(ctx, out_dev, codes, reinterpret_cast<const uint16_t *>(scales), d_stride, scratch, tok_stride, nrows, k, ntok, s);
    const int ngrp = k / 256;
    const int warps = ngrp >= 8 ? 8 : (ngrp >= 4 ? 4 : (ngrp >= 2 ? 2 : 1));
    const int tgroups = (ntok + 3) / 4;
    const int ntg = tgroups >= 4 ? 4 : (tgroups >= 2 ? 2 : 1);
    cfg.gridDim = dim3((nrows + 15) / 16, (tgroups + ntg - 1) / ntg); cfg.blockDim = dim3(warps * 32);
    const uint16_t *dpl = reinterpret_cast<const uint16_t *>(scales);
    const uint8_t *xop = scratch;
#define Q8_LAUNCH(WP, TG) JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_q8_mma_kernel<WP, TG>, codes, dpl, d_stride, xop, tok_stride, out_dev, nrows, k, ntok))
#define Q8_LAUNCH_W(WP) do { if (ntg == 4) Q8_LAUNCH(WP, 4); else if (ntg == 2) Q8_LAUNCH(WP, 2); else Q8_LAUNCH(WP, 1); } while (0)
    if (warps == 8) Q8_LAUNCH_W(8);
    else if (warps == 4) Q8_LAUNCH_W(4);
    else if (warps == 2) Q8_LAUNCH_W(2);
    else Q8_LAUNCH_W(1);
#undef Q8_LAUNCH_W
#undef Q8_LAUNCH
    ctx->st.launches++;
    return JL_OK;
}
