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
//                - a warp-task is 16 rows x one 256-element super-block, fetched by
//                  ONE TMA copy (box 144 B x 16 rows) into a per-warp ring;
//                - the 4-bit codes become unsigned bytes with three ALU ops per
//                  eight weights; activations are prepared once per matvec as two
//                  int8 digits per value (x*s ~ 256 q1 + q2) in MMA fragment order;
//                - mma.sync.m16n8k32.s32.u8.s8 against a block-diagonal B operand
//                  collects four per-sub-block integer sums at once; sc and m fold
//                  in as integers, d, dmin and 1/s in f32;
//                - warps of a CTA cover different super-blocks of the same rows
//                  and meet through shared memory in fixed order, so the result
//                  is run-to-run bit-stable.
#include "jl_internal.cuh"
#include "tma.cuh"
#include "raw_formats.cuh"

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
        } else if (jl_type_raw_simt(TYPE)) {
            // raw ggml blocks; each weight exactly as quant.Dequant32 forms it
            constexpr int BE = TYPE == JL_TYPE_Q5_K || TYPE == JL_TYPE_Q6_K ? 256 : 32;
            constexpr int BB = TYPE == JL_TYPE_Q4_0 ? 18 : TYPE == JL_TYPE_Q5_0 ? 22 : TYPE == JL_TYPE_Q5_1 ? 24 : TYPE == JL_TYPE_Q5_K ? 176 : 210;
            const uint8_t *blk = data + ((size_t)row * (k / BE) + (size_t)(si * 32 / BE)) * BB;
            const int e0 = (si * 32) % BE;
            for (int l = 0; l < 32; l++) acc = fmaf(jl_raw_weight(TYPE, blk, e0 + l), xs[l], acc);
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

// Q6_K decode without a byte loop: one warp per row, two super-blocks per pass. A super-block is two halves of 128
// elements; in a half, byte l of ql / ql + 32 / qh carries elements l, l + 32, l + 64, l + 96 (low nibbles, low
// nibbles of the second run, high nibbles, high nibbles; two bits of qh each). Eight lanes take a half, lane i of them
// the four positions l = 4i .. 4i + 3: three 32-bit words (read as 16-bit halves: a 210-byte block is only 2-byte
// aligned) give it 16 codes, which become floats by byte placement (0x4B0000qq reads as 2^23 + q), and its four
// float4 of the activation row. Each weight is formed as quant.Dequant32 forms it: (d * sc) rounded, times (q - 32)
// rounded (format/quant/dequant.go:443-470). NT tokens share the decoded weights.
__device__ __forceinline__ uint32_t q6k_ld32(const uint8_t *p) {
    const uint16_t *h = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)__ldg(h) | ((uint32_t)__ldg(h + 1) << 16);
}
template <int NT>
__global__ void __launch_bounds__(256) gemv_q6k_kernel(const uint8_t *__restrict__ data, const float *__restrict__ X,
                                                       float *__restrict__ Y, int nrows, int k, int ntok) {
    const int row = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    const int tok0 = blockIdx.y * NT;
    if (row >= nrows) return;
    const int nsb = k / 256;
    const int hl = lane >> 3, i = lane & 7;            // half hl of the pass's two super-blocks, positions 4i..4i+3
    const int n = hl & 1;
    const uint8_t *rowp = data + (size_t)row * nsb * 210;
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = 0.f;
    for (int sb = hl >> 1; sb < nsb; sb += 2) {
        const uint8_t *blk = rowp + (size_t)sb * 210;
        const uint32_t A = q6k_ld32(blk + n * 64 + 4 * i), B = q6k_ld32(blk + n * 64 + 32 + 4 * i);
        const uint32_t H = q6k_ld32(blk + 128 + n * 32 + 4 * i);
        const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t *>(blk + 208))));
        const int8_t *scp = reinterpret_cast<const int8_t *>(blk + 192 + n * 8 + (i >> 2));
        // the four 32-runs of the half: codes of positions 4i..4i+3, one byte each
        const uint32_t c4[4] = {(A & 0x0F0F0F0Fu) | ((H & 0x03030303u) << 4), (B & 0x0F0F0F0Fu) | ((H & 0x0C0C0C0Cu) << 2),
                                ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u), ((B >> 4) & 0x0F0F0F0Fu) | ((H & 0xC0C0C0C0u) >> 2)};
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const float dsc = __fmul_rn(d, (float)(int)__ldg(scp + 2 * c));
            float w[4];
#pragma unroll
            for (int j = 0; j < 4; j++)   // 0x4B0000qq = 2^23 + q; minus (2^23 + 32) = q - 32, exact
                w[j] = __fmul_rn(dsc, __uint_as_float(__byte_perm(c4[c], 0x4B000000u, 0x7650 + j)) - 8388640.f);
            const size_t e0 = (size_t)sb * 256 + n * 128 + c * 32 + 4 * i;
#pragma unroll
            for (int t = 0; t < NT; t++) {
                if (tok0 + t < ntok) {
                    const float4 x = __ldg(reinterpret_cast<const float4 *>(X + (size_t)(tok0 + t) * k + e0));
                    acc[t] = fmaf(w[0], x.x, acc[t]); acc[t] = fmaf(w[1], x.y, acc[t]);
                    acc[t] = fmaf(w[2], x.z, acc[t]); acc[t] = fmaf(w[3], x.w, acc[t]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; t++) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && tok0 + t < ntok) Y[(size_t)(tok0 + t) * nrows + row] = v;
    }
}

// Q5_K the same way: lane l takes position l of each of the super-block's eight sub-blocks (five coalesced byte loads
// per super-block: qh[l] and the four code bytes that carry position l), every weight formed as quant.Dequant32 forms
// it, (d sc) q - (dmin m) with each product and the difference rounded (format/quant/dequant.go:399-441).
template <int NT>
__global__ void __launch_bounds__(256) gemv_q5k_kernel(const uint8_t *__restrict__ data, const float *__restrict__ X,
                                                       float *__restrict__ Y, int nrows, int k, int ntok) {
    const int row = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    const int tok0 = blockIdx.y * NT;
    if (row >= nrows) return;
    const int nsb = k / 256;
    const uint8_t *rowp = data + (size_t)row * nsb * 176;
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = 0.f;
    for (int sb = 0; sb < nsb; sb++) {
        const uint8_t *blk = rowp + (size_t)sb * 176;
        const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t *>(blk))));
        const float dmin = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t *>(blk + 2))));
        const uint32_t qh = __ldg(blk + 16 + lane);
        uint32_t qs[4];
#pragma unroll
        for (int g = 0; g < 4; g++) qs[g] = __ldg(blk + 48 + g * 32 + lane);
#pragma unroll
        for (int sub = 0; sub < 8; sub++) {
            uint8_t sc, m;
            jl_raw_scale_min_k4(sub, blk + 4, &sc, &m);
            const float dsc = __fmul_rn(d, (float)sc), dm = __fmul_rn(dmin, (float)m);
            const uint32_t b = qs[sub >> 1];
            const int q = (int)((sub & 1) ? (b >> 4) : (b & 0xF)) + (int)(((qh >> sub) & 1u) << 4);
            const float w = __fsub_rn(__fmul_rn(dsc, (float)q), dm);
            const size_t e = (size_t)sb * 256 + sub * 32 + lane;
#pragma unroll
            for (int t = 0; t < NT; t++)
                if (tok0 + t < ntok) acc[t] = fmaf(w, __ldg(X + (size_t)(tok0 + t) * k + e), acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < NT; t++) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && tok0 + t < ntok) Y[(size_t)(tok0 + t) * nrows + row] = v;
    }
}

// Q4_0 / Q5_0 / Q5_1 (32-element blocks of 18 / 22 / 24 bytes, 2-byte aligned): a lane takes a whole block per pass --
// its scale(s), the 16 code bytes as 16-bit loads, Q5's 32 high bits -- and the 32 activations that go with it.
// Weights as quant.Dequant32 forms them: (q - 8) d, (q - 16) d, and q d + m as one fused multiply-add
// (format/quant/dequant.go:85-146).
template <uint32_t TYPE, int NT>
__global__ void __launch_bounds__(256) gemv_q45_kernel(const uint8_t *__restrict__ data, const float *__restrict__ X,
                                                       float *__restrict__ Y, int nrows, int k, int ntok) {
    constexpr int BB = TYPE == JL_TYPE_Q4_0 ? 18 : (TYPE == JL_TYPE_Q5_0 ? 22 : 24);
    constexpr int QOFS = TYPE == JL_TYPE_Q4_0 ? 2 : (TYPE == JL_TYPE_Q5_0 ? 6 : 8);
    const int row = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
    const int tok0 = blockIdx.y * NT;
    if (row >= nrows) return;
    const int nblk = k / 32;
    const uint8_t *rowp = data + (size_t)row * nblk * BB;
    float acc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = 0.f;
    for (int b = lane; b < nblk; b += 32) {
        const uint16_t *h = reinterpret_cast<const uint16_t *>(rowp + (size_t)b * BB);
        const float d = __half2float(__ushort_as_half(__ldg(h)));
        const float m = TYPE == JL_TYPE_Q5_1 ? __half2float(__ushort_as_half(__ldg(h + 1))) : 0.f;
        uint32_t qh = 0;
        if (TYPE != JL_TYPE_Q4_0) qh = (uint32_t)__ldg(h + QOFS / 2 - 2) | ((uint32_t)__ldg(h + QOFS / 2 - 1) << 16);
        uint32_t qs[4];
#pragma unroll
        for (int i = 0; i < 4; i++) qs[i] = (uint32_t)__ldg(h + QOFS / 2 + 2 * i) | ((uint32_t)__ldg(h + QOFS / 2 + 2 * i + 1) << 16);
        float w[32];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const uint32_t byte = (qs[j >> 2] >> (8 * (j & 3))) & 0xFFu;
            int lo = (int)(byte & 0xF), hi = (int)(byte >> 4);
            if (TYPE != JL_TYPE_Q4_0) { lo |= (int)((qh >> j) & 1u) << 4; hi |= (int)((qh >> (j + 16)) & 1u) << 4; }
            if (TYPE == JL_TYPE_Q4_0) { w[j] = __fmul_rn((float)(lo - 8), d); w[j + 16] = __fmul_rn((float)(hi - 8), d); }
            else if (TYPE == JL_TYPE_Q5_0) { w[j] = __fmul_rn((float)(lo - 16), d); w[j + 16] = __fmul_rn((float)(hi - 16), d); }
            else { w[j] = fmaf((float)lo, d, m); w[j + 16] = fmaf((float)hi, d, m); }
        }
#pragma unroll
        for (int t = 0; t < NT; t++) {
            if (tok0 + t < ntok) {
                const float4 *x4 = reinterpret_cast<const float4 *>(X + (size_t)(tok0 + t) * k + (size_t)b * 32);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 x = __ldg(x4 + i);
                    acc[t] = fmaf(w[4 * i], x.x, acc[t]); acc[t] = fmaf(w[4 * i + 1], x.y, acc[t]);
                    acc[t] = fmaf(w[4 * i + 2], x.z, acc[t]); acc[t] = fmaf(w[4 * i + 3], x.w, acc[t]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; t++) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && tok0 + t < ntok) Y[(size_t)(tok0 + t) * nrows + row] = v;
    }
}

// ---------------------------------------------------------------- MMA family
//
// Q4_K decode on the tensor cores, one token.
//
// A warp-task is 16 rows x one 256-element super-block (2304 bytes of weights).
// Lane (g, t) of the warp owns rows g and g+8 and the 32 code bytes of 64-element
// group t, i.e. sub-blocks 2t (low nibbles) and 2t+1 (high nibbles).
//
//   weights      one TMA copy per task (2-D tensor map over the raw bytes, box =
//                144 B x 16 rows) into a per-warp shared-memory ring; the first STAGES
//                tasks of every warp are requested in the kernel's first instructions,
//                before it waits for its predecessor in the stream.
//   A operand    the 4-bit codes as unsigned bytes: (w & 0x0F0F0F0F) and, for the odd sub-block,
//                (w & 0xF0F0F0F0) = 16 x the code, divided out of the integer sum afterwards (exact):
//                two ALU ops per eight weights.
//   activations  made once per matvec by q4k_xprep_kernel: per super-block a scale
//                s = 32512 / amax and two int8 digits, x*s ~ 256 q1 + q2 (|err| <= 0.5,
//                i.e. 1.5e-5 of the super-block's amax), already laid out as MMA B
//                fragments, plus the integer sum of 256 q1 + q2 over each sub-block.
//   B operand    block-diagonal: column 2t carries digit 1 and column 2t+1 digit 2 of
//                group t, all other columns are zero, so the eight columns of one
//                accumulator collect four sub-block sums separately (even sub-blocks
//                in `ce`, odd in `co`) instead of seven columns idling.
//   mma.sync     m16n8k32 u8 x s8 -> s32: exact. Eight per task.
//   fold         lane (g, t) ends with the integer dot products of sub-blocks 2t and
//                2t+1 for its two rows; sc, m enter as integers (IMAD), d, dmin and
//                1/s in f32: out += (d (sc_e P_e + sc_o P_o) - dmin (m_e S_e + m_o S_o)) / s.
//   reduce       the t lanes by shuffle, the warps of a CTA (which hold different
//                super-blocks of the same 16 rows) through shared memory in fixed
//                order: run-to-run bit-stable.

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#include "q4k_prep.cuh"
static size_t q4k_xprep_bytes(int nsb, int ntok) {
    return (size_t)ntok * nsb * Q4K_XP_SB_BYTES + Q4K_XP_ZERO_BYTES;
}

// One warp per (super-block, token): the operand of a whole matvec, made once.
__global__ void __launch_bounds__(128)
q4k_xprep_kernel(const float *__restrict__ X, uint8_t *__restrict__ scratch, int nsb, int ntok) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");  // x comes from the previous kernel
    const int sb = blockIdx.x * 4 + (threadIdx.x >> 5), tok = blockIdx.y;
    if (sb >= nsb) return;
    q4k_prep_sb(reinterpret_cast<const float4 *>(X + ((size_t)tok * nsb + sb) * 256),
                scratch + ((size_t)tok * nsb + sb) * Q4K_XP_SB_BYTES, threadIdx.x & 31);
}

#define Q4K_TILE_BYTES (16 * 144)
// FUSED = the warp makes the operand of each super-block it consumes itself, in shared
// memory, from X: no prep kernel in front and no kernel boundary in the dependency chain
// (what a latency-bound shape wants), at the price of every 16-row CTA redoing the
// conversion (what a throughput-bound shape does not want). `xsrc` is X when FUSED, the
// prepared scratch otherwise.
// XG = the prepared operand is read from global memory (it stays in L1: every CTA of an SM reads the same
// few KB) instead of being staged in each CTA's shared memory, which then holds weight tiles only: more CTAs
// per SM, i.e. more weight bytes in flight.
// RG > 1 (with CPREP) = one launch per matvec without the per-16-row redundancy of FUSED: the CTA covers RG row
// groups (WARPS / RG warps each), converts the WHOLE activation row into its shared memory once, then runs the
// split form's loop on it. `xsrc` is X. For callers that overlap many matvecs the kernel-launch rate, not HBM, is
// what two launches per matvec run into.
template <int WARPS, int STAGES, int MINB, bool FUSED, bool XG = false, int RG = 1, bool CPREP = false>
__global__ void __launch_bounds__(WARPS * 32, MINB)
gemv_q4k_tma_kernel(const __grid_constant__ CUtensorMap wmap, int row0, const void *__restrict__ xsrc,
                    float *__restrict__ Y, int nrows, int nsb, int ntok, int *status) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int WPR = WARPS / RG;             // warps per row group
    const int rgi = warp / WPR, wq = warp % WPR;
    const int rg = blockIdx.x * RG + rgi, tok = blockIdx.y;
    // shared memory: [WARPS][STAGES] weight tiles | activation operand (nsb x 640 B + 128 zero)
    //                | red[WARPS][16] | barriers [WARPS][STAGES] + 1
    uint8_t *tiles = smem + (size_t)warp * STAGES * Q4K_TILE_BYTES;
    uint8_t *xop = smem + (size_t)WARPS * STAGES * Q4K_TILE_BYTES;
    const uint32_t xop_bytes = XG ? 0u : (uint32_t)(FUSED ? WARPS : nsb) * Q4K_XP_SB_BYTES;
    float *red = reinterpret_cast<float *>(xop + xop_bytes + Q4K_XP_ZERO_BYTES);
    uint64_t *bars_all = reinterpret_cast<uint64_t *>(red + WARPS * 16);
    uint64_t *bars = bars_all + warp * STAGES;
    uint64_t *xbar = bars_all + WARPS * STAGES;

    // The weight ring and its barriers are private to the warp: requested at once.
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(smem_u32(bars + s), 1);
        if (warp == 0) mbar_init(smem_u32(xbar), 1);
        mbar_init_fence();
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            const int sbi = wq + s * WPR;
            if (sbi < nsb) {
                mbar_arrive_expect_tx(smem_u32(bars + s), Q4K_TILE_BYTES);
                tma_load_2d(smem_u32(tiles + s * Q4K_TILE_BYTES), &wmap, sbi * 144, row0 + rg * 16,
                            smem_u32(bars + s));
            }
        }
    }
    if (tid < Q4K_XP_ZERO_BYTES / 4) reinterpret_cast<uint32_t *>(xop + xop_bytes)[tid] = 0u;
    __syncthreads();  // xbar initialised, zero fragment written
    // Programmatic dependent launch: the next kernel in the stream may start now; this one
    // waits for its predecessor (the activation prep) only before it copies the operand.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool lost = false;
    if (CPREP) {
        for (int sb = warp; sb < nsb; sb += WARPS)
            q4k_prep_sb(reinterpret_cast<const float4 *>(static_cast<const float *>(xsrc) + ((size_t)tok * nsb + sb) * 256),
                        xop + (size_t)sb * Q4K_XP_SB_BYTES, lane);
        __syncthreads();
    } else if (!FUSED && !XG) {
        if (tid == 0) {
            mbar_arrive_expect_tx(smem_u32(xbar), xop_bytes);
            bulk_load_1d(smem_u32(xop), static_cast<const uint8_t *>(xsrc) + (size_t)tok * xop_bytes, xop_bytes,
                         smem_u32(xbar));
        }
        lost = !__all_sync(0xffffffffu, mbar_wait(smem_u32(xbar), 0, status));
    }

    const bool bsel = ((g >> 1) == t);  // lanes that feed a non-zero B column: digit (g & 1) of group t
    const uint8_t *zero = xop + xop_bytes;
    const int sh = 8 * (2 * (t & 1));   // bit offset of this lane's scale bytes inside a header word
    float accA = 0.f, accB = 0.f;

    for (int it = 0, sb = wq; sb < nsb && !lost; it++, sb += WPR) {
        const int s = it % STAGES;
        const uint32_t parity = (uint32_t)(it / STAGES) & 1u;
        uint8_t *xsb = XG ? const_cast<uint8_t *>(static_cast<const uint8_t *>(xsrc)) + ((size_t)tok * nsb + sb) * Q4K_XP_SB_BYTES
                          : xop + (size_t)(FUSED ? warp : sb) * Q4K_XP_SB_BYTES;
        if (FUSED) {
            __syncwarp();  // the previous super-block's operand has been consumed
            q4k_prep_sb(reinterpret_cast<const float4 *>(static_cast<const float *>(xsrc) +
                                                          ((size_t)tok * nsb + sb) * 256), xsb, lane);
            __syncwarp();
        }
        const uint8_t *xf = bsel ? xsb + t * Q4K_XP_GROUP_BYTES + (g & 1) * 8 : zero;
        const int4 ax = XG ? __ldg(reinterpret_cast<const int4 *>(xsb + Q4K_XP_AUX_OFS + t * 16))
                           : *reinterpret_cast<const int4 *>(xsb + Q4K_XP_AUX_OFS + t * 16);
        uint2 xfe[4], xfo[4];
        if (XG) {
#pragma unroll
            for (int cp = 0; cp < 4; cp++) {
                xfe[cp] = bsel ? __ldg(reinterpret_cast<const uint2 *>(xf + cp * 16)) : make_uint2(0u, 0u);
                xfo[cp] = bsel ? __ldg(reinterpret_cast<const uint2 *>(xf + 64 + cp * 16)) : make_uint2(0u, 0u);
            }
        }
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(bars + s), parity, status))) { lost = true; break; }
        const uint8_t *tile = tiles + s * Q4K_TILE_BYTES;
        const uint4 hA = *reinterpret_cast<const uint4 *>(tile + g * 144);
        const uint4 qA0 = *reinterpret_cast<const uint4 *>(tile + g * 144 + 16 + 32 * t);
        const uint4 qA1 = *reinterpret_cast<const uint4 *>(tile + g * 144 + 32 + 32 * t);
        const uint4 hB = *reinterpret_cast<const uint4 *>(tile + (g + 8) * 144);
        const uint4 qB0 = *reinterpret_cast<const uint4 *>(tile + (g + 8) * 144 + 16 + 32 * t);
        const uint4 qB1 = *reinterpret_cast<const uint4 *>(tile + (g + 8) * 144 + 32 + 32 * t);
        __syncwarp();  // every lane holds its share: the stage may be refilled
        if (lane == 0) {
            const int nx = sb + STAGES * WPR;
            if (nx < nsb) {
                mbar_arrive_expect_tx(smem_u32(bars + s), Q4K_TILE_BYTES);
                tma_load_2d(smem_u32(tiles + s * Q4K_TILE_BYTES), &wmap, nx * 144, row0 + rg * 16,
                            smem_u32(bars + s));
            }
        }

        const uint32_t wa[8] = {qA0.x, qA0.y, qA0.z, qA0.w, qA1.x, qA1.y, qA1.z, qA1.w};
        const uint32_t wb[8] = {qB0.x, qB0.y, qB0.z, qB0.w, qB1.x, qB1.y, qB1.z, qB1.w};
        int ce[4] = {0, 0, 0, 0}, co[4] = {0, 0, 0, 0};
        const uint32_t m4 = 0x0F0F0F0Fu, h4 = 0xF0F0F0F0u;
#pragma unroll
        for (int cp = 0; cp < 4; cp++) {
            const uint2 fe = XG ? xfe[cp] : *reinterpret_cast<const uint2 *>(xf + cp * 16);
            const uint2 fo = XG ? xfo[cp] : *reinterpret_cast<const uint2 *>(xf + 64 + cp * 16);
            const uint32_t a0 = wa[2 * cp], a2 = wa[2 * cp + 1], a1 = wb[2 * cp], a3 = wb[2 * cp + 1];
            mma_u8s8(ce, a0 & m4, a1 & m4, a2 & m4, a3 & m4, fe.x, fe.y);
            mma_u8s8(co, a0 & h4, a1 & h4, a2 & h4, a3 & h4, fo.x, fo.y);   // the high nibbles in place: 16 x the code
        }

        // sub-blocks e = 2t and o = 2t+1 (format/quant/dequant.go:360-365):
        //   j < 4 : sc = q[j] & 63,                          m = q[j+4] & 63
        //   j >= 4: sc = (q[j+4] & 15) | (q[j-4] >> 6) << 4, m = (q[j+4] >> 4) | (q[j] >> 6) << 4
        const float inv_scale = __int_as_float(ax.z);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 &h = r ? hB : hA;
            const uint32_t a = h.y >> sh, b = h.z >> sh, c = h.w >> sh;
            uint32_t scp, mp;
            if (t < 2) { scp = a & 0x3F3Fu; mp = b & 0x3F3Fu; }
            else { scp = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u); mp = ((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u); }
            const int pe = (ce[2 * r] << 8) + ce[2 * r + 1];   // sum q (256 q1 + q2), sub-block e
            const int po = ((co[2 * r] << 8) + co[2 * r + 1]) >> 4;   // the odd sub-block's codes entered as 16 q: exact
            const int dotq = (int)(scp & 0xFF) * pe + (int)(scp >> 8) * po;      // < 2^31: 2 * 63 * 15 * 32 * 32639
            const int dotm = (int)(mp & 0xFF) * ax.x + (int)(mp >> 8) * ax.y;
            const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
            const float v = (dd.x * (float)dotq - dd.y * (float)dotm) * inv_scale;
            if (r) accB += v; else accA += v;
        }
    }
    if (lost && lane == 0) atomicExch(status, 1);  // a copy never landed: say so, never spin on

    accA += __shfl_xor_sync(0xffffffffu, accA, 1);
    accA += __shfl_xor_sync(0xffffffffu, accA, 2);
    accB += __shfl_xor_sync(0xffffffffu, accB, 1);
    accB += __shfl_xor_sync(0xffffffffu, accB, 2);
    if (t == 0) {
        red[warp * 16 + g] = accA;
        red[warp * 16 + g + 8] = accB;
    }
    __syncthreads();
    if (tid < 16 * RG) {  // fixed order over the warps of a row group: run-to-run bit-stable
        const int rgo = tid >> 4, r = tid & 15;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < WPR; w++) sum += red[(rgo * WPR + w) * 16 + r];
        const int row = (blockIdx.x * RG + rgo) * 16 + r;
        if (row < nrows) Y[(size_t)tok * nrows + row] = sum;
    }
}
static size_t q4k_tma_smem(int warps, int stages, int nsb, bool fused = false, bool xg = false) {
    return (size_t)warps * stages * Q4K_TILE_BYTES + (xg ? 0 : (size_t)(fused ? warps : nsb) * Q4K_XP_SB_BYTES) + Q4K_XP_ZERO_BYTES +
           (size_t)warps * 16 * 4 + (size_t)(warps * stages + 1) * 8;
}

// Scratch the Q4_K tensor-core decode needs for a shape (the prepared activation operand).
size_t jl_gemv_scratch_bytes(uint32_t type, int k, int ntok) {
    if (type == JL_TYPE_Q8_0 && k % 256 == 0) return jl_gemv_q8_scratch_bytes(k, ntok);
    if (type == JL_TYPE_MXFP4 && k % 64 == 0) return jl_gemv_mxfp4_scratch_bytes(k, ntok);
    return type == JL_TYPE_Q4_K && k % 256 == 0 ? q4k_xprep_bytes(k / 256, ntok) : 0;
}

// ------------------------------------------------------------------ dispatch

// The instantiations of the Q4_K tensor-core decode kernel, one row each: its form (jl_decode_form), warps per
// CTA, TMA ring depth per warp, CTAs per SM the registers are held to, 16-row groups per CTA. Selection returns
// an index into this table and BOTH jl_select and the launch read the same row, so what is reported is what runs.
typedef void (*q4k_kernel_fn)(const CUtensorMap, int, const void *, float *, int, int, int, int *);
struct q4k_variant {
    int form, warps, stages, minb, rg;
    q4k_kernel_fn fn;
};
#define Q4K_V(FORM, WP, ST, MB, FU, XG, RG, CP) \
    {FORM, WP, ST, MB, RG, (q4k_kernel_fn)gemv_q4k_tma_kernel<WP, ST, MB, FU, XG, RG, CP>}
static const q4k_variant q4k_variants[] = {
    // the first row of a form is the form's default
    Q4K_V(JL_FORM_SPLIT, 4, 4, 4, false, false, 1, false),
    Q4K_V(JL_FORM_SPLIT, 8, 2, 2, false, false, 1, false),
    Q4K_V(JL_FORM_SPLIT, 8, 4, 2, false, false, 1, false),
    Q4K_V(JL_FORM_SPLIT, 2, 8, 8, false, false, 1, false),
    Q4K_V(JL_FORM_FUSED, 16, 1, 1, true, false, 1, false),
    Q4K_V(JL_FORM_FUSED, 16, 2, 1, true, false, 1, false),
    Q4K_V(JL_FORM_FUSED, 8, 2, 2, true, false, 1, false),
    Q4K_V(JL_FORM_FUSED, 4, 4, 4, true, false, 1, false),
    Q4K_V(JL_FORM_WIDE, 16, 2, 1, false, false, 4, true),
    Q4K_V(JL_FORM_WIDE, 16, 2, 2, false, false, 4, true),
    Q4K_V(JL_FORM_WIDE, 16, 3, 1, false, false, 4, true),
    Q4K_V(JL_FORM_WIDE, 8, 3, 3, false, false, 4, true),
    Q4K_V(JL_FORM_WIDE, 8, 3, 3, false, false, 2, true),
    Q4K_V(JL_FORM_WIDE, 16, 2, 2, false, false, 8, true),
    Q4K_V(JL_FORM_L1, 4, 3, 8, false, true, 1, false),
    Q4K_V(JL_FORM_L1, 2, 3, 16, false, true, 1, false),
    Q4K_V(JL_FORM_L1, 4, 4, 5, false, true, 1, false),
    Q4K_V(JL_FORM_L1, 2, 8, 5, false, true, 1, false),
};
#undef Q4K_V
static const int Q4K_NVARIANTS = (int)(sizeof q4k_variants / sizeof q4k_variants[0]);

static size_t q4k_variant_smem(const q4k_variant &v, int nsb) {
    return q4k_tma_smem(v.warps, v.stages, nsb, v.form == JL_FORM_FUSED, v.form == JL_FORM_L1);
}

// First row of `form` that matches the pinned warps / stages / row groups (0 = any) and fits shared memory.
static int q4k_find(int form, int warps, int stages, int rg, int minb, int nsb) {
    for (int i = 0; i < Q4K_NVARIANTS; i++) {
        const q4k_variant &v = q4k_variants[i];
        if (v.form != form || (warps && v.warps != warps) || (stages && v.stages != stages) || (rg && v.rg != rg) ||
            (minb && v.minb != minb))
            continue;
        if (q4k_variant_smem(v, nsb) > 200 * 1024) continue;
        return i;
    }
    return -1;
}

// Which variant serves (nrows x nsb super-blocks, ntok tokens). have_x: the caller hands f32 activations (false:
// the operand was already prepared by a producer kernel, so only the forms that read a prepared operand apply).
// The reference decides per (quant, rows, k, ntok) (jit/gpu/tier/layer.go:10953-11016, tier.go:124-137).
static int q4k_pick(const jl_ctx *ctx, int nrows, int nsb, int ntok, bool have_x) {
    const jl_opts &o = ctx->opts;
    const int nrg = (nrows + 15) / 16;
    if (ctx->force_variant >= 0) return ctx->force_variant;       // a tuning trial is timing this variant
    if (have_x && o.decode_form == JL_FORM_AUTO && !o.pin_warps && !(o.flags & JL_FLAG_DECODE_CONCURRENT)) {
        // a measured verdict for this shape (tune.cu) overrides the table below
        auto it = ctx->tuned.find(jl_tune_shape_key(JL_TYPE_Q4_K, nrows, nsb * 256, ntok));
        if (it != ctx->tuned.end()) return it->second;
    }
    int form = o.decode_form;
    if (form < JL_FORM_AUTO || form > JL_FORM_L1) form = JL_FORM_AUTO;
    if (!have_x && (form == JL_FORM_FUSED || form == JL_FORM_WIDE)) form = JL_FORM_AUTO;   // those convert x themselves
    int idx = -1;
    if (form != JL_FORM_AUTO) {
        idx = q4k_find(form, o.pin_warps, o.pin_stages, o.pin_row_groups, 0, nsb);
        if (idx < 0) idx = q4k_find(form, 0, 0, 0, 0, nsb);
        if (idx >= 0) return idx;
    }
    if (o.flags & JL_FLAG_DECODE_CONCURRENT) {
        // Overlapped matvecs run into the kernel-launch rate before HBM: ONE launch per matvec, the CTA (64 rows,
        // 8 warps, weight tiles three deep) converting the activation row itself (measured at 4096x4096, 8
        // overlapped chains: 1.62 us against 1.87 us for prep + decode). With the operand already prepared, or a
        // row too long for shared memory, the small-CTA variants that read the operand through L1.
        if (have_x && nsb <= 64) idx = q4k_find(JL_FORM_WIDE, 8, 3, 4, 3, nsb);
        if (idx < 0) idx = nrg >= 512 ? q4k_find(JL_FORM_L1, 2, 3, 1, 0, nsb) : q4k_find(JL_FORM_L1, 4, 3, 1, 0, nsb);
        if (idx >= 0) return idx;
    }
    if (have_x && nsb <= 16 && nrows >= 1024) {
        // A lone matvec of a short row: the single-launch wide form also has the shortest chain (4096x4096: 5.1 us
        // against 5.9 us); one CTA per SM while the launch fits one wave, two above.
        idx = q4k_find(JL_FORM_WIDE, 16, 2, 4, (nrows + 63) / 64 <= ctx->sm_count ? 1 : 2, nsb);
        if (idx >= 0 && (!o.pin_warps || o.pin_warps == 16)) return idx;
    }
    // Latency-bound shapes (about one wave of warp-tasks or less) take the fused form, the rest the split form.
    const long tasks = (long)nrg * nsb * ntok;
    form = (have_x && tasks <= (long)ctx->sm_count * 16) ? JL_FORM_FUSED : JL_FORM_SPLIT;
    idx = q4k_find(form, o.pin_warps, o.pin_stages, 0, 0, nsb);
    if (idx < 0) idx = q4k_find(form, 0, 0, 0, 0, nsb);
    if (idx < 0) idx = q4k_find(JL_FORM_SPLIT, 0, 0, 0, 0, nsb);
    return idx;
}

// tune.cu: the variants a shape may run, the table's pick first.
int jl_gemv_tune_candidates(jl_ctx *ctx, int nrows, int k, int ntok, int *out, int cap) {
    const int nsb = k / 256;
    if (k % 256 || ntok < 1 || ntok > 8 || cap < 1) return 0;
    const uint64_t key = jl_tune_shape_key(JL_TYPE_Q4_K, nrows, k, ntok);
    int held = -1;
    auto it = ctx->tuned.find(key);
    if (it != ctx->tuned.end()) { held = it->second; ctx->tuned.erase(it); }
    const int first = q4k_pick(ctx, nrows, nsb, ntok, true);
    if (held >= 0) ctx->tuned[key] = held;
    if (first < 0) return 0;
    int n = 0;
    out[n++] = first;
    for (int i = 0; i < Q4K_NVARIANTS && n < cap; i++)
        if (i != first && q4k_variant_smem(q4k_variants[i], nsb) <= 200 * 1024) out[n++] = i;
    return n;
}
int jl_gemv_variant_index(int form, int warps, int stages, int minb, int rg, int nsb) {
    if (warps < 1 || stages < 1 || minb < 1 || rg < 1) return -1;
    return q4k_find(form, warps, stages, rg, minb, nsb);
}
void jl_gemv_variant_describe(int idx, int *form, int *warps, int *stages, int *minb, int *rg) {
    const q4k_variant &v = q4k_variants[idx];
    *form = v.form; *warps = v.warps; *stages = v.stages; *minb = v.minb; *rg = v.rg;
}

static bool q4k_mma_ok(uint32_t type, int k) {
    // the activation operand of the whole row must fit one CTA's shared memory beside the default ring
    return type == JL_TYPE_Q4_K && k % 256 == 0 && q4k_find(JL_FORM_SPLIT, 0, 0, 0, 0, k / 256) >= 0;
}

static void q4k_fill_choice(const q4k_variant &v, int nrows, int nsb, int ntok, jl_choice *c) {
    const int wpr = v.warps / v.rg;
    c->kernel = JL_K_MMA; c->form = v.form; c->warps = v.warps; c->stages = v.stages; c->rows_per_cta = 16 * v.rg;
    c->split_k = wpr < nsb ? wpr : nsb;
    c->tile_m = 16; c->tile_n = 8; c->tile_k = 32;
    c->grid = (((nrows + 15) / 16 + v.rg - 1) / v.rg) * ntok;
    c->launches = (v.form == JL_FORM_SPLIT || v.form == JL_FORM_L1) ? 2 : 1;   // the prep launch in front
}

int jl_gemv_choice(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out) {
    jl_choice c = {};
    const int pin = ctx->opts.pin_kernel;
    if (type == JL_TYPE_MXFP4 && k % 64 == 0 && pin != JL_K_SIMT) {
        // e2m1 codes become f16 A fragments by bit placement; mma.sync.m16n8k16, four tokens per launch row
        if (pin == JL_K_TC5) return JL_DECLINED;
        const int nspan = k / 64;
        c.kernel = JL_K_MMA; c.warps = nspan >= 32 ? 8 : (nspan >= 16 ? 4 : (nspan >= 8 ? 2 : 1)); c.rows_per_cta = 16;
        c.split_k = c.warps; c.tile_m = 16; c.tile_n = 8; c.tile_k = 16;
        c.grid = (nrows + 15) / 16 * ((ntok + 3) / 4);
        c.launches = 2;
        *out = c;
        return JL_OK;
    }
    if (type == JL_TYPE_Q8_0 && k % 256 == 0 && pin != JL_K_SIMT) {
        // int8 codes feed mma.sync.m16n8k32.s8.s8 as they are; four tokens per launch row
        if (pin == JL_K_TC5) return JL_DECLINED;
        const int ngrp = k / 256;
        c.kernel = JL_K_MMA; c.warps = ngrp >= 8 ? 8 : (ngrp >= 4 ? 4 : (ngrp >= 2 ? 2 : 1)); c.rows_per_cta = 16;
        c.split_k = c.warps; c.tile_m = 16; c.tile_n = 8; c.tile_k = 32;
        const int tgroups = (ntok + 3) / 4, ntg = tgroups >= 4 ? 4 : (tgroups >= 2 ? 2 : 1);
        c.grid = (nrows + 15) / 16 * ((tgroups + ntg - 1) / ntg);
        if (ntok > 8 && ntok <= 32) {   // the batch kernel: a row tile per CTA, k-slices as one cluster
            int bw, ks;
            jl_gemv_q8_batch_plan(nrows, k, &bw, &ks);
            c.warps = bw; c.rows_per_cta = 16 * bw; c.split_k = ks;
            c.grid = (nrows + 16 * bw - 1) / (16 * bw) * ks;
        }
        c.launches = 2;
        *out = c;
        return JL_OK;
    }
    if (pin == JL_K_SIMT || !q4k_mma_ok(type, k) || (ctx->opts.flags & JL_FLAG_NO_TMA)) {
        if (pin == JL_K_MMA || pin == JL_K_TC5) return JL_DECLINED;
        c.kernel = JL_K_SIMT; c.warps = 8; c.rows_per_cta = 8; c.split_k = 1;
        c.grid = (nrows + 7) / 8 * ntok;
        c.launches = 1;
    } else {
        const int idx = q4k_pick(ctx, nrows, k / 256, ntok, true);
        if (idx < 0) return JL_DECLINED;
        q4k_fill_choice(q4k_variants[idx], nrows, k / 256, ntok, &c);
    }
    *out = c;
    return JL_OK;
}

int jl_launch_gemv(jl_ctx *ctx, float *out_dev, const jl_weight *w, int expert, const float *x_dev,
                   int ntok, int kernel, cudaStream_t s) {
    const int nrows = w->nrows, k = w->k;
    size_t rows_off = (size_t)expert * nrows;
    const uint8_t *data = w->data;
    const uint8_t *scales = w->scales;
    if (w->type == JL_TYPE_Q4_K || jl_type_raw_simt(w->type)) data += rows_off * jl_row_bytes(w->type, k);
    else if (w->type == JL_TYPE_Q8_0) { data += rows_off * (size_t)k; scales += rows_off * (size_t)w->scale_stride * 2; }
    else { data += rows_off * (size_t)(k / 32) * 16; scales += rows_off * (size_t)w->scale_stride; }

    if (kernel == JL_K_MMA && w->type == JL_TYPE_MXFP4)
        return jl_launch_gemv_mxfp4(ctx, out_dev, data, scales, w->scale_stride, x_dev, nrows, k, ntok, s);
    if (kernel == JL_K_MMA && w->type == JL_TYPE_Q8_0)
        return jl_launch_gemv_q8(ctx, out_dev, data, scales, w->scale_stride, x_dev, nrows, k, ntok, s);
    if (kernel == JL_K_MMA && !w->has_map_sb16) {
        if (ctx->opts.pin_kernel == JL_K_MMA)
            return jl_set_err(ctx, JL_DECLINED, "the tensor-core decode kernel needs the weight's tensor map");
        kernel = JL_K_SIMT;
    }
    if (kernel == JL_K_MMA && w->type == JL_TYPE_Q4_K) {
        const int nsb = k / 256;
        const size_t need = q4k_xprep_bytes(nsb, ntok);
        if (ctx->scratch_cap < need)
            return jl_set_err(ctx, JL_ENOMEM, "decode scratch holds %zu bytes, %d x %d token(s) need %zu "
                              "(jl_reserve sizes it)", ctx->scratch_cap, k, ntok, need);
        uint8_t *scratch = (uint8_t *)ctx->scratch;
        const bool prepared = x_dev == nullptr;   // the caller's kernels wrote the operand into the scratch already
        const int idx = q4k_pick(ctx, nrows, nsb, ntok, !prepared);
        if (idx < 0) return jl_set_err(ctx, JL_DECLINED, "no decode variant fits %d x %d", nrows, k);
        const q4k_variant &v = q4k_variants[idx];
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        const int nattr = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
        const bool converts = v.form == JL_FORM_FUSED || v.form == JL_FORM_WIDE;   // the kernel reads x itself
        if (!converts && !prepared) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((nsb + 3) / 4, ntok); cfg.blockDim = dim3(128); cfg.stream = s;
            cfg.attrs = at; cfg.numAttrs = nattr;
            JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, q4k_xprep_kernel, x_dev, scratch, nsb, ntok));
            ctx->st.launches++;
        }
        const void *xsrc = converts ? (const void *)x_dev : (const void *)scratch;
        const size_t smem = q4k_variant_smem(v, nsb);
        if (smem > 48 * 1024)
            JL_CUDA(ctx, cudaFuncSetAttribute((const void *)v.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(((nrows + 15) / 16 + v.rg - 1) / v.rg, ntok); cfg.blockDim = dim3(v.warps * 32);
        cfg.dynamicSmemBytes = smem; cfg.stream = s; cfg.attrs = at; cfg.numAttrs = nattr;
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, v.fn, w->map_sb16, expert * nrows, xsrc, out_dev, nrows, nsb, ntok,
                                        ctx->dev_status));
    } else {
        dim3 grid((nrows + 7) / 8, ntok);
        const dim3 g1((nrows + 7) / 8, 1), g4((nrows + 7) / 8, (ntok + 3) / 4);
#define JL_ROWK(KERNEL) do { if (ntok == 1) KERNEL<1><<<g1, 256, 0, s>>>(data, x_dev, out_dev, nrows, k, ntok); \
                             else KERNEL<4><<<g4, 256, 0, s>>>(data, x_dev, out_dev, nrows, k, ntok); } while (0)
#define JL_ROWK45(T) do { if (ntok == 1) gemv_q45_kernel<T, 1><<<g1, 256, 0, s>>>(data, x_dev, out_dev, nrows, k, ntok); \
                           else gemv_q45_kernel<T, 4><<<g4, 256, 0, s>>>(data, x_dev, out_dev, nrows, k, ntok); } while (0)
        // the raw formats' own row kernels (a lane takes many codes at a time; up to four tokens share the decoded weights)
        if (w->type == JL_TYPE_Q6_K) JL_ROWK(gemv_q6k_kernel);
        else if (w->type == JL_TYPE_Q5_K) JL_ROWK(gemv_q5k_kernel);
        else if (w->type == JL_TYPE_Q4_0) JL_ROWK45(JL_TYPE_Q4_0);
        else if (w->type == JL_TYPE_Q5_0) JL_ROWK45(JL_TYPE_Q5_0);
        else if (w->type == JL_TYPE_Q5_1) JL_ROWK45(JL_TYPE_Q5_1);
#undef JL_ROWK
#undef JL_ROWK45
        else if (w->type == JL_TYPE_Q4_K)
            gemv_simt_kernel<JL_TYPE_Q4_K><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
        else if (w->type == JL_TYPE_Q8_0)
            gemv_simt_kernel<JL_TYPE_Q8_0><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
        else if (w->type == JL_TYPE_MXFP4)
            gemv_simt_kernel<JL_TYPE_MXFP4><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
#define JL_SIMT_RAW(T) else if (w->type == T) gemv_simt_kernel<T><<<grid, 256, 0, s>>>(data, scales, w->scale_stride, x_dev, out_dev, nrows, k, ntok);
        JL_SIMT_RAW(JL_TYPE_Q4_0) JL_SIMT_RAW(JL_TYPE_Q5_0) JL_SIMT_RAW(JL_TYPE_Q5_1) JL_SIMT_RAW(JL_TYPE_Q5_K) JL_SIMT_RAW(JL_TYPE_Q6_K)
#undef JL_SIMT_RAW
        else return jl_set_err(ctx, JL_DECLINED, "type %u has no decode kernel", w->type);
    }
    ctx->st.launches++;
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}

// ------------------------------------------------------ allocation-free entry point
//
// jl_matvec_q4k_noalloc is for callers that may not allocate device memory: code running
// under a stream capture or inside another library's allocator callbacks, a runtime that
// pre-plans every byte of HBM and forbids late cudaMalloc, a real-time serving loop where an
// allocation would mean a device-wide synchronisation. It is the split form of the Q4_K
// decode (activation prep kernel -> tensor-core kernel) with the prepared activation
// operand kept in a fixed __device__ array instead of a context's scratch buffer.
//
// The array belongs to the loaded library: every GPU that loads it holds the
// JL_NOALLOC_SCRATCH_BYTES until the process exits, every call on a device shares it (calls
// whose kernels can overlap on the GPU race on it: keep them on one stream), and a call
// finds the previous call's contents there -- the prep kernel rewrites every byte the
// decode kernel reads, so nothing has to start at zero except the status words, which the
// kernels only ever set and jl_noalloc_status clears.
#define JL_NOALLOC_MAX_K 16384
#define JL_NOALLOC_SCRATCH_BYTES ((JL_NOALLOC_MAX_K / 256) * Q4K_XP_SB_BYTES + Q4K_XP_ZERO_BYTES)
static __device__ __align__(256) uint8_t jl_noalloc_scratch[JL_NOALLOC_SCRATCH_BYTES];
static __device__ int jl_noalloc_status_words[2];   // [0] timeout code, [1] wait limit (0 = default)

// In host code the names above are only handles of the symbols; the device addresses are
// asked for once per device, with that device current.
static std::mutex jl_noalloc_mu;
static uint8_t *jl_noalloc_scratch_addr[64];
static int *jl_noalloc_status_addr[64];

static int jl_noalloc_setup(int *dev_out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return JL_ECUDA;
    std::lock_guard<std::mutex> lk(jl_noalloc_mu);
    if (!jl_noalloc_scratch_addr[dev]) {   // first call on this device: before any stream capture
        void *p = nullptr, *q = nullptr;
        if (cudaGetSymbolAddress(&p, jl_noalloc_scratch) != cudaSuccess) { cudaGetLastError(); return JL_ECUDA; }
        if (cudaGetSymbolAddress(&q, jl_noalloc_status_words) != cudaSuccess) { cudaGetLastError(); return JL_ECUDA; }
        jl_noalloc_scratch_addr[dev] = (uint8_t *)p;
        jl_noalloc_status_addr[dev] = (int *)q;
    }
    *dev_out = dev;
    return JL_OK;
}

JL_EXPORT int jl_noalloc_max_k(void) { return JL_NOALLOC_MAX_K; }

// Reads and clears the entry point's status word on the current device: JL_ETIMEDOUT when a
// bounded wait of an earlier call ran out (that call's output is then incomplete). Copies
// through the caller's stack; allocates nothing.
JL_EXPORT int jl_noalloc_status(void *stream) {
    int dev;
    int rc = jl_noalloc_setup(&dev);
    if (rc) return rc;
    int word = 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (cudaMemcpyAsync(&word, jl_noalloc_status_addr[dev], sizeof word, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        cudaGetLastError();
        return JL_ECUDA;
    }
    if (!word) return JL_OK;
    if (cudaMemsetAsync(jl_noalloc_status_addr[dev], 0, sizeof(int), s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
        cudaGetLastError();
        return JL_ECUDA;
    }
    return JL_ETIMEDOUT;
}

JL_EXPORT int jl_matvec_q4k_noalloc(float *out_dev, const void *w_dev, const float *x_dev, int nrows, int k,
                                    void *stream) {
    if (!out_dev || !w_dev || !x_dev || nrows < 1 || k < 256 || k % 256) return JL_EINVAL;
    if (k > JL_NOALLOC_MAX_K) return JL_ENOMEM;   // beyond the fixed scratch: refuse, never grow
    if (((uintptr_t)w_dev & 15) || ((uintptr_t)x_dev & 15)) return JL_EINVAL;
    int dev;
    int rc = jl_noalloc_setup(&dev);
    if (rc) return rc;
    uint8_t *scratch = jl_noalloc_scratch_addr[dev];
    int *status = jl_noalloc_status_addr[dev];
    const int nsb = k / 256;
    const size_t row_bytes = (size_t)nsb * 144;
    CUtensorMap map;   // encoded on the host into this stack object: no device memory involved
    if (!jl_make_tmap_2d(&map, w_dev, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, (uint64_t)nrows, row_bytes, 144, 16,
                         CU_TENSOR_MAP_SWIZZLE_NONE))
        return JL_ENOTSUP;
    cudaStream_t s = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((nsb + 3) / 4, 1); cfg.blockDim = dim3(128); cfg.stream = s;
        cfg.attrs = at; cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, q4k_xprep_kernel, x_dev, scratch, nsb, 1) != cudaSuccess) {
            cudaGetLastError();
            return JL_ECUDA;
        }
    }
    const size_t smem = q4k_tma_smem(4, 4, nsb, false);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(gemv_q4k_tma_kernel<4, 4, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return JL_ECUDA;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((nrows + 15) / 16, 1); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gemv_q4k_tma_kernel<4, 4, 4, false>, map, 0, (const void *)scratch, out_dev, nrows,
                           nsb, 1, status) != cudaSuccess) {
        cudaGetLastError();
        return JL_ECUDA;
    }
    return JL_OK;
}
