/*
 * jl_oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A CPU restatement, in plain C, of the arithmetic jitllm's quantized-matmul
 * path is defined by. Nothing the library ships links, loads or calls this
 * file: only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg do, and there only as the checker / the thing timed as "the CPU path".
 *
 * The reference is Go and no Go toolchain exists on the build machine, so the
 * reference itself cannot be run. Every function below names the reference
 * file:line it restates. The block decoders are pinned bit-for-bit against the
 * reference's committed golden vectors (llama.cpp / gguf-py outputs); the
 * matvec/matmul/MoE OUTPUT arithmetic has no committed vector in the reference
 * tree ("parity unpinned by committed vectors" for those) and is pinned by
 * construction: it is the composition of the pinned decoders with a
 * compensated / f64 dot product.
 *
 * Build: see oracle/Makefile (gcc -O2, no -march flags: SIMD arms are selected
 * at run time with __builtin_cpu_supports so the .so runs on any x86-64 host).
 */
#define _GNU_SOURCE
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ggml type ids -- format/quant/types.go:12-55 */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q5_K = 13,
       ORC_Q6_K = 14, ORC_BF16 = 30, ORC_MXFP4 = 39 };

/* format/quant/types.go:61-85 (blockInfo): elements and bytes per block. */
ORC_API int orc_block_elems(uint32_t t) {
    switch (t) {
    case ORC_F32: case ORC_F16: case ORC_BF16: return 1;
    case ORC_Q8_0: case ORC_Q4_0: case ORC_Q5_0: case ORC_Q5_1: return 32;
    case ORC_Q4_K: case ORC_Q5_K: case ORC_Q6_K: return 256;
    case ORC_MXFP4: return 32;
    }
    return 0;
}
ORC_API int orc_block_bytes(uint32_t t) {
    switch (t) {
    case ORC_F32: return 4;
    case ORC_F16: case ORC_BF16: return 2;
    case ORC_Q8_0: return 34;
    case ORC_Q4_0: return 18;
    case ORC_Q5_0: return 22;
    case ORC_Q5_1: return 24;
    case ORC_Q4_K: return 144;
    case ORC_Q5_K: return 176;
    case ORC_Q6_K: return 210;
    case ORC_MXFP4: return 17;
    }
    return 0;
}

/* ------------------------------------------------------------------ half */

/* format/quant/dequant.go:12-32 (DecodeHalf / f16): exact binary16 -> f64. */
ORC_API double orc_half_decode(uint16_t u) {
    double sign = (u & 0x8000) ? -1.0 : 1.0;
    int exp = (u >> 10) & 0x1f;
    int mant = u & 0x3ff;
    if (exp == 0) return sign * (double)mant * ldexp(1.0, -24);
    if (exp == 0x1f) return mant ? NAN : sign * INFINITY;
    return sign * (double)(1024 + mant) * ldexp(1.0, exp - 25);
}

/* format/quant/dequant.go:478-517 (EncodeHalf): f32 -> binary16, RNE. */
ORC_API uint16_t orc_half_encode(float f) {
    uint32_t b; memcpy(&b, &f, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
    int32_t exp = (int32_t)(b >> 23) & 0xFF;
    uint32_t man = b & 0x7FFFFF;
    if (exp == 0xFF) return man ? (sign | 0x7E00) : (sign | 0x7C00);
    int32_t e = exp - 127 + 15;
    if (e >= 0x1F) return sign | 0x7C00;
    if (e <= 0) {
        if (e < -10) return sign;
        man |= 0x800000;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t h = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) h++;
        return sign | (uint16_t)h;
    }
    uint16_t h = (uint16_t)((uint16_t)e << 10 | (uint16_t)(man >> 13));
    uint32_t rem = man & 0x1FFF;
    if (rem > 0x1000 || (rem == 0x1000 && (h & 1))) h++;
    return sign | h;
}

static inline uint16_t le16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* The same value as orc_half_decode, by bit manipulation (exact; used in the
 * timed loops where a libm call per block would dominate). */
static inline float half_to_f32(uint16_t u) {
    uint32_t sign = (uint32_t)(u & 0x8000) << 16, exp = (u >> 10) & 0x1f, man = u & 0x3ff, b;
    if (exp == 0) {
        if (!man) b = sign;
        else {
            int sh = 0;
            while (!(man & 0x400)) { man <<= 1; sh++; }
            b = sign | (uint32_t)(113 - sh) << 23 | (man & 0x3ff) << 13;
        }
    } else if (exp == 0x1f) b = sign | 0x7f800000u | man << 13;
    else b = sign | (exp + 112) << 23 | man << 13;
    float f; memcpy(&f, &b, 4);
    return f;
}

/* ------------------------------------------------------------- decoders */

/* format/quant/dequant.go:360-365 and jit/gpu/kernels/pack.go:422-428. */
static inline void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) { *sc = q[j] & 63; *m = q[j + 4] & 63; return; }
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *m  = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
}

/* format/quant/dequant.go:266-268 (MXFP4Values): e2m1 doubled. */
static const int8_t k_mxfp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

/* One decoder body, two destinations, like the reference's generic dequant
 * (format/quant/dequant.go:55-264). STORE narrows once. */
#define DEQUANT_BODY(T)                                                                     \
    int be = orc_block_elems(t), bb = orc_block_bytes(t);                                   \
    if (!be) return -1;                                                                     \
    if (n % (size_t)be) return -2;                                                          \
    size_t blocks = n / (size_t)be;                                                         \
    switch (t) {                                                                            \
    case ORC_F32:                                                                           \
        for (size_t i = 0; i < n; i++) { float v; memcpy(&v, src + 4 * i, 4); dst[i] = (T)v; } \
        break;                                                                              \
    case ORC_F16:                                                                           \
        for (size_t i = 0; i < n; i++) dst[i] = (T)orc_half_decode(le16(src + 2 * i));      \
        break;                                                                              \
    case ORC_BF16:                                                                          \
        for (size_t i = 0; i < n; i++) {                                                    \
            uint32_t u = (uint32_t)le16(src + 2 * i) << 16; float v; memcpy(&v, &u, 4);     \
            dst[i] = (T)v;                                                                  \
        }                                                                                   \
        break;                                                                              \
    case ORC_Q8_0: /* dequant.go:148-157: {f16 d; i8 qs[32]} */                             \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const uint8_t *blk = src + b * 34;                                              \
            double d = orc_half_decode(le16(blk));                                          \
            for (int j = 0; j < 32; j++) dst[b * 32 + j] = (T)((double)(int8_t)blk[2 + j] * d); \
        }                                                                                   \
        break;                                                                              \
    case ORC_MXFP4: /* dequant.go:159-174: {u8 e; u8 qs[16]}, lo=j, hi=j+16, 2^(e-128) */   \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const uint8_t *blk = src + b * 17;                                              \
            double d = ldexp(1.0, (int)blk[0] - 128);                                       \
            for (int j = 0; j < 16; j++) {                                                  \
                dst[b * 32 + j]      = (T)((double)k_mxfp4[blk[1 + j] & 0xF] * d);          \
                dst[b * 32 + j + 16] = (T)((double)k_mxfp4[blk[1 + j] >> 4] * d);           \
            }                                                                               \
        }                                                                                   \
        break;                                                                              \
    case ORC_Q4_K: /* dequant.go:367-397: products and the subtraction in f32 */            \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const uint8_t *blk = src + b * 144;                                             \
            float d = (float)orc_half_decode(le16(blk));                                    \
            float dmin = (float)orc_half_decode(le16(blk + 2));                             \
            const uint8_t *scales = blk + 4, *qs = blk + 16;                                \
            size_t o = b * 256; int is = 0;                                                 \
            for (int j = 0; j < 256; j += 64) {                                             \
                const uint8_t *q = qs + j / 2;                                              \
                uint8_t sc1, m1, sc2, m2;                                                   \
                scale_min_k4(is, scales, &sc1, &m1);                                        \
                scale_min_k4(is + 1, scales, &sc2, &m2);                                    \
                volatile float d1 = d * (float)sc1, min1 = dmin * (float)m1;                \
                volatile float d2 = d * (float)sc2, min2 = dmin * (float)m2;                \
                for (int l = 0; l < 32; l++) {                                              \
                    volatile float p = d1 * (float)(q[l] & 0xF);                            \
                    volatile float v = p - min1; dst[o++] = (T)(double)v;                   \
                }                                                                           \
                for (int l = 0; l < 32; l++) {                                              \
                    volatile float p = d2 * (float)(q[l] >> 4);                             \
                    volatile float v = p - min2; dst[o++] = (T)(double)v;                   \
                }                                                                           \
                is += 2;                                                                    \
            }                                                                               \
        }                                                                                   \
        break;                                                                              \
    case ORC_Q4_0: /* dequant.go:85-101: {f16 d; u8 qs[16]}, lo = j, hi = j + 16, (q - 8) d in f64 */ \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const uint8_t *blk = src + b * 18;                                              \
            double d = orc_half_decode(le16(blk));                                          \
            for (int j = 0; j < 16; j++) {                                                  \
                dst[b * 32 + j]      = (T)((double)((int)(blk[2 + j] & 0xF) - 8) * d);      \
                dst[b * 32 + j + 16] = (T)((double)((int)(blk[2 + j] >> 4) - 8) * d);       \
            }                                                                               \
        }                                                                                   \
        break;                                                                              \
    case ORC_Q5_0: /* dequant.go:103-125: {f16 d; u32 qh; u8 qs[16]}, element l takes bit l of qh */ \
    case ORC_Q5_1: /* dequant.go:127-146: {f16 d; f16 m; u32 qh; u8 qs[16]}, d q + m */     \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const int one = t == ORC_Q5_1;                                                  \
            const uint8_t *blk = src + b * (one ? 24 : 22);                                 \
            double d = orc_half_decode(le16(blk));                                          \
            double m = one ? orc_half_decode(le16(blk + 2)) : 0;                            \
            const uint8_t *hp = blk + (one ? 4 : 2), *qs = hp + 4;                          \
            uint32_t qh = (uint32_t)hp[0] | (uint32_t)hp[1] << 8 | (uint32_t)hp[2] << 16 | (uint32_t)hp[3] << 24; \
            for (int j = 0; j < 16; j++) {                                                  \
                int lo = qs[j] & 0xF, hi = qs[j] >> 4;                                      \
                if (qh & (1u << j)) lo += 16;                                               \
                if (qh & (1u << (j + 16))) hi += 16;                                        \
                dst[b * 32 + j]      = one ? (T)((double)lo * d + m) : (T)((double)(lo - 16) * d); \
                dst[b * 32 + j + 16] = one ? (T)((double)hi * d + m) : (T)((double)(hi - 16) * d); \
            }                                                                               \
        }                                                                                   \
        break;                                                                              \
    case ORC_Q5_K: /* dequant.go:399-441: {f16 d, dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} */ \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const uint8_t *blk = src + b * 176;                                             \
            float d = (float)orc_half_decode(le16(blk));                                    \
            float dmin = (float)orc_half_decode(le16(blk + 2));                             \
            const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;                \
            size_t o = b * 256; int is = 0; uint8_t u1 = 1, u2 = 2;                         \
            for (int j = 0; j < 256; j += 64) {                                             \
                const uint8_t *q = qs + j / 2;                                              \
                uint8_t sc1, m1, sc2, m2;                                                   \
                scale_min_k4(is, scales, &sc1, &m1);                                        \
                scale_min_k4(is + 1, scales, &sc2, &m2);                                    \
                volatile float d1 = d * (float)sc1, min1 = dmin * (float)m1;                \
                volatile float d2 = d * (float)sc2, min2 = dmin * (float)m2;                \
                for (int l = 0; l < 32; l++) {                                              \
                    int v = (q[l] & 0xF) + ((qh[l] & u1) ? 16 : 0);                         \
                    volatile float p = d1 * (float)v;                                       \
                    volatile float w = p - min1; dst[o++] = (T)(double)w;                   \
                }                                                                           \
                for (int l = 0; l < 32; l++) {                                              \
                    int v = (q[l] >> 4) + ((qh[l] & u2) ? 16 : 0);                          \
                    volatile float p = d2 * (float)v;                                       \
                    volatile float w = p - min2; dst[o++] = (T)(double)w;                   \
                }                                                                           \
                is += 2; u1 = (uint8_t)(u1 << 2); u2 = (uint8_t)(u2 << 2);                  \
            }                                                                               \
        }                                                                                   \
        break;                                                                              \
    case ORC_Q6_K: /* dequant.go:443-470: {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}, (d sc) q in f32 */ \
        for (size_t b = 0; b < blocks; b++) {                                               \
            const uint8_t *blk = src + b * 210;                                             \
            float d = (float)orc_half_decode(le16(blk + 208));                              \
            for (int n = 0; n < 256; n += 128) {                                            \
                const uint8_t *ql = blk + n / 2, *qh = blk + 128 + n / 4;                   \
                const int8_t *sc = (const int8_t *)(blk + 192 + n / 16);                    \
                for (int l = 0; l < 32; l++) {                                              \
                    int is = l / 16;                                                        \
                    int q[4];                                                               \
                    q[0] = (int)(int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;   \
                    q[1] = (int)(int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32; \
                    q[2] = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;    \
                    q[3] = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32; \
                    for (int j = 0; j < 4; j++) {                                           \
                        volatile float ds = d * (float)sc[is + 2 * j];                      \
                        volatile float w = ds * (float)q[j];                                \
                        dst[b * 256 + n + 32 * j + l] = (T)(double)w;                       \
                    }                                                                       \
                }                                                                           \
            }                                                                               \
        }                                                                                   \
        break;                                                                              \
    default: return -1;                                                                     \
    }                                                                                       \
    (void)bb;                                                                               \
    return 0;

/* quant.Dequant32 (dequant.go:50). n = number of ELEMENTS. */
ORC_API int orc_dequant_f32(uint32_t t, const uint8_t *src, size_t n, float *dst) { DEQUANT_BODY(float) }
/* quant.Dequant (dequant.go:40). */
ORC_API int orc_dequant_f64(uint32_t t, const uint8_t *src, size_t n, double *dst) { DEQUANT_BODY(double) }

/* ------------------------------------------------- integer unpack (extract) */

/* jit/gpu/kernels/pack.go:252-386 (extract) + :388-395 (e8m0Store), for the
 * three formats on this path. One record per 32-element SUB-block:
 *   q[32]  the integer codes (Q4_K 0..15, Q8_0 -128..127, MXFP4 raw e2m1 code)
 *   d      raw f16 bits of the super-scale (MXFP4: the stored byte e-1)
 *   dmin   raw f16 bits of the super-minimum (Q4_K only, else 0)
 *   sc, m  6-bit sub-block scale and minimum (Q4_K only, else 0)
 * nblocks counts FORMAT blocks (a Q4_K block yields 8 records). */
ORC_API int orc_unpack(uint32_t t, const uint8_t *src, size_t nblocks, int8_t *q,
                       uint16_t *d, uint16_t *dmin, uint8_t *sc, uint8_t *m) {
    size_t r = 0;
    switch (t) {
    case ORC_Q8_0:
        for (size_t b = 0; b < nblocks; b++, r++) {
            const uint8_t *blk = src + b * 34;
            for (int l = 0; l < 32; l++) q[r * 32 + l] = (int8_t)blk[2 + l];
            d[r] = le16(blk); dmin[r] = 0; sc[r] = 0; m[r] = 0;
        }
        return 0;
    case ORC_MXFP4:
        for (size_t b = 0; b < nblocks; b++, r++) {
            const uint8_t *blk = src + b * 17;
            for (int l = 0; l < 16; l++) {
                q[r * 32 + l] = (int8_t)(blk[1 + l] & 0xF);
                q[r * 32 + l + 16] = (int8_t)(blk[1 + l] >> 4);
            }
            d[r] = (uint16_t)(uint8_t)(blk[0] - 1); dmin[r] = 0; sc[r] = 0; m[r] = 0;
        }
        return 0;
    case ORC_Q4_K:
        for (size_t b = 0; b < nblocks; b++) {
            const uint8_t *blk = src + b * 144;
            for (int s = 0; s < 8; s++, r++) {
                scale_min_k4(s, blk + 4, &sc[r], &m[r]);
                const uint8_t *grp = blk + 16 + (s / 2) * 32;
                for (int l = 0; l < 32; l++)
                    q[r * 32 + l] = (int8_t)((s % 2 == 0) ? (grp[l] & 0xF) : (grp[l] >> 4));
                d[r] = le16(blk); dmin[r] = le16(blk + 2);
            }
        }
        return 0;
    case ORC_Q4_0:   /* pack.go:254-259 */
        for (size_t b = 0; b < nblocks; b++, r++) {
            const uint8_t *blk = src + b * 18;
            for (int l = 0; l < 16; l++) {
                q[r * 32 + l] = (int8_t)(blk[2 + l] & 0xF);
                q[r * 32 + l + 16] = (int8_t)(blk[2 + l] >> 4);
            }
            d[r] = le16(blk); dmin[r] = 0; sc[r] = 0; m[r] = 0;
        }
        return 0;
    case ORC_Q5_0:   /* pack.go:261-273 */
    case ORC_Q5_1:   /* pack.go:275-290: the minimum goes out with its sign bit flipped */
        for (size_t b = 0; b < nblocks; b++, r++) {
            const int one = t == ORC_Q5_1;
            const uint8_t *blk = src + b * (one ? 24 : 22);
            const uint8_t *hp = blk + (one ? 4 : 2), *qs = hp + 4;
            uint32_t qh = (uint32_t)hp[0] | (uint32_t)hp[1] << 8 | (uint32_t)hp[2] << 16 | (uint32_t)hp[3] << 24;
            for (int l = 0; l < 16; l++) {
                q[r * 32 + l] = (int8_t)(qs[l] & 0xF);
                q[r * 32 + l + 16] = (int8_t)(qs[l] >> 4);
            }
            for (int l = 0; l < 32; l++)
                if (qh & (1u << l)) q[r * 32 + l] = (int8_t)(q[r * 32 + l] + 16);
            d[r] = le16(blk); dmin[r] = one ? (uint16_t)(le16(blk + 2) ^ 0x8000) : 0; sc[r] = 0; m[r] = 0;
        }
        return 0;
    case ORC_Q5_K:   /* pack.go:332-348 */
        for (size_t b = 0; b < nblocks; b++) {
            const uint8_t *blk = src + b * 176;
            for (int s = 0; s < 8; s++, r++) {
                scale_min_k4(s, blk + 4, &sc[r], &m[r]);
                const uint8_t *qh = blk + 16, *ql = blk + 48 + (s / 2) * 32;
                for (int l = 0; l < 32; l++) {
                    int v = (s % 2 == 1) ? (ql[l] >> 4) : (ql[l] & 0xF);
                    if (qh[l] & (1u << s)) v += 16;
                    q[r * 32 + l] = (int8_t)v;
                }
                d[r] = le16(blk); dmin[r] = le16(blk + 2);
            }
        }
        return 0;
    case ORC_Q6_K:   /* pack.go:367-384: one record per SIXTEEN elements; the scale stored biased by 128 */
        for (size_t b = 0; b < nblocks; b++) {
            const uint8_t *blk = src + b * 210;
            for (int s = 0; s < 16; s++, r++) {
                int g = s / 8, e0 = (s % 8) * 16;
                const uint8_t *ql = blk + g * 64, *qh = blk + 128 + g * 32;
                for (int l = 0; l < 16; l++) {
                    int e = e0 + l, lo = e % 32, sh = 2 * (e / 32);
                    uint8_t nib = ql[lo + (e / 32) % 2 * 32];
                    nib = (e / 32 >= 2) ? (uint8_t)(nib >> 4) : (uint8_t)(nib & 0xF);
                    q[r * 16 + l] = (int8_t)(nib | (((qh[lo] >> sh) & 3) << 4));
                }
                d[r] = le16(blk + 208); dmin[r] = 0;
                sc[r] = (uint8_t)((int)(int8_t)blk[192 + s] + 128); m[r] = 0;
            }
        }
        return 0;
    }
    return -1;
}

/* ----------------------------------------------------------- thread helper */

typedef void (*orc_range_fn)(void *ctx, int lo, int hi);

/* Rows over a persistent OpenMP team (the reference spreads rows over its
 * worker pool, engine/nn/jit.go:1019-1080, engine/sched/pool.go:609-641). */
static void orc_parallel(orc_range_fn fn, void *ctx, int n, int nthreads) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads > n) nthreads = n > 0 ? n : 1;
    if (nthreads == 1) { fn(ctx, 0, n); return; }
#pragma omp parallel num_threads(nthreads)
    {
        int nt = omp_get_num_threads(), i = omp_get_thread_num();
        int lo = (int)((long long)n * i / nt), hi = (int)((long long)n * (i + 1) / nt);
        if (hi > lo) fn(ctx, lo, hi);
    }
}

/* --------------------------------------------------------- float oracles */

static size_t row_bytes(uint32_t t, int k) { return (size_t)(k / orc_block_elems(t)) * (size_t)orc_block_bytes(t); }

/* internal/oracle/oracle.go:23-61 (MatVec): Dequant32 row + Neumaier-
 * compensated f32 dot. volatile pins every step to f32 (no x87/FMA fusing). */
ORC_API int orc_matvec(float *out, uint32_t t, const uint8_t *w, const float *x, int nrows, int k) {
    int be = orc_block_elems(t);
    if (!be || k % be) return -1;
    size_t rb = row_bytes(t, k);
    float *row = malloc(sizeof(float) * (size_t)k);
    for (int r = 0; r < nrows; r++) {
        orc_dequant_f32(t, w + (size_t)r * rb, (size_t)k, row);
        volatile float sum = 0, comp = 0;
        for (int i = 0; i < k; i++) {
            volatile float p = row[i] * x[i];
            volatile float tt = sum + p;
            if (fabsf(sum) >= fabsf(p)) { volatile float a = sum - tt; volatile float b = a + p; comp = comp + b; }
            else { volatile float a = p - tt; volatile float b = a + sum; comp = comp + b; }
            sum = tt;
        }
        out[r] = sum + comp;
    }
    free(row);
    return 0;
}

/* The f64 twin the reference's tests evaluate beside every kernel
 * (jit/gpu/backend/mmavolta_test.go:160-185): f64 dot of Dequant32(W) and x.
 * out is [ntok][nrows] (token-major, engine/nn/matmul.go:20-27); x is
 * [ntok][k] f32. */
struct mm64 { double *out; uint32_t t; const uint8_t *w; const float *x; int nrows, k, ntok; };
static void mm64_rows(void *p, int lo, int hi) {
    struct mm64 *a = p;
    size_t rb = row_bytes(a->t, a->k);
    float *row = malloc(sizeof(float) * (size_t)a->k);
    for (int r = lo; r < hi; r++) {
        orc_dequant_f32(a->t, a->w + (size_t)r * rb, (size_t)a->k, row);
        for (int tk = 0; tk < a->ntok; tk++) {
            const float *x = a->x + (size_t)tk * a->k;
            double s = 0;
            for (int i = 0; i < a->k; i++) s += (double)row[i] * (double)x[i];
            a->out[(size_t)tk * a->nrows + r] = s;
        }
    }
    free(row);
}
ORC_API int orc_matmul_f64(double *out, uint32_t t, const uint8_t *w, const float *x,
                           int nrows, int k, int ntok, int nthreads) {
    int be = orc_block_elems(t);
    if (!be || k % be) return -1;
    struct mm64 a = {out, t, w, x, nrows, k, ntok};
    orc_parallel(mm64_rows, &a, nrows, nthreads);
    return 0;
}

/* ------------------------------------------- int8 activations (CPU JIT twin) */

/* internal/oracle/quantize.go:80-119 (QuantizeQ8Window). n elements, window
 * 32 or 256. pairs[2b] = d, pairs[2b+1] = -sum(q)*biasC/8 per 32-block.
 * math.Round is round-half-away-from-zero == C round(). */
ORC_API void orc_quantize_q8_window(int8_t *dst, float *pairs, const float *x, int n,
                                    double biasC, int window) {
    int per = window / 32; if (per < 1) per = 1;
    int nb = n / 32;
    for (int b = 0; b < nb; b++) {
        int off = b * 32;
        int w0 = (b / per) * per * 32, w1 = w0 + per * 32;
        if (w1 > n) w1 = n;
        uint32_t amaxBits = 0;
        for (int i = w0; i < w1; i++) {
            uint32_t u; memcpy(&u, &x[i], 4); u &= 0x7fffffffu;
            if (u > amaxBits) amaxBits = u;
        }
        float amax; memcpy(&amax, &amaxBits, 4);
        volatile float d = amax / 127.0f;
        volatile float inv = 0;
        if (d != 0) inv = 1.0f / d;
        int sum = 0;
        for (int i = 0; i < 32; i++) {
            volatile float vi = x[off + i] * inv;
            int q = (int)round((double)vi);
            dst[off + i] = (int8_t)q;
            sum += q;
        }
        pairs[2 * b] = d;
        pairs[2 * b + 1] = (float)(-(double)sum * biasC / 8.0);
    }
}

/* jit/cpu/matvec.go:78-105 (BiasC) for this path's formats. MXFP4's is the
 * biased code table's +12 (jit/gpu/kernels/matvec.go:168-177). */
ORC_API double orc_bias_c(uint32_t t) {
    switch (t) { case ORC_Q4_K: return 1; case ORC_Q8_0: return 128; case ORC_MXFP4: return 12; }
    return 0;
}

/* 32 unsigned weight bytes x 32 int8 activations -> 8 int32 lane sums: what one
 * VPDPBUSD produces (jit/cpu/matvec.go:725-752). Scalar arm. */
static inline void dot32_lanes_scalar(const uint8_t *u, const int8_t *a, int32_t lanes[8]) {
    for (int l = 0; l < 8; l++) {
        int32_t s = 0;
        for (int i = 0; i < 4; i++) s += (int32_t)u[4 * l + i] * (int32_t)a[4 * l + i];
        lanes[l] = s;
    }
}

#if defined(__x86_64__)
__attribute__((target("avx2")))
static inline __m256i dot32_avx2(__m256i u, __m256i a) {
    /* maddubs saturates at int16: 2*255*127 > 32767 only if u > 129; the
     * callers below keep u <= 255 only for Q8_0, whose arm splits the bytes. */
    __m256i p = _mm256_maddubs_epi16(u, a);
    return _mm256_madd_epi16(p, _mm256_set1_epi16(1));
}
#endif

struct mvi8 {
    float *out; uint32_t t; const uint8_t *w; const int8_t *qa; const float *pairs;
    int nrows, k, ntok; int use_avx2;
};

/* One row of the CPU JIT's arithmetic (jit/cpu/matvec.go:580-777 for Q4_K;
 * its own gate states the quantity: sum_b d_a[b] * sum_i w[32b+i]*q[32b+i],
 * jit/cpu/matvec_test.go:117-130). Eight f32 lane accumulators, horizontal sum
 * once per row, the bias term entering as pair = -sum(q)*biasC/8 per lane. */
static float row_int8_scalar(uint32_t t, const uint8_t *row, const int8_t *qa, const float *pairs, int k) {
    float acc[8] = {0};
    int32_t lanes[8];
    uint8_t u[32];
    if (t == ORC_Q4_K) {
        for (int sb = 0; sb < k / 256; sb++) {
            const uint8_t *blk = row + (size_t)sb * 144;
            float d = half_to_f32(le16(blk)), dmin = half_to_f32(le16(blk + 2));
            for (int g = 0; g < 8; g++) {
                uint8_t sc, m; scale_min_k4(g, blk + 4, &sc, &m);
                int b = sb * 8 + g;
                float dx = pairs[2 * b], pair = pairs[2 * b + 1];
                volatile float S0 = (float)sc * d; volatile float S = S0 * dx;
                volatile float M0 = (float)(8 * m) * dmin; volatile float M = M0 * dx;
                const uint8_t *grp = blk + 16 + (g / 2) * 32;
                for (int l = 0; l < 32; l++) u[l] = (g & 1) ? (grp[l] >> 4) : (grp[l] & 0xF);
                dot32_lanes_scalar(u, qa + b * 32, lanes);
                acc[0] += M * pair; /* broadcast over 8 lanes then summed == 8*M*pair/8 */
                for (int l = 0; l < 8; l++) acc[l] += S * (float)lanes[l];
            }
        }
        /* acc[0] holds 1x the min term where the JIT holds it in 8 lanes of 1/8:
         * M carries the factor 8 and pair the 1/8, so one lane's product is the
         * whole term. */
    } else if (t == ORC_Q8_0) {
        for (int b = 0; b < k / 32; b++) {
            const uint8_t *blk = row + (size_t)b * 34;
            float d = half_to_f32(le16(blk));
            float dx = pairs[2 * b], pair = pairs[2 * b + 1];
            volatile float S = d * dx;
            for (int l = 0; l < 32; l++) u[l] = blk[2 + l] ^ 0x80;
            dot32_lanes_scalar(u, qa + b * 32, lanes);
            for (int l = 0; l < 8; l++) acc[l] += S * ((float)lanes[l] + pair);
        }
    } else if (t == ORC_MXFP4) {
        for (int b = 0; b < k / 32; b++) {
            const uint8_t *blk = row + (size_t)b * 17;
            float d = ldexpf(1.0f, (int)blk[0] - 128);
            float dx = pairs[2 * b], pair = pairs[2 * b + 1];
            volatile float S = d * dx;
            for (int l = 0; l < 16; l++) {
                u[l] = (uint8_t)(k_mxfp4[blk[1 + l] & 0xF] + 12);
                u[l + 16] = (uint8_t)(k_mxfp4[blk[1 + l] >> 4] + 12);
            }
            dot32_lanes_scalar(u, qa + b * 32, lanes);
            for (int l = 0; l < 8; l++) acc[l] += S * ((float)lanes[l] + pair);
        }
    }
    float s = 0;
    for (int l = 0; l < 8; l++) s += acc[l];
    return s;
}

#if defined(__x86_64__)
__attribute__((target("avx2,fma")))
static float hsum8(__m256 v) {
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    lo = _mm_add_ps(lo, hi);
    lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
    lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
    return _mm_cvtss_f32(lo);
}

__attribute__((target("avx2,fma")))
static float row_int8_avx2(uint32_t t, const uint8_t *row, const int8_t *qa, const float *pairs, int k) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    const __m256i mask4 = _mm256_set1_epi8(0x0F);
    if (t == ORC_Q4_K) {
        for (int sb = 0; sb < k / 256; sb++) {
            const uint8_t *blk = row + (size_t)sb * 144;
            float d = half_to_f32(le16(blk)), dmin = half_to_f32(le16(blk + 2));
            for (int j = 0; j < 4; j++) {
                __m256i qs = _mm256_loadu_si256((const __m256i *)(blk + 16 + j * 32));
                __m256i lo = _mm256_and_si256(qs, mask4);
                __m256i hi = _mm256_and_si256(_mm256_srli_epi16(qs, 4), mask4);
                uint8_t sc0, m0, sc1, m1;
                scale_min_k4(2 * j, blk + 4, &sc0, &m0);
                scale_min_k4(2 * j + 1, blk + 4, &sc1, &m1);
                int b = sb * 8 + 2 * j;
                float dx0 = pairs[2 * b], p0 = pairs[2 * b + 1];
                float dx1 = pairs[2 * b + 2], p1 = pairs[2 * b + 3];
                __m256i a0 = _mm256_loadu_si256((const __m256i *)(qa + b * 32));
                __m256i a1 = _mm256_loadu_si256((const __m256i *)(qa + b * 32 + 32));
                __m256 f0 = _mm256_cvtepi32_ps(dot32_avx2(lo, a0));
                __m256 f1 = _mm256_cvtepi32_ps(dot32_avx2(hi, a1));
                float S0 = (float)sc0 * d * dx0, S1 = (float)sc1 * d * dx1;
                float M0 = (float)m0 * dmin * dx0, M1 = (float)m1 * dmin * dx1; /* 8m * pair/8 folded */
                acc0 = _mm256_fmadd_ps(_mm256_set1_ps(S0), f0, acc0);
                acc1 = _mm256_fmadd_ps(_mm256_set1_ps(S1), f1, acc1);
                acc0 = _mm256_fmadd_ps(_mm256_set1_ps(M0), _mm256_set1_ps(p0), acc0);
                acc1 = _mm256_fmadd_ps(_mm256_set1_ps(M1), _mm256_set1_ps(p1), acc1);
            }
        }
    } else if (t == ORC_Q8_0) {
        /* u = q ^ 0x80 can reach 255, where maddubs would saturate: split the
         * byte into its low 7 bits and its top bit so each product stays small. */
        const __m256i m7 = _mm256_set1_epi8(0x7F), top = _mm256_set1_epi8((char)0x80);
        for (int b = 0; b < k / 32; b++) {
            const uint8_t *blk = row + (size_t)b * 34;
            float d = half_to_f32(le16(blk));
            float dx = pairs[2 * b], pair = pairs[2 * b + 1];
            __m256i q = _mm256_loadu_si256((const __m256i *)(blk + 2));
            __m256i u = _mm256_xor_si256(q, top);
            __m256i a = _mm256_loadu_si256((const __m256i *)(qa + b * 32));
            __m256i s = _mm256_add_epi32(dot32_avx2(_mm256_and_si256(u, m7), a),
                                         dot32_avx2(_mm256_and_si256(u, top), a));
            __m256 f = _mm256_add_ps(_mm256_cvtepi32_ps(s), _mm256_set1_ps(pair));
            acc0 = _mm256_fmadd_ps(_mm256_set1_ps(d * dx), f, acc0);
        }
    } else {
        return row_int8_scalar(t, row, qa, pairs, k);
    }
    return hsum8(_mm256_add_ps(acc0, acc1));
}
#endif

static void mvi8_rows(void *p, int lo, int hi) {
    struct mvi8 *a = p;
    size_t rb = row_bytes(a->t, a->k);
    int nb = a->k / 32;
    for (int r = lo; r < hi; r++) {
        const uint8_t *row = a->w + (size_t)r * rb;
        for (int tk = 0; tk < a->ntok; tk++) {
            const int8_t *qa = a->qa + (size_t)tk * a->k;
            const float *pairs = a->pairs + (size_t)tk * 2 * nb;
            float v;
#if defined(__x86_64__)
            if (a->use_avx2) v = row_int8_avx2(a->t, row, qa, pairs, a->k); else
#endif
            v = row_int8_scalar(a->t, row, qa, pairs, a->k);
            a->out[(size_t)tk * a->nrows + r] = v;
        }
    }
}

/* Which SIMD arm orc_matmul_int8 will take on this host: 0 scalar, 1 AVX2+FMA. */
ORC_API int orc_simd_level(void) {
#if defined(__x86_64__)
    __builtin_cpu_init();
    if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 1;
#endif
    return 0;
}

/* The reference CPU path, restated: engine/nn/jit.go:928-1081 (matVec:
 * quantize x once, rows over the pool) and engine/nn/matmul.go:27-189 (MatMul:
 * same arithmetic per token, out token-major). x [ntok][k] f32, out
 * [ntok][nrows] f32. window = 32, or 256 when every matvec type of the model
 * is a k-quant (jit/cpu/matvec.go:46-62). simd: -1 auto, 0 scalar, 1 AVX2. */
ORC_API int orc_matmul_int8(float *out, uint32_t t, const uint8_t *w, const float *x, int nrows,
                            int k, int ntok, int window, int nthreads, int simd) {
    int be = orc_block_elems(t);
    if (!be || k % be || k % 32) return -1;
    if (t != ORC_Q4_K && t != ORC_Q8_0 && t != ORC_MXFP4) return -1;
    int nb = k / 32;
    int8_t *qa = malloc((size_t)ntok * (size_t)k);
    float *pairs = malloc(sizeof(float) * 2 * (size_t)nb * (size_t)ntok);
    double bc = orc_bias_c(t);
    for (int tk = 0; tk < ntok; tk++)
        orc_quantize_q8_window(qa + (size_t)tk * k, pairs + (size_t)tk * 2 * nb, x + (size_t)tk * k, k, bc, window);
    struct mvi8 a = {out, t, w, qa, pairs, nrows, k, ntok, simd < 0 ? orc_simd_level() : simd};
    orc_parallel(mvi8_rows, &a, nrows, nthreads);
    free(qa); free(pairs);
    return 0;
}

/* ----------------------------------------------------------------- router */

/* engine/nn/moetopk.go:362 (Softmax32JIT) is a generated kernel with a
 * polynomial exp; its own gate compares it with libm under a tolerance
 * (internal/oracle/moe.go:361-370), so this is libm in f64, narrowed once. */
ORC_API void orc_softmax(float *sc, const float *logits, int n) {
    double mx = -INFINITY, s = 0;
    for (int i = 0; i < n; i++) if (logits[i] > mx) mx = logits[i];
    for (int i = 0; i < n; i++) s += exp((double)logits[i] - mx);
    for (int i = 0; i < n; i++) sc[i] = (float)(exp((double)logits[i] - mx) / s);
}

/* internal/oracle/moe.go:329-359 (moeLexTopK): k largest, descending, lowest
 * index wins a tie, NaN never eligible. */
static int lex_topk(const float *v, int n, int k, int *out) {
    int cnt = 0, prevIdx = -1; float prevVal = 0;
    for (int i = 0; i < k; i++) {
        int best = -1; float bestVal = 0;
        for (int e = 0; e < n; e++) {
            float x = v[e];
            if (x != x) continue;
            if (i > 0 && !(x < prevVal || (x == prevVal && e > prevIdx))) continue;
            if (best < 0 || x > bestVal) { best = e; bestVal = x; }
        }
        if (best < 0) break;
        out[cnt++] = best; prevVal = bestVal; prevIdx = best;
    }
    return cnt;
}

/* internal/oracle/moe.go:197-327 (MoERouter), ungrouped (NGroup <= 1), over
 * already-gated scores. bias (selection only) and exp_scale may be NULL.
 * Outputs: sel/wt in selection order, ord/owt ascending id, *sum the divisor. */
ORC_API int orc_moe_router(const float *scores, int n, int k, int norm, float scale,
                           const float *bias, const float *exp_scale,
                           int32_t *sel, int32_t *ord, float *wt, float *owt, float *sum_out) {
    if (k <= 0 || n <= 0 || k > n) return -1;
    if (scale == 0) scale = 1;
    float *bi = malloc(sizeof(float) * (size_t)n);
    for (int e = 0; e < n; e++) { volatile float b = bias ? scores[e] + bias[e] : scores[e]; bi[e] = b; }
    int *selI = malloc(sizeof(int) * (size_t)k), *ordI = malloc(sizeof(int) * (size_t)k);
    int got = lex_topk(bi, n, k, selI);
    for (int i = 0; i < got; i++) ordI[i] = selI[i];
    for (int i = 1; i < got; i++)
        for (int j = i; j > 0 && ordI[j] < ordI[j - 1]; j--) { int tmp = ordI[j]; ordI[j] = ordI[j - 1]; ordI[j - 1] = tmp; }
    float *w = malloc(sizeof(float) * (size_t)k);
    for (int i = 0; i < got; i++) w[i] = scores[selI[i]];
    volatile float sum = 1;
    if (norm) {
        sum = 0;
        for (int i = 0; i < got; i++) sum = sum + w[i];   /* selection order, one add at a time */
        sum = sum + 1e-20f;                               /* moeSumFloor */
    }
    for (int i = 0; i < got; i++) {
        volatile float v = w[i] / sum;
        if (scale != 1) v = v * scale;
        if (exp_scale) v = v * exp_scale[selI[i]];
        w[i] = v;
    }
    for (int i = 0; i < got; i++) { sel[i] = selI[i]; wt[i] = w[i]; }
    for (int i = 0; i < got; i++) {
        ord[i] = ordI[i];
        for (int j = 0; j < got; j++) if (selI[j] == ordI[i]) owt[i] = w[j];
    }
    *sum_out = sum;
    free(bi); free(selI); free(ordI); free(w);
    return got;
}

/* internal/oracle/oracle.go:128-137 and jit/gpu/kernels/actkind.go:13-39. */
ORC_API double orc_silu(double x) { return x / (1 + exp(-x)); }
ORC_API double orc_swiglu_oai(double gate, double up) {
    double x = fmin(gate, 7), y = fmax(fmin(up, 7), -7);
    return x / (1 + exp(-1.702 * x)) * (y + 1);
}

/* The mixture layer, float oracle. engine/model/moe.go:502-760 (moeBatch /
 * moeBatchExpert): every row is routed; then experts ascending, each over the
 * rows that chose it (rows ascending): G = gate.x, U = up.x, [+bias],
 * A = act(G,U), Y = down.A, [+bias], out[row] += w * Y. Accumulation order per
 * output element is therefore ascending expert id (engine/model/moe.go:127-134).
 *
 * h [ntok][hidden] f32; gate/up banks [E][ffn][hidden/32*17]; down bank
 * [E][hidden][ffn/32*17] (MXFP4) or any supported type `t`; sel/wt
 * [ntok][top_k] in selection order from orc_moe_router. out [ntok][hidden] is
 * ADDED to (the caller passes the residual or zeros). Dots are f64, the
 * intermediate act is kept in f64 -> f32 once (the reference keeps f32).
 * act_kind 0 = SiLU gate, 1 = SwiGLU-OAI. Biases may be NULL. */
struct moe_job {
    float *out; const float *h; uint32_t t; const uint8_t *gate, *up, *down;
    const float *bgate, *bup, *bdown; const int32_t *sel; const float *wt;
    int ntok, n_expert, top_k, hidden, ffn, act_kind;
    int e; int m; const int *rows; const float *w; float *A; /* per-expert stage */
};
static void moe_gu_rows(void *p, int lo, int hi) {
    struct moe_job *a = p;
    size_t rb = row_bytes(a->t, a->hidden);
    float *wg = malloc(sizeof(float) * (size_t)a->hidden), *wu = malloc(sizeof(float) * (size_t)a->hidden);
    for (int f = lo; f < hi; f++) {
        orc_dequant_f32(a->t, a->gate + ((size_t)a->e * a->ffn + f) * rb, (size_t)a->hidden, wg);
        orc_dequant_f32(a->t, a->up + ((size_t)a->e * a->ffn + f) * rb, (size_t)a->hidden, wu);
        for (int r = 0; r < a->m; r++) {
            const float *x = a->h + (size_t)a->rows[r] * a->hidden;
            double g = 0, u = 0;
            for (int i = 0; i < a->hidden; i++) { g += (double)wg[i] * x[i]; u += (double)wu[i] * x[i]; }
            float gf = (float)g, uf = (float)u;
            if (a->bgate) gf += a->bgate[(size_t)a->e * a->ffn + f];
            if (a->bup) uf += a->bup[(size_t)a->e * a->ffn + f];
            double act = a->act_kind == 1 ? orc_swiglu_oai(gf, uf) : orc_silu(gf) * uf;
            a->A[(size_t)r * a->ffn + f] = (float)act;
        }
    }
    free(wg); free(wu);
}
static void moe_down_rows(void *p, int lo, int hi) {
    struct moe_job *a = p;
    size_t rb = row_bytes(a->t, a->ffn);
    float *wd = malloc(sizeof(float) * (size_t)a->ffn);
    for (int d = lo; d < hi; d++) {
        orc_dequant_f32(a->t, a->down + ((size_t)a->e * a->hidden + d) * rb, (size_t)a->ffn, wd);
        for (int r = 0; r < a->m; r++) {
            const float *x = a->A + (size_t)r * a->ffn;
            double y = 0;
            for (int i = 0; i < a->ffn; i++) y += (double)wd[i] * x[i];
            float yf = (float)y;
            if (a->bdown) yf += a->bdown[(size_t)a->e * a->hidden + d];
            volatile float contrib = a->w[r] * yf;
            volatile float acc = a->out[(size_t)a->rows[r] * a->hidden + d] + contrib;
            a->out[(size_t)a->rows[r] * a->hidden + d] = acc;
        }
    }
    free(wd);
}
ORC_API int orc_moe_layer(float *out, const float *h, uint32_t t, const uint8_t *gate, const uint8_t *up,
                          const uint8_t *down, const float *bgate, const float *bup, const float *bdown,
                          const int32_t *sel, const float *wt, int ntok, int n_expert, int top_k,
                          int hidden, int ffn, int act_kind, int nthreads) {
    int be = orc_block_elems(t);
    if (!be || hidden % be || ffn % be) return -1;
    struct moe_job a = {out, h, t, gate, up, down, bgate, bup, bdown, sel, wt,
                        ntok, n_expert, top_k, hidden, ffn, act_kind, 0, 0, NULL, NULL, NULL};
    int *rows = malloc(sizeof(int) * (size_t)ntok);
    float *w = malloc(sizeof(float) * (size_t)ntok);
    float *A = malloc(sizeof(float) * (size_t)ntok * (size_t)ffn);
    for (int e = 0; e < n_expert; e++) {
        int m = 0;
        for (int i = 0; i < ntok; i++)
            for (int j = 0; j < top_k; j++)
                if (sel[i * top_k + j] == e) { rows[m] = i; w[m] = wt[i * top_k + j]; m++; break; }
        if (!m) continue;
        a.e = e; a.m = m; a.rows = rows; a.w = w; a.A = A;
        orc_parallel(moe_gu_rows, &a, ffn, nthreads);
        orc_parallel(moe_down_rows, &a, hidden, nthreads);
    }
    free(rows); free(w); free(A);
    return 0;
}

/* ------------------------------------------------ container-packed planes */

/* kernels.PackWeights (jit/gpu/kernels/pack.go:27-239) for the formats of this path: the device / container
 * layout [sub-block][word][row]. qs, d, sc are caller-zeroed u32 arrays of orc_packed_words() lengths; `stride` is
 * the row count of the whole buffer and `row0` where this weight starts in it (engine/nn/device.go:62-80).
 *   payload   packSub (pack.go:186-224): sub-block si of row r is words (si*pw + w)*stride + r, pw = 4 (4-bit: byte j
 *             holds element j in its low and j + 16 in its high nibble) or 8 (Q8_0: the signed bytes in order)
 *   d plane   DIndex / DSlots (pack.go:545-575): Q4_K one word per (super-block, row) = d | dmin << 16; Q8_0 two
 *             rows a word (f16 each); MXFP4 four rows a word (the stored exponent byte e - 1 each)
 *   sc plane  Q4_K only: the 96-bit stream of sixteen 6-bit fields, scale then minimum per sub-block
 *             (scstream.go:26-62), three words per (super-block, row) */
static int orc_dslots(uint32_t t) { return t == ORC_MXFP4 ? 4 : (t == ORC_Q8_0 ? 2 : 1); }
ORC_API int orc_packed_words(uint32_t t, int stride, int k, size_t *nqs, size_t *nd, size_t *nsc) {
    if (t != ORC_Q4_K && t != ORC_Q8_0 && t != ORC_MXFP4) return -1;
    if (k <= 0 || k % orc_block_elems(t)) return -2;
    const int nsub = k / 32, pw = t == ORC_Q8_0 ? 8 : 4, ds = orc_dslots(t);
    const int nsuper = t == ORC_Q4_K ? k / 256 : nsub;
    *nqs = (size_t)stride * nsub * pw;
    *nd = (size_t)nsuper * ((stride + ds - 1) / ds);
    *nsc = t == ORC_Q4_K ? (size_t)nsuper * 3 * stride : 0;
    return 0;
}
static void sc_put(uint32_t *w3, int sub, int min, uint8_t v) {
    const int f = 2 * sub + (min ? 1 : 0), w = f * 6 / 32, b = f * 6 % 32, hi = b > 26 ? b - 26 : 0;
    w3[w] |= (uint32_t)(v & 63) << b;
    if (hi > 0) w3[w + 1] |= (uint32_t)(v & 63) >> (6 - hi);
}
ORC_API int orc_pack_weights(uint32_t t, const uint8_t *src, int nrows, int k, int row0, int stride,
                             uint32_t *qs, uint32_t *d, uint32_t *sc) {
    size_t nq, nd, ns;
    if (orc_packed_words(t, stride, k, &nq, &nd, &ns)) return -1;
    if (row0 < 0 || row0 + nrows > stride) return -2;
    const int be = orc_block_elems(t), bb = orc_block_bytes(t), per = be / 32, nblk = k / be;
    const int pw = t == ORC_Q8_0 ? 8 : 4, ds = orc_dslots(t);
    const size_t nsub_blocks = (size_t)nrows * nblk;
    int8_t *q = malloc(nsub_blocks * be);
    uint16_t *db = malloc(nsub_blocks * per * 2), *dm = malloc(nsub_blocks * per * 2);
    uint8_t *scv = malloc(nsub_blocks * per), *mv = malloc(nsub_blocks * per);
    orc_unpack(t, src, nsub_blocks, q, db, dm, scv, mv);         /* extract, one record per 32 elements */
    for (int r = 0; r < nrows; r++) {
        const int R = row0 + r;
        for (int si = 0; si < k / 32; si++) {
            const size_t rec = (size_t)r * (k / 32) + si;
            const int8_t *qq = q + rec * 32;
            uint8_t out[32] = {0};
            if (pw == 4) for (int l = 0; l < 32; l++) out[l % 16] |= (uint8_t)((qq[l] & 15) << (4 * (l / 16)));
            else for (int l = 0; l < 32; l++) out[l] = (uint8_t)qq[l];
            for (int w = 0; w < pw; w++)
                qs[((size_t)si * pw + w) * stride + R] = (uint32_t)out[4 * w] | (uint32_t)out[4 * w + 1] << 8 |
                                                         (uint32_t)out[4 * w + 2] << 16 | (uint32_t)out[4 * w + 3] << 24;
            const int sup = t == ORC_Q4_K ? si / 8 : si;
            if (ds == 1) d[(size_t)sup * stride + R] |= (uint32_t)db[rec] | (uint32_t)dm[rec] << 16;
            else if (ds == 2) d[(size_t)sup * ((stride + 1) / 2) + R / 2] |= (uint32_t)db[rec] << (16 * (R % 2));
            else d[(size_t)sup * ((stride + 3) / 4) + R / 4] |= (uint32_t)(db[rec] & 0xFF) << (8 * (R % 4));
            if (t == ORC_Q4_K) {
                uint32_t w3[3] = {0, 0, 0};
                sc_put(w3, si % 8, 0, scv[rec]);
                sc_put(w3, si % 8, 1, mv[rec]);
                for (int w = 0; w < 3; w++) sc[((size_t)sup * 3 + w) * stride + R] |= w3[w];
            }
        }
    }
    free(q); free(db); free(dm); free(scv); free(mv);
    return 0;
}
