// Element accessors of the ggml formats that stay as raw blocks on the device (Q4_0, Q5_0, Q5_1, Q5_K, Q6_K):
// where element e of a block keeps its integer code, which scale fields go with it, and the weight's value computed
// exactly as quant.Dequant32 computes it (format/quant/dequant.go:85-146, 399-470). Shared by the host unpack, the
// resident unpack kernel and the one-warp-per-row matvec kernel, so all three read a block the same way.
#pragma once
#include <cstdint>

#include "jl_internal.cuh"

__host__ __device__ static inline uint16_t jl_raw_le16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
__host__ __device__ static inline uint32_t jl_raw_le32(const uint8_t *p) {
    return (uint32_t)p[0] | (uint32_t)p[1] << 8 | (uint32_t)p[2] << 16 | (uint32_t)p[3] << 24;
}
__host__ __device__ static inline void jl_raw_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) { *sc = q[j] & 63; *m = q[j + 4] & 63; }
    else { *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

// The unsigned integer code of element e (0 .. block elements - 1) as the reference's extract reports it
// (jit/gpu/kernels/pack.go:252-386): Q4_0 0..15, Q5_x and Q5_K 0..31, Q6_K 0..63.
__host__ __device__ static inline int jl_raw_code(uint32_t t, const uint8_t *blk, int e) {
    switch (t) {
    case JL_TYPE_Q4_0: {
        const uint8_t b = blk[2 + (e & 15)];
        return e < 16 ? (b & 0xF) : (b >> 4);
    }
    case JL_TYPE_Q5_0: case JL_TYPE_Q5_1: {
        const int hdr = t == JL_TYPE_Q5_1 ? 4 : 2;
        const uint8_t b = blk[hdr + 4 + (e & 15)];
        const uint32_t qh = jl_raw_le32(blk + hdr);
        return (e < 16 ? (b & 0xF) : (b >> 4)) + (((qh >> e) & 1u) ? 16 : 0);   // element e takes bit e of qh
    }
    case JL_TYPE_Q5_K: {
        const int s = e >> 5, l = e & 31;                     // sub-block s: low nibbles when s is even
        const uint8_t b = blk[48 + (s >> 1) * 32 + l];
        return ((s & 1) ? (b >> 4) : (b & 0xF)) + (((blk[16 + l] >> s) & 1) ? 16 : 0);
    }
    case JL_TYPE_Q6_K: {
        const int n = e >> 7, j = (e >> 5) & 3, l = e & 31;   // half n, 32-run j of the half, position l
        const uint8_t b = blk[n * 64 + l + (j & 1) * 32];
        const int nib = j >= 2 ? (b >> 4) : (b & 0xF);
        return nib | (((blk[128 + n * 32 + l] >> (2 * j)) & 3) << 4);
    }
    }
    return 0;
}

// The scale fields of record s (Q6_K: the s-th 16 elements; else the s-th 32 elements) in the integer view.
__host__ __device__ static inline void jl_raw_record(uint32_t t, const uint8_t *blk, int s, uint16_t *d, uint16_t *dmin, uint8_t *sc,
                                                     uint8_t *m) {
    *d = 0; *dmin = 0; *sc = 0; *m = 0;
    switch (t) {
    case JL_TYPE_Q4_0: case JL_TYPE_Q5_0: *d = jl_raw_le16(blk); break;
    case JL_TYPE_Q5_1: *d = jl_raw_le16(blk); *dmin = (uint16_t)(jl_raw_le16(blk + 2) ^ 0x8000); break;
    case JL_TYPE_Q5_K: *d = jl_raw_le16(blk); *dmin = jl_raw_le16(blk + 2); jl_raw_scale_min_k4(s, blk + 4, sc, m); break;
    case JL_TYPE_Q6_K: *d = jl_raw_le16(blk + 208); *sc = (uint8_t)((int)(int8_t)blk[192 + s] + 128); break;
    }
}

#ifdef __CUDACC__
// The f32 weight of element e, rounded where quant.Dequant32 rounds.
__device__ static inline float jl_raw_weight(uint32_t t, const uint8_t *blk, int e) {
    const int q = jl_raw_code(t, blk, e);
    switch (t) {
    case JL_TYPE_Q4_0:   // (q - 8) d: exact
        return __fmul_rn((float)(q - 8), __half2float(__ushort_as_half(jl_raw_le16(blk))));
    case JL_TYPE_Q5_0:   // (q - 16) d: exact
        return __fmul_rn((float)(q - 16), __half2float(__ushort_as_half(jl_raw_le16(blk))));
    case JL_TYPE_Q5_1:   // q d + m in f64, narrowed once: one fused multiply-add gives the same f32
        return fmaf((float)q, __half2float(__ushort_as_half(jl_raw_le16(blk))), __half2float(__ushort_as_half(jl_raw_le16(blk + 2))));
    case JL_TYPE_Q5_K: {  // (d sc) q - (dmin m), every product and the difference rounded to f32
        uint8_t sc, m;
        jl_raw_scale_min_k4(e >> 5, blk + 4, &sc, &m);
        const float d = __half2float(__ushort_as_half(jl_raw_le16(blk))), dmin = __half2float(__ushort_as_half(jl_raw_le16(blk + 2)));
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
    }
    case JL_TYPE_Q6_K: {  // (d sc) (q - 32), sc the int8 scale of the element's 16-run
        const float d = __half2float(__ushort_as_half(jl_raw_le16(blk + 208)));
        const int n = e >> 7, j = (e >> 5) & 3, l = e & 31;
        const int sc = (int)(int8_t)blk[192 + n * 8 + (l >> 4) + 2 * j];
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)(q - 32));
    }
    }
    return 0.f;
}
#endif
