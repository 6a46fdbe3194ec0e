// One warp-task of the Q4_K tensor-core decode: 16 rows x one 256-element super-block against the
// prepared activation operand (q4k_prep.cuh), as a function the block kernel shares with nothing
// else's tuning: the arithmetic is the decode kernel's (gemv.cu), restated here.
//
// Lane (g, t) of the warp owns rows g and g+8 of the tile and the 32 code bytes of 64-element
// group t. The B operand is block-diagonal (column 2t carries digit 1 and column 2t+1 digit 2 of
// group t), so the eight columns of one m16n8k32 u8 x s8 accumulator collect four sub-block sums.
// sc and m enter as integers, d, dmin and 1/s in f32 (format/quant/dequant.go:360-397).
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

#include "q4k_prep.cuh"

__device__ __forceinline__ void q4k_dot_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The six 16-byte pieces of the tile one lane consumes: header + two code chunks of rows g and g+8.
struct q4k_lane_tile {
    uint4 hA, qA0, qA1, hB, qB0, qB1;
};
__device__ __forceinline__ q4k_lane_tile q4k_lane_load(const uint8_t *tile, int g, int t) {
    q4k_lane_tile r;
    r.hA = *reinterpret_cast<const uint4 *>(tile + g * 144);
    r.qA0 = *reinterpret_cast<const uint4 *>(tile + g * 144 + 16 + 32 * t);
    r.qA1 = *reinterpret_cast<const uint4 *>(tile + g * 144 + 32 + 32 * t);
    r.hB = *reinterpret_cast<const uint4 *>(tile + (g + 8) * 144);
    r.qB0 = *reinterpret_cast<const uint4 *>(tile + (g + 8) * 144 + 16 + 32 * t);
    r.qB1 = *reinterpret_cast<const uint4 *>(tile + (g + 8) * 144 + 32 + 32 * t);
    return r;
}

// xsb: the super-block's prepared operand (Q4K_XP_SB_BYTES, shared memory); zero: 128 zero bytes.
// Adds this lane's share of the two rows' dot products to accA (row g) and accB (row g + 8); the
// four t lanes of a row still have to be summed.
__device__ __forceinline__ void q4k_dot_task(const q4k_lane_tile &w, const uint8_t *xsb, const uint8_t *zero, int g, int t,
                                             float &accA, float &accB) {
    const bool bsel = ((g >> 1) == t);  // lanes that feed a non-zero B column: digit (g & 1) of group t
    const uint8_t *xf = bsel ? xsb + t * Q4K_XP_GROUP_BYTES + (g & 1) * 8 : zero;
    const int4 ax = *reinterpret_cast<const int4 *>(xsb + Q4K_XP_AUX_OFS + t * 16);
    const int sh = 8 * (2 * (t & 1));   // bit offset of this lane's scale bytes inside a header word
    const uint32_t wa[8] = {w.qA0.x, w.qA0.y, w.qA0.z, w.qA0.w, w.qA1.x, w.qA1.y, w.qA1.z, w.qA1.w};
    const uint32_t wb[8] = {w.qB0.x, w.qB0.y, w.qB0.z, w.qB0.w, w.qB1.x, w.qB1.y, w.qB1.z, w.qB1.w};
    int ce[4] = {0, 0, 0, 0}, co[4] = {0, 0, 0, 0};
    const uint32_t m4 = 0x0F0F0F0Fu, h4 = 0xF0F0F0F0u;
#pragma unroll
    for (int cp = 0; cp < 4; cp++) {
        const uint2 fe = *reinterpret_cast<const uint2 *>(xf + cp * 16);
        const uint2 fo = *reinterpret_cast<const uint2 *>(xf + 64 + cp * 16);
        const uint32_t a0 = wa[2 * cp], a2 = wa[2 * cp + 1], a1 = wb[2 * cp], a3 = wb[2 * cp + 1];
        q4k_dot_mma(ce, a0 & m4, a1 & m4, a2 & m4, a3 & m4, fe.x, fe.y);
        q4k_dot_mma(co, a0 & h4, a1 & h4, a2 & h4, a3 & h4, fo.x, fo.y);   // the high nibbles in place: 16 x the code
    }
    const float inv_scale = __int_as_float(ax.z);
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint4 &h = r ? w.hB : w.hA;
        const uint32_t a = h.y >> sh, b = h.z >> sh, c = h.w >> sh;
        uint32_t scp, mp;
        if (t < 2) { scp = a & 0x3F3Fu; mp = b & 0x3F3Fu; }
        else { scp = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u); mp = ((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u); }
        const int pe = (ce[2 * r] << 8) + ce[2 * r + 1];   // sum q (256 q1 + q2), sub-block 2t
        const int po = ((co[2 * r] << 8) + co[2 * r + 1]) >> 4;   // sub-block 2t + 1, whose codes entered as 16 q: exact
        const int dotq = (int)(scp & 0xFF) * pe + (int)(scp >> 8) * po;
        const int dotm = (int)(mp & 0xFF) * ax.x + (int)(mp >> 8) * ax.y;
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
        const float v = (dd.x * (float)dotq - dd.y * (float)dotm) * inv_scale;
        if (r) accB += v; else accA += v;
    }
}
