// The prepared activation operand of the Q4_K decode kernel, shared by the kernels that produce it:
// the prep kernel in front of a matvec, the decode kernel's fused form, and the decode-step neighbours
// (norm, attention, SiLU*up), which write it directly so that no prep launch sits between them and the
// matvec that consumes their output.
#pragma once
#include <cstdint>

// Prepared activation operand, per (token, super-block): Q4K_XP_SB_BYTES bytes.
//   [0, 576)    4 groups x 144 B (128 used; 144 staggers the shared-memory banks):
//               slot (hl, cp) at hl*64 + cp*16 = {digit1[8], digit2[8]} for the 8
//               activations that code words 2cp and 2cp+1 of nibble half hl multiply
//   [576, 640)  4 x {int32 S[2t], int32 S[2t+1], float 1/s, 0}
// followed, after all super-blocks of all tokens, by 128 zero bytes (the B fragment
// of the lanes that feed a zero column).
#define Q4K_XP_GROUP_BYTES 144
#define Q4K_XP_AUX_OFS 576
#define Q4K_XP_SB_BYTES 640
#define Q4K_XP_ZERO_BYTES 128
// The activation operand of one super-block, by one warp: lane l holds activations 4l..4l+3 (v0) and
// 128+4l..128+4l+3 (v1) of the super-block; out points at its Q4K_XP_SB_BYTES (global scratch or
// shared memory).
__device__ __forceinline__ void q4k_prep_sb_vals(const float4 v0, const float4 v1, uint8_t *out, int lane) {
    float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                       fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const bool live = amax > 0.f && amax < __int_as_float(0x7f800000);
    const float scale = live ? 32512.f / amax : 0.f;
    const float inv_scale = live ? amax / 32512.f : 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float4 v = h ? v1 : v0;
        const int q = lane + 32 * h;             // quad index: element 4q = 64 t + 32 hl + 4 c
        const int t = q >> 4, hl = (q >> 3) & 1, c = q & 7;
        const float xs[4] = {v.x * scale, v.y * scale, v.z * scale, v.w * scale};
        uint32_t d1 = 0, d2 = 0;
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float q1f = rintf(xs[j] * (1.f / 256.f));
            const int q1 = (int)q1f;
            int q2 = (int)rintf(xs[j] - 256.f * q1f);
            q2 = max(-127, min(127, q2));
            d1 |= (uint32_t)(q1 & 0xFF) << (8 * j);
            d2 |= (uint32_t)(q2 & 0xFF) << (8 * j);
            sum += 256 * q1 + q2;
        }
        uint8_t *slot = out + t * Q4K_XP_GROUP_BYTES + hl * 64 + (c >> 1) * 16 + (c & 1) * 4;
        *reinterpret_cast<uint32_t *>(slot) = d1;
        *reinterpret_cast<uint32_t *>(slot + 8) = d2;
        // the 8 lanes sharing (t, hl) hold one 32-element sub-block
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        const int other = __shfl_xor_sync(0xffffffffu, sum, 8);  // the other nibble half
        if ((q & 15) == 0)
            *reinterpret_cast<int4 *>(out + Q4K_XP_AUX_OFS + t * 16) =
                make_int4(sum, other, __float_as_int(inv_scale), 0);
    }
}


__device__ __forceinline__ void q4k_prep_sb(const float4 *__restrict__ x4, uint8_t *out, int lane) {
    q4k_prep_sb_vals(__ldg(x4 + lane), __ldg(x4 + 32 + lane), out, lane);
}
