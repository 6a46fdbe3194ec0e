// tcgen05 / TMEM helpers and the activation-row conversion shared by the dense prefill GEMM
// (gemm_tc5.cu) and the grouped expert GEMM (moe.cu).
#pragma once

#include "jl_internal.cuh"
#include "tma.cuh"

#define TC5_M 128           // rows of one MMA (tcgen05 cta_group::1 M)
#define TC5_MS 2            // MMAs that share one activation tile: a CTA tile is 256 weight rows
#define TC5_ROWS (TC5_M * TC5_MS)
#define TC5_KB 64           // k per shared-memory stage (128 bytes of f16: one swizzle atom)
#define TC5_A_BYTES (TC5_M * TC5_KB * 2)   // one 128-row operand
#define TC5_THREADS 448     // 14 warps: 4 epilogue, producer, MMA, 8 dequant
// MMA issuers of the prefill GEMM: with 2, warp 5 issues the MMAs of the tile's first 128 rows and warp 14 those of
// the second 128 (separate accumulators, same activation stage), so one thread's barrier waits and commits run
// while the other's MMAs execute: a single issuer spends ~500 clocks per k-block outside its MMAs and the tensor
// pipe idles for them.
#define TC5_ISSUERS 2
#define TC5_GEMM_THREADS (TC5_THREADS + 32 * (TC5_ISSUERS - 1))
#define TC5_MMA2_WARP (TC5_THREADS / 32)
#define TC5_DQ_THREADS 256  // one thread per tile row

// ------------------------------------------------------------- activations

// Eight consecutive activations of a token row as f32 (k is a multiple of 8).
__device__ __forceinline__ void act_load8(const void *x, int x_dtype, size_t idx, float (&v)[8]) {
    if (x_dtype == JL_DT_F32) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(x) + idx));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(x) + idx) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + idx));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (x_dtype == JL_DT_BF16) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            } else {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
            }
        }
    }
}

// One CTA per destination row `tok`. dst rows: `split` ? (2 tok: hi, 2 tok + 1: lo) : tok. The
// source row is rowmap[tok] when a map is given (the mixture layer gathers token rows into
// expert order this way), else tok. A map entry outside [0, nsrc) reads row 0 instead (its destination row
// belongs to no expert's list and is never consumed): a stale or hostile map cannot send the load out of bounds.
static __global__ void __launch_bounds__(256)
act_to_f16_kernel(const void *__restrict__ x, int x_dtype, __half *__restrict__ dst, float *__restrict__ inv_scale,
                  int k, int split, const int *__restrict__ rowmap, int nsrc) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float wmax[8];
    const int tok = blockIdx.x, tid = threadIdx.x;
    int src = tok;
    if (rowmap) {
        src = rowmap[tok];
        if ((unsigned)src >= (unsigned)nsrc) src = 0;
    }
    const size_t base = (size_t)src * k;
    float amax = 0.f;
    for (int c = tid; c < k / 8; c += 256) {
        float v[8];
        act_load8(x, x_dtype, base + (size_t)c * 8, v);
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((tid & 31) == 0) wmax[tid >> 5] = amax;
    __syncthreads();
    amax = wmax[0];
#pragma unroll
    for (int w = 1; w < 8; w++) amax = fmaxf(amax, wmax[w]);
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
    int s = 14 - e;
    if (amax == 0.f || !(amax < __int_as_float(0x7f800000))) s = 0;
    s = max(-100, min(100, s));
    const float scale = __uint_as_float((uint32_t)(127 + s) << 23);
    if (tid == 0) inv_scale[tok] = __uint_as_float((uint32_t)(127 - s) << 23);
    __half *hi = dst + (size_t)(split ? 2 * tok : tok) * k;
    __half *lo = hi + k;
    for (int c = tid; c < k / 8; c += 256) {
        float v[8];
        act_load8(x, x_dtype, base + (size_t)c * 8, v);
        uint32_t h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float a = v[2 * i] * scale, b = v[2 * i + 1] * scale;
            const __half2 hh = __floats2half2_rn(a, b);
            const float2 back = __half22float2(hh);
            const __half2 ll = __floats2half2_rn(a - back.x, b - back.y);
            h[i] = *reinterpret_cast<const uint32_t *>(&hh);
            l[i] = *reinterpret_cast<const uint32_t *>(&ll);
        }
        *reinterpret_cast<uint4 *>(hi + (size_t)c * 8) = make_uint4(h[0], h[1], h[2], h[3]);
        if (split) *reinterpret_cast<uint4 *>(lo + (size_t)c * 8) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

// --------------------------------------------------------------- tcgen05 PTX

__device__ __forceinline__ void tc5_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc5_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One lane of the (converged) warp; and a value broadcast from lane 0, which also tells the compiler that it is the
// same in every lane.
__device__ __forceinline__ bool tc5_elect() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ int tc5_uniform(int v) { return __shfl_sync(0xffffffffu, v, 0); }
__device__ __forceinline__ void tc5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc5_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate = 0 overwrites D.
__device__ __forceinline__ void tc5_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base + i), columns c..c+31.
__device__ __forceinline__ void tc5_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc5_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc5_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc5_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, SWIZZLE_128B: rows of 128 bytes, 8-row atoms of
// 1024 bytes (stride byte offset 1024), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t tc5_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset
    d |= (uint64_t)1 << 46;                       // version
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: D f32, A and B f16, both K-major, M x N.
__host__ __device__ constexpr uint32_t tc5_idesc(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Byte i of `codes` (0x80 | q) as the float 1 + q/128: 0x3F in byte 3, the code in byte 2.
__device__ __forceinline__ float tc5_code_float(uint32_t codes, int i) {
    return __uint_as_float(__byte_perm(codes, 0x3F000000u, 0x7054 | (i << 8)));
}
// Two f32 FMAs in one instruction (fma.rn.f32x2): d = a * b + c on both halves.
__device__ __forceinline__ void tc5_fma2(float &d0, float &d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %4};\n\t"
        "mov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}

__device__ __forceinline__ uint4 ldg_nc16(const void *p) {
    uint4 v;
    // allocating in L1 on purpose: the neighbouring 16 bytes of the sector are the next load of the same thread
    // (measured: L1::no_allocate costs the prefill GEMM 24 %)
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
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

// Bounded wait that also gives up when another role of the CTA has aborted. abort_flag[0] is the CTA's abort
// word in shared memory, abort_flag[1] the wait limit in microseconds (0 = default), copied there at start-up.
__device__ __forceinline__ uint64_t tc5_limit_ns(volatile int *abort_flag) {
    const uint32_t us = (uint32_t)abort_flag[1];
    return (uint64_t)(us ? us : JL_WAIT_DEFAULT_US) * 1000ull;
}
__device__ __forceinline__ bool tc5_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t limit = tc5_limit_ns(abort_flag), t0 = jl_gtime_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (jl_gtime_ns() - t0 > limit) break;
    }
    *abort_flag = 1;
    return false;
}

// The same, for a role that is not on the critical path: backs off between polls so that it
// does not take issue slots from the dequant warps it shares a scheduler with.
__device__ __forceinline__ bool tc5_wait_relaxed(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t limit = tc5_limit_ns(abort_flag), t0 = jl_gtime_ns();
    for (uint32_t i = 0;; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(256);
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            if (jl_gtime_ns() - t0 > limit) break;
        }
    }
    *abort_flag = 1;
    return false;
}
