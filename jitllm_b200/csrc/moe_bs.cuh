// Block-scaled arm of the MXFP4 mixture layer: tcgen05.mma kind::mxf8f6f4.block_scale consumes the e2m1 codes and
// their e8m0 block scales AS THEY ARE, so no warp converts a weight. The price is on the activation side: they are
// quantised per 32 elements to e4m3 with a ue8m0 scale (the MX format the instruction takes), which the reference's
// f32-activation arithmetic does not do: this arm is reported with its own measured error and is selected only by
// jl_moe_desc.arm = JL_MOE_ARM_BLOCK_SCALED. (The reference has no counterpart: its grouped expert GEMM runs on
// mma.sync, jit/gpu/kernels/gemm70.go:123-129.)
//
// Operand layout in shared memory, K-major, 128-byte swizzle, 128 elements of K per stage:
//   A (weights)  the instruction reads 4-bit operands as 16 packed values in the low 8 bytes of every 16-byte unit.
//                The resident code plane keeps a block's 32 codes in 16 bytes, byte j = element j | element j+16 << 4;
//                the eight unpack warps copy bytes 0..7 and 8..15 of a block into two units. The K ORDER inside a
//                block is therefore 0, 16, 1, 17, ...: the activation quantiser writes its bytes in the same order
//                (a dot product does not care in which order both sides list k, and the scale blocks are untouched).
//   B (activations)  one e4m3 byte per element, by TMA.
//   scale factors  one 32-bit word per (row or token, stage) = the four block scales of the stage, in the 512-byte
//                atom [(r % 32) * 16 + (r / 32) * 4] that tcgen05.cp.32x128b.warpx4 spreads over four TMEM columns; the
//                instruction descriptor's a_sf_id / b_sf_id pick the byte (block) for each K = 32 MMA.
#pragma once
#include <cuda_fp8.h>

#include "tc5.cuh"

#define BS_KB 128                       // elements of K per stage: four MX blocks, four K = 32 MMAs
#define BS_SF_ATOM 512                  // scale-factor atom: 128 rows x 4 blocks
#define BS_SF_COLS 16
#define BS_MAX_KB 64                    // stages of one row at most (k <= 8192)
#ifndef BS_EXP_MOVERS
#define BS_EXP_MOVERS 1                   // experiment builds set 0: the eight warps stay out of the stage handshake (timing only)
#endif
#ifndef BS_SA
#define BS_SA 4                         // weight stages in flight (32 KB of shared memory each)
#define BS_SB 4                         // activation stages (8 KB each)
#endif
#ifdef BS_EXP_NOMMA
#define BS_EXP_MMA 0
#else
#define BS_EXP_MMA 1
#endif
#ifndef BS_L2_AHEAD
#define BS_L2_AHEAD 0                   // stages by which the weight tiles are asked for in L2 ahead of their copy (off: 4 / 8 / 16 measured slower than none)
#endif
#define BS_ISSUERS 2                    // MMA issuer threads: warp 5 takes the tile's first 128 rows, warp 14 the second 128
#define BS_THREADS (TC5_THREADS + 32 * (BS_ISSUERS - 1))
#define BS_PF 4                         // stages of raw codes an unpack thread keeps in flight                   // TMEM columns of one scale-factor set: A tile 0, A tile 1, B, spare

// Instruction descriptor, kind::mxf8f6f4 block-scaled: A e2m1, B e4m3, scales ue8m0, both K-major, D f32.
__host__ __device__ constexpr uint32_t bs_idesc(int m, int n, int a_sf, int b_sf) {
    return ((uint32_t)b_sf << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(m >> 4) << 24) |
           ((uint32_t)a_sf << 29);
}
// Shared-memory descriptor of a scale-factor atom: 32 rows of 16 bytes, no swizzle, 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t bs_sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;               // leading byte offset: a single 16-byte column, unused
    d |= (uint64_t)(128 >> 4) << 32;      // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;               // version
    return d;                             // swizzle field 0: none
}
__device__ __forceinline__ void bs_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void bs_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                       uint32_t tsfa, uint32_t tsfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
        : "memory");
}

// Position of element i of a 32-element block in the K order both operands use: 0, 16, 1, 17, ...
__host__ __device__ constexpr int bs_kpos(int i) { return i < 16 ? 2 * i : 2 * (i - 16) + 1; }

// One CTA per destination row: q[row][k] e4m3 bytes (block-permuted K order), sf[row][sf_stride] ue8m0 bytes. The
// source row is rowmap[row] when a map is given (entries outside [0, nsrc) read row 0: their destination belongs to
// no expert's list). The scale is the smallest power of two that brings the block's amax within e4m3's 448.
// A warp takes four blocks at a time: lane l holds elements 4 (l % 8) .. + 3 of block l / 8; elements e and e + 16 are
// neighbours in the permuted order, so lanes q and q + 4 of a block trade their codes and lane q < 4 stores 8 bytes.
// ndig > 1: the row is written as ndig e4m3 "digits" that share the block scales -- digit d + 1 is the e4m3 rounding of
// what digits 0..d leave of x / scale (the subtraction is exact in f32) -- into planes `plane` bytes apart. Each digit
// adds four significant bits: three of them carry an activation to 2^-12 of its block's largest element.
static __global__ void __launch_bounds__(256)
act_to_mx8_kernel(const void *__restrict__ x, int x_dtype, uint8_t *__restrict__ q, uint8_t *__restrict__ sf, int k, int sf_stride,
                  const int *__restrict__ rowmap, int nsrc, int ndig, size_t plane) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int src = row;
    if (rowmap) {
        src = rowmap[row];
        if ((unsigned)src >= (unsigned)nsrc) src = 0;
    }
    const size_t base = (size_t)src * k;
    const int nblk = k / 32, sub = lane >> 3, qd = lane & 7;
    for (int b0 = warp * 4; b0 < sf_stride; b0 += 32) {
        const int b = b0 + sub;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (b < nblk) {
            const size_t i = base + (size_t)b * 32 + 4 * qd;
            if (x_dtype == JL_DT_F32) {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(x) + i));
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            } else {
                const uint2 t = __ldg(reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(x) + i));
                if (x_dtype == JL_DT_BF16) {
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&t.x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&t.y));
                    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
                } else {
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&t.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&t.y));
                    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
                }
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 4; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // the block's eight lanes
        int se = 0;
        if (amax > 0.f && amax < __int_as_float(0x7f800000)) {
            int ex;
            const float m = frexpf(amax * (1.f / 448.f), &ex);     // amax / 448 = m 2^ex, m in [0.5, 1)
            se = m == 0.5f ? ex - 1 : ex;
            se = max(-126, min(127, se));
        }
        const float sc = __uint_as_float((uint32_t)(127 - se) << 23);
        float t[4];
#pragma unroll
        for (int j = 0; j < 4; j++) t[j] = v[j] * sc;
        for (int dgt = 0; dgt < ndig; dgt++) {
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const __nv_fp8_storage_t c = __nv_cvt_float_to_fp8(t[j], __NV_SATFINITE, __NV_E4M3);
                mine |= (uint32_t)(uint8_t)c << (8 * j);
                if (ndig > 1) t[j] -= __half2float(__half(__nv_cvt_fp8_to_halfraw(c, __NV_E4M3)));   // what this digit leaves
            }
            const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 4);   // lanes qd and qd + 4: elements e and e + 16
            if (b < nblk && qd < 4) {
                // bytes 8 qd .. 8 qd + 7: elements 4 qd + j (even positions) and 16 + 4 qd + j (odd positions)
                const uint32_t w0 = __byte_perm(mine, other, 0x5140), w1 = __byte_perm(mine, other, 0x7362);
                *reinterpret_cast<uint2 *>(q + (size_t)dgt * plane + (size_t)row * k + (size_t)b * 32 + 8 * qd) = make_uint2(w0, w1);
            }
        }
        if (b < nblk) {
            if (qd == 0) sf[(size_t)row * sf_stride + b] = (uint8_t)(127 + se);
        } else if (b < sf_stride && qd == 0) {
            sf[(size_t)row * sf_stride + b] = 127;                         // padding of the scale row: 2^0
        }
    }
}

// ------------------------------------------------------------------------------------------- the grouped GEMM
// (moe_gemm_params and moe_act come from moe.cu, which includes this file after defining them.)

template <int NT, int SA, int SB>
struct moe_bs_smem {
    static constexpr int ACC_COLS = TC5_MS * NT;
    static constexpr int ACC_BUFS = 2 * ACC_COLS + 2 * BS_SF_COLS <= 512 ? 2 : 1;   // one set: a unit's drain is not overlapped
    static constexpr int B_BYTES = NT * BS_KB;                 // e4m3: one byte per element
    static constexpr int A_OFS = 0;
    static constexpr int B_OFS = SA * TC5_MS * TC5_A_BYTES;    // an A tile is 128 rows x 128 bytes, as in the f16 arm
    static constexpr int SFA_OFS = B_OFS + SB * B_BYTES;
    static constexpr int SFB_OFS = SFA_OFS + SA * TC5_MS * BS_SF_ATOM;
    static constexpr int BAR_OFS = SFB_OFS + SA * BS_SF_ATOM;   // the activation scale atoms ride the A ring
    static constexpr int NBARS = 2 * SA + 4;                   // full[SA] empty[SA] acc_full[2] acc_empty[2]
    static_assert(SA == SB, "a stage is one weight tile pair + one activation tile behind one barrier");
    static constexpr int MISC_OFS = BAR_OFS + NBARS * 8;
    static constexpr int CNT_OFS = MISC_OFS + 16;              // the experts' list offsets: 257 ints (a length is a difference)
    static constexpr int TOTAL = CNT_OFS + 1040 + 1024;
    static constexpr int TMEM_COLS = 512;                      // accumulators (ACC_COLS x 2) + two scale-factor sets
    static_assert(ACC_COLS * ACC_BUFS + 2 * BS_SF_COLS <= TMEM_COLS && NT <= 128, "TMEM budget; one scale atom serves 128 columns");
};

#ifdef BS_EXP_TRACE        // timing experiment: CTA 0's MMA thread and producer thread stamp their first 512 stages
__device__ long long bs_trace[2][512][4];
__device__ unsigned long long bs_cta_t[2][160][2];     // per launch kind (mode) and CTA: global timer at entry and exit
#define BS_TR(role, i, j) do { if (blockIdx.x == 0 && (i) < 512u && (threadIdx.x >> 5) < 6 && (threadIdx.x & 31) == 0) bs_trace[role][i][j] = clock64(); } while (0)
#else
#define BS_TR(role, i, j) do { } while (0)
#endif

// Roles as in moe_gemm_kernel: warps 0..3 epilogue, 4 producer (activation tiles by TMA + their scale words), 5 MMA
// issuer (scale factors to TMEM, then four K = 32 MMAs per tile and stage), 6..13 unpack (thread r owns tile row r).
// TMAA: the weight tiles come by TMA as well (tensor maps of packed 4-bit type whose copies leave the 8-byte gaps the
// instruction wants: nothing touches a code between HBM and the tensor core), and the eight warps only move the
// scale words. Without it (the driver refused the maps) they also copy the codes through registers.
// T tokens of an expert's list per unit, each as DIG e4m3 digit columns (column d T + t of the tile: digit d of token
// t), T DIG <= NT = the MMAs' N. One digit: T = NT = 64. Three digits: T = 40 in N = 128 -- the drain adds a token's
// three columns, which brings the arm inside the parity bar of the exact one at the block-scaled MMAs' speed.
template <int NT, int T, int DIG, int SA, int SB, bool TMAA>
__global__ void __launch_bounds__(BS_THREADS, 1)
moe_gemm_bs_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap amap0,
                   const __grid_constant__ CUtensorMap amap1, const moe_gemm_params p) {
    using L = moe_bs_smem<NT, SA, SB>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::BAR_OFS);
    // One "full" and one "empty" barrier per stage: the issuers' time per stage is what bounds this kernel, and every
    // wait or commit they make costs them ~200 clocks even when it succeeds at once.
    uint64_t *full = bars, *empty = bars + SA;
    uint64_t *acc_full = bars + 2 * SA, *acc_empty = acc_full + 2;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::MISC_OFS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::MISC_OFS + 4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = (p.k + BS_KB - 1) / BS_KB;
    const int nblk = p.k / 32;
    int *s_off = reinterpret_cast<int *>(smem + L::CNT_OFS);

    if (tid == 0) {
        for (int s = 0; s < SA; s++) { mbar_init(smem_u32(full + s), BS_EXP_MOVERS * (TC5_DQ_THREADS / 32) + 1); mbar_init(smem_u32(empty + s), BS_ISSUERS); }
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(acc_full + i), BS_ISSUERS); mbar_init(smem_u32(acc_empty + i), 4); }
        abort_flag[0] = 0;
        abort_flag[1] = p.status[1];
        mbar_init_fence();
    }
    if (warp == 5) tc5_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), L::TMEM_COLS);
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // The list lengths and offsets, once, into shared memory: every role walks the unit list and asks for them at each
    // unit, live or not (from global memory that is an L2 round trip per unit and role). The walk ends at the longest
    // list's last token tile.
    if (tid <= p.n_expert) s_off[tid] = p.off[tid];      // off[n_expert] = the number of listed pairs
    __syncthreads();
    int longest = 0;
    for (int e = 0; e < p.n_expert; e++) longest = max(longest, (s_off[e + 1] - s_off[e]));
    const int nunits = p.n_expert * p.row_tiles * min(p.max_tok_tiles, (longest + T - 1) / T);

#define BS_UNIT(u)                                                                    \
    const int tt = (u) / (p.n_expert * p.row_tiles);                                  \
    const int e = ((u) / p.row_tiles) % p.n_expert, rt = (u) % p.row_tiles;           \
    const int m_eff = (s_off[e + 1] - s_off[e]), col0 = s_off[e] + tt * T;                             \
    const bool live = tt * T < m_eff;                                                 \
    (void)rt; (void)col0; (void)m_eff

#ifdef BS_EXP_TRACE
    if (tid == 0) bs_cta_t[p.mode][blockIdx.x][0] = jl_gtime_ns();
#endif
    if (warp == 4) {
        // TMA only, one lane: activation tile, then the two weight tiles. (Nothing in this warp writes shared memory:
        // a proxy fence here would wait for the copies in flight and put their latency into every stage.)
        if (lane == 0) {
            uint32_t kb_it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
                BS_UNIT(u);
                if (!live) continue;
                for (int kb = 0; kb < nkb && ok; kb++, kb_it++) {
                    const uint32_t s = kb_it % SA, ph = (kb_it / SA) & 1;
                    BS_TR(1, kb_it, 0);
                    if (kb_it >= (uint32_t)SA) ok = tc5_wait(smem_u32(empty + s), ph ^ 1, abort_flag);
                    if (!ok) break;
                    BS_TR(1, kb_it, 1);
                    // the activation tile and (TMAA) two boxes of 128 rows x 128 codes; in shared memory a code row takes
                    // 128 bytes (16 codes in the low half of every 16-byte unit), but the barrier counts the 64 bytes per
                    // row that are copied
#if defined(BS_EXP_NOA)
                    mbar_arrive_expect_tx(smem_u32(full + s), DIG * T * BS_KB);
#elif defined(BS_EXP_HALFA)
                    mbar_arrive_expect_tx(smem_u32(full + s), DIG * T * BS_KB + (TMAA ? TC5_A_BYTES / 2 : 0));
#else
                    mbar_arrive_expect_tx(smem_u32(full + s), DIG * T * BS_KB + (TMAA ? TC5_MS * TC5_A_BYTES / 2 : 0));
#endif
#pragma unroll
                    for (int dg = 0; dg < DIG; dg++)       // digit plane dg: rows dg * npairs + position (box: T rows)
                        tma_load_2d(sbase + L::B_OFS + s * L::B_BYTES + dg * T * BS_KB, &xmap, kb * BS_KB, dg * p.npairs + col0,
                                    smem_u32(full + s));
                    if (TMAA) {
                        const int y0 = e * p.rows + (p.mode == 0 ? rt * TC5_M : rt * TC5_ROWS);
                        const uint32_t dst = sbase + L::A_OFS + s * TC5_MS * TC5_A_BYTES;
#ifndef BS_EXP_NOA
                        tma_load_2d(dst, &amap0, kb * BS_KB, y0, smem_u32(full + s));
#ifndef BS_EXP_HALFA
                        tma_load_2d(dst + TC5_A_BYTES, p.mode == 0 ? &amap1 : &amap0, kb * BS_KB, p.mode == 0 ? y0 : y0 + TC5_M,
                                    smem_u32(full + s));
#endif
#endif
#if BS_L2_AHEAD > 0
                        // BS_L2_AHEAD stages further on, the same two boxes are asked for as far as L2 (of this unit, or
                        // of the unit this CTA takes next): the ring alone keeps too few bytes in flight to cover HBM's
                        // latency
                        int pk = kb + BS_L2_AHEAD, py = y0;
                        if (pk >= nkb) {
                            const int un = u + (int)gridDim.x;
                            pk -= nkb;
                            py = un < nunits && pk < nkb ? ((un / p.row_tiles) % p.n_expert) * p.rows +
                                                              (un % p.row_tiles) * (p.mode == 0 ? TC5_M : TC5_ROWS) : -1;
                        }
                        if (py >= 0) {
                            tma_prefetch_2d(&amap0, pk * BS_KB, py);
                            tma_prefetch_2d(p.mode == 0 ? &amap1 : &amap0, pk * BS_KB, p.mode == 0 ? py : py + TC5_M);
                        }
#endif
                    }
                    BS_TR(1, kb_it, 2);
                }
            }
        }
    } else if (warp == 5 || warp == TC5_THREADS / 32) {
        // Each issuer owns the accumulators of its 128-row operand and its own copies of the scale factors in TMEM
        // (nothing orders one thread's tcgen05.cp against another thread's MMAs): while one waits on the stage
        // barriers and commits, the other's MMAs execute.
        // The WHOLE warp runs the loop and one elected lane issues the tcgen05 instructions: every value the
        // instructions take (descriptors, TMEM addresses, barrier addresses) is then the same in all lanes, which lets
        // the compiler keep it where the instructions read it; what comes from memory is made so by a broadcast.
        const int wu = tc5_uniform(warp);
        const int ms_lo = BS_ISSUERS == 2 ? (wu == 5 ? 0 : 1) : 0, ms_hi = BS_ISSUERS == 2 ? ms_lo + 1 : TC5_MS;
        const uint32_t sfb_col = BS_ISSUERS == 2 ? 8 + 4 * ms_lo : 8;
        const bool leader = tc5_elect();
        const uint32_t tbase = (uint32_t)tc5_uniform((int)tmem_base), sb_u = (uint32_t)tc5_uniform((int)sbase);
        const uint32_t bars_u = sb_u + L::BAR_OFS;            // full[s] at +8 s, empty[s] at +8 (SA + s), acc_full at +16 SA
        {
            uint32_t kb_it = 0, unit_it = 0;
            bool ok = true, ready = false;
            const uint32_t tsf0 = tbase + L::ACC_COLS * L::ACC_BUFS;
            for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
                if (tc5_uniform(*abort_flag)) break;
                const int e = (u / p.row_tiles) % p.n_expert, tt = u / (p.n_expert * p.row_tiles);
                if (tt * T >= tc5_uniform((s_off[e + 1] - s_off[e]))) continue;                         // not a live unit
                const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
                if (unit_it >= (uint32_t)L::ACC_BUFS)
                    ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * (2 * SA + 2 + ab), aph ^ 1, abort_flag));
                if (!ok) break;
                tc5_fence_after();
                const uint32_t d_tmem = tbase + ab * L::ACC_COLS;
                for (int kb = 0; kb < nkb && ok; kb++, kb_it++) {
                    const uint32_t s = kb_it % SA, sa = s, ph = (kb_it / SA) & 1;
                    BS_TR(0, kb_it, 0);
                    if (!__all_sync(0xffffffffu, ready)) ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * s, ph, abort_flag));
                    BS_TR(0, kb_it, 1);
                    if (!ok) break;
                    tc5_fence_after();
                    // the next stage's barrier is probed now, so that the probe's latency passes under this stage's MMAs
                    ready = mbar_test_wait(bars_u + 8 * ((kb_it + 1) % SA), ((kb_it + 1) / SA) & 1);
                    BS_TR(0, kb_it, 2);
                    const uint32_t tsf = tsf0 + (kb_it & 1) * BS_SF_COLS;         // two sets, alternating
                    const uint64_t bdesc = tc5_smem_desc(sb_u + L::B_OFS + s * L::B_BYTES);
                    const int nj = min(BS_KB / 32, nblk - kb * (BS_KB / 32));     // the last stage of a row may be short
                    if (leader) {
#if !defined(BS_EXP_NOMMA) && !defined(BS_EXP_NOCP)
                        for (int ms = ms_lo; ms < ms_hi; ms++)
                            bs_cp_sf(tsf + ms * 4, bs_sf_desc(sb_u + L::SFA_OFS + (sa * TC5_MS + ms) * BS_SF_ATOM));
                        bs_cp_sf(tsf + sfb_col, bs_sf_desc(sb_u + L::SFB_OFS + sa * BS_SF_ATOM));
#endif
                        for (int ms = ms_lo; ms < ms_hi; ms++) {
                            const uint64_t adesc = tc5_smem_desc(sb_u + L::A_OFS + (sa * TC5_MS + ms) * TC5_A_BYTES);
#pragma unroll
                            for (int j = 0; j < BS_KB / 32; j++)
                                if (j < nj && BS_EXP_MMA)
                                    bs_mma(d_tmem + ms * NT, adesc + 2 * j, bdesc + 2 * j, bs_idesc(TC5_M, NT, j, j), (kb | j) != 0,
                                           tsf + ms * 4, tsf + sfb_col);
                        }
                        tc5_commit(bars_u + 8 * (SA + s));
                    }
                    BS_TR(0, kb_it, 3);
                }
                if (!ok) break;
                if (leader) tc5_commit(bars_u + 8 * (2 * SA + ab));
                unit_it++;
            }
        }
    } else if (warp >= 6 && warp < TC5_THREADS / 32 && BS_EXP_MOVERS) {
        // ---- unpack: thread r owns tile row r. mode 0: rows 0..127 gate, 128..255 up (same row index); mode 1: 256
        //      consecutive rows of down. Per stage: four blocks of 16 code bytes -> eight 16-byte units (codes in the low
        //      half), and the four block scales as one word of the scale-factor atom.
        const int r = tid - 192;
        const uint32_t swz = (uint32_t)(r & 7);
        const int a_row_ofs = (r >> 7) * TC5_A_BYTES + (r & 127) * 128;
        const int sf_ofs = (r >> 7) * BS_SF_ATOM + ((r & 127) & 31) * 16 + ((r & 127) >> 5) * 4;
        if constexpr (TMAA) {
            // The codes come by TMA: a thread moves one word of weight scales (its row's four blocks) and, for r < NT,
            // one word of activation scales per stage. The words run BS_PF stages ahead in registers as ONE stream over
            // all of the CTA's units, so that a new unit's first words are already here when its first stage opens
            // (loaded at the unit's start they put an HBM round trip into every unit).
            const bool second = p.mode == 0 && r >= 128;
            const uint8_t *eplane = second ? p.e1 : p.e0;
            int lu = blockIdx.x, lkb = 0;                      // the load cursor: unit, stage
            const uint32_t *ea = nullptr, *eb = nullptr;
            auto enter = [&]() {                               // first live unit at or after lu; its two rows of words
                for (; lu < nunits; lu += gridDim.x) {
                    BS_UNIT(lu);
                    if (!live) continue;
                    const int row = p.mode == 0 ? min(rt * TC5_M + (r & 127), p.rows - 1) : min(rt * TC5_ROWS + r, p.rows - 1);
                    ea = reinterpret_cast<const uint32_t *>(eplane + ((size_t)e * p.rows + row) * p.e_stride);
                    eb = reinterpret_cast<const uint32_t *>(p.sfb + (size_t)min(col0 + r % T, p.npairs - 1) * p.sfb_stride);   // column r: token r % T
                    return;
                }
            };
            auto load_one = [&](uint32_t &wa, uint32_t &wb) -> bool {
                if (lu >= nunits) return false;
                wa = __ldg(ea + lkb);
                wb = r < DIG * T ? __ldg(eb + lkb) : 0x7F7F7F7Fu;
                if (++lkb == nkb) { lkb = 0; lu += gridDim.x; enter(); }
                return true;
            };
            enter();
            uint32_t wa[BS_PF], wb[BS_PF];
            bool have[BS_PF];
#pragma unroll
            for (int j = 0; j < BS_PF; j++) { wa[j] = wb[j] = 0u; have[j] = load_one(wa[j], wb[j]); }
            bool ok = true;
            for (uint32_t it0 = 0; ok; it0 += BS_PF) {
#pragma unroll
                for (int j = 0; j < BS_PF; j++) {
                    if (!have[j]) { ok = false; break; }       // the stream has ended
                    const uint32_t it = it0 + j, s = it % SA, ph = (it / SA) & 1;
                    if (it >= (uint32_t)SA) ok = tc5_wait(smem_u32(empty + s), ph ^ 1, abort_flag);
                    if (!ok) break;
                    *reinterpret_cast<uint32_t *>(smem + L::SFA_OFS + s * TC5_MS * BS_SF_ATOM + sf_ofs) = wa[j];
                    if (r < NT) *reinterpret_cast<uint32_t *>(smem + L::SFB_OFS + s * BS_SF_ATOM + (r & 31) * 16 + (r >> 5) * 4) = wb[j];
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(full + s));
                    // refilled AFTER the fence: a proxy fence waits for the thread's loads in flight
                    have[j] = load_one(wa[j], wb[j]);
                }
            }
        } else {
        uint32_t kb_it = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
            BS_UNIT(u);
            if (!live) continue;
            const bool second = p.mode == 0 && r >= 128;
            const int row = p.mode == 0 ? min(rt * TC5_M + (r & 127), p.rows - 1) : min(rt * TC5_ROWS + r, p.rows - 1);
            const size_t grow = (size_t)e * p.rows + row;
            const uint8_t *codes = (second ? p.c1 : p.c0) + grow * nblk * 16;
            const uint8_t *ebytes = (second ? p.e1 : p.e0) + grow * p.e_stride;
            const uint32_t *sfb_row = reinterpret_cast<const uint32_t *>(p.sfb + (size_t)min(col0 + r % T, p.npairs - 1) * p.sfb_stride);
            uint32_t sfbw[BS_PF];                          // threads r < NT: token col0 + r's scale words, BS_PF stages ahead
#pragma unroll
            for (int j = 0; j < BS_PF; j++) sfbw[j] = (r < NT && j < nkb) ? __ldg(sfb_row + j) : 0x7F7F7F7Fu;
            auto load_stage = [&](int kb, uint4 (&c)[4], uint32_t &sfw) {
                sfw = 0x7F7F7F7Fu;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int blk = kb * 4 + b;
                    c[b] = make_uint4(0, 0, 0, 0);
                    if (blk < nblk) {
                        if (!TMAA) c[b] = ldg_nc16(codes + (size_t)blk * 16);
                        sfw = (sfw & ~(0xFFu << (8 * b))) | ((uint32_t)ebytes[blk] << (8 * b));
                    }
                }
            };
            // raw codes run BS_PF stages (64 bytes of the row each) ahead of their use, in registers: slot j is refilled
            // with stage kb + BS_PF the moment stage kb has been copied out of it
            uint4 q[BS_PF][4];
            uint32_t sfw[BS_PF];
#pragma unroll
            for (int j = 0; j < BS_PF; j++) {
                sfw[j] = 0x7F7F7F7Fu;
#pragma unroll
                for (int b = 0; b < 4; b++) q[j][b] = make_uint4(0, 0, 0, 0);
                if (j < nkb) load_stage(j, q[j], sfw[j]);
            }
            for (int kb0 = 0; kb0 < nkb && ok; kb0 += BS_PF) {
#pragma unroll
                for (int j = 0; j < BS_PF; j++) {
                    const int kb = kb0 + j;
                    if (kb >= nkb) break;
                    const uint32_t s = kb_it % SA, ph = (kb_it / SA) & 1;
                    uint4 c[4];
#pragma unroll
                    for (int b = 0; b < 4; b++) c[b] = q[j][b];
                    const uint32_t sf_cur = sfw[j], sfb_cur = sfbw[j];
                    if (kb_it >= (uint32_t)SA) ok = tc5_wait(smem_u32(empty + s), ph ^ 1, abort_flag);
                    if (!ok) break;
                    if (!TMAA) {
                        uint8_t *arow = smem + L::A_OFS + s * TC5_MS * TC5_A_BYTES + a_row_ofs;
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            *reinterpret_cast<uint4 *>(arow + (((uint32_t)(2 * b) ^ swz) << 4)) = make_uint4(c[b].x, c[b].y, 0u, 0u);
                            *reinterpret_cast<uint4 *>(arow + (((uint32_t)(2 * b + 1) ^ swz) << 4)) = make_uint4(c[b].z, c[b].w, 0u, 0u);
                        }
                    }
                    *reinterpret_cast<uint32_t *>(smem + L::SFA_OFS + s * TC5_MS * BS_SF_ATOM + sf_ofs) = sf_cur;
                    if (r < NT) *reinterpret_cast<uint32_t *>(smem + L::SFB_OFS + s * BS_SF_ATOM + (r & 31) * 16 + (r >> 5) * 4) = sfb_cur;
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(full + s));
                    kb_it++;
                    // refilled AFTER the fence: a proxy fence waits for the thread's loads in flight
#ifndef BS_EXP_NOSFLOAD
                    if (kb + BS_PF < nkb) {
#else
                    if (false) {
#endif
                        load_stage(kb + BS_PF, q[j], sfw[j]);
                        if (r < NT) sfbw[j] = __ldg(sfb_row + kb + BS_PF);
                    }
                }
            }
        }
        }
    } else if (warp < 4) {
        // ---- epilogue: warp w reads TMEM lanes 32w..32w+31 (tile rows), 32 token columns at a time
        uint32_t unit_it = 0;
        for (int u = blockIdx.x; u < nunits && !*abort_flag; u += gridDim.x) {
            BS_UNIT(u);
            if (!live) continue;
            const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
            if (!tc5_wait_relaxed(smem_u32(acc_full + ab), aph, abort_flag)) break;
            tc5_fence_after();
            const uint32_t tacc = tmem_base + ab * L::ACC_COLS + ((uint32_t)(warp * 32) << 16);
            const int pos_end = s_off[e] + (s_off[e + 1] - s_off[e]);
            if constexpr (DIG > 1) {
                // a token's DIG digit columns (d T + t) are added, most significant first, eight tokens at a time
                const int row0 = rt * TC5_M + warp * 32 + lane;                       // mode 0: the gate / up row of this lane
                const float bg = (p.mode == 0 && p.b0 && row0 < p.rows) ? p.b0[(size_t)e * p.rows + row0] : 0.f;
                const float bu = (p.mode == 0 && p.b1 && row0 < p.rows) ? p.b1[(size_t)e * p.rows + row0] : 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < T; c0 += 8) {
#ifdef BS_EXP_NOEPI
                    break;
#endif
                    const int pos0 = col0 + c0;
                    if (pos0 >= pos_end) break;                          // warp-uniform: the rest of the tile is past the list
                    if (p.mode == 0) {
                        float g[8], uu[8];
                        uint32_t vg[DIG][8], vu[DIG][8];
#pragma unroll
                        for (int dg = 0; dg < DIG; dg++) {
                            tc5_ld8(tacc + dg * T + c0, vg[dg]);
                            tc5_ld8(tacc + NT + dg * T + c0, vu[dg]);
                        }
                        tc5_wait_ld();                                   // one wait for the chunk's 2 DIG loads
#pragma unroll
                        for (int dg = 0; dg < DIG; dg++)
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                g[j] = dg ? g[j] + __uint_as_float(vg[dg][j]) : __uint_as_float(vg[dg][j]);
                                uu[j] = dg ? uu[j] + __uint_as_float(vu[dg][j]) : __uint_as_float(vu[dg][j]);
                            }
                        const int row = row0;
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int pos = pos0 + j;
                            if (row < p.rows && pos < pos_end) p.outp[(size_t)pos * p.rows + row] = moe_act(p.act, g[j] + bg, uu[j] + bu);
                        }
                    } else {
#pragma unroll 1
                        for (int ms = 0; ms < TC5_MS; ms++) {
                            float y[8];
                            uint32_t v[DIG][8];
#pragma unroll
                            for (int dg = 0; dg < DIG; dg++) tc5_ld8(tacc + ms * NT + dg * T + c0, v[dg]);
                            tc5_wait_ld();
#pragma unroll
                            for (int dg = 0; dg < DIG; dg++)
#pragma unroll
                                for (int j = 0; j < 8; j++) y[j] = dg ? y[j] + __uint_as_float(v[dg][j]) : __uint_as_float(v[dg][j]);
                            const int row = rt * TC5_ROWS + ms * TC5_M + warp * 32 + lane;
                            const float bd = (p.b0 && row < p.rows) ? p.b0[(size_t)e * p.rows + row] : 0.f;
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const int pos = pos0 + j;
                                if (row < p.rows && pos < pos_end)
                                    p.outp[(size_t)(p.out_rowmap ? p.out_rowmap[pos] : pos) * p.rows + row] = y[j] + bd;
                            }
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
#ifdef BS_EXP_NOEPI
                break;
#endif
                const int pos0 = col0 + c0;
                if (pos0 >= pos_end) break;                              // warp-uniform: the rest of the tile is past the list
                if (p.mode == 0) {
                    uint32_t vg[32], vu[32];
                    tc5_ld32(tacc + c0, vg);
                    tc5_ld32(tacc + NT + c0, vu);
                    tc5_wait_ld();
                    const int row = rt * TC5_M + warp * 32 + lane;
                    const float bg = (p.b0 && row < p.rows) ? p.b0[(size_t)e * p.rows + row] : 0.f;
                    const float bu = (p.b1 && row < p.rows) ? p.b1[(size_t)e * p.rows + row] : 0.f;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int pos = pos0 + j;
                        if (row < p.rows && pos < pos_end)
                            p.outp[(size_t)pos * p.rows + row] = moe_act(p.act, __uint_as_float(vg[j]) + bg, __uint_as_float(vu[j]) + bu);
                    }
                } else {
#pragma unroll 1
                    for (int ms = 0; ms < TC5_MS; ms++) {
                        uint32_t v[32];
                        tc5_ld32(tacc + ms * NT + c0, v);
                        tc5_wait_ld();
                        const int row = rt * TC5_ROWS + ms * TC5_M + warp * 32 + lane;
                        const float bd = (p.b0 && row < p.rows) ? p.b0[(size_t)e * p.rows + row] : 0.f;
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int pos = pos0 + j;
                            if (row < p.rows && pos < pos_end)
                                p.outp[(size_t)(p.out_rowmap ? p.out_rowmap[pos] : pos) * p.rows + row] = __uint_as_float(v[j]) + bd;
                        }
                    }
                }
            }
            tc5_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(acc_empty + ab));
            unit_it++;
        }
    }
#undef BS_UNIT
    tc5_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(p.status, 3);
#ifdef BS_EXP_TRACE
    if (tid == 0) bs_cta_t[p.mode][blockIdx.x][1] = jl_gtime_ns();
#endif
    if (warp == 5) {
        tc5_fence_after();
        tc5_dealloc(tmem_base, L::TMEM_COLS);
    }
}
