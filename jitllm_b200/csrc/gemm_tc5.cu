// Prefill GEMM: out[tok][row] = sum_k dequant(W)[row][k] * x[tok][k], Q4_K weights.
//
// The reference's prompt GEMM (jit/gpu/kernels/gemm70.go:99-131, chosen by f16Gemm,
// jit/gpu/tier/rows.go:1289-1327) dequantizes a CTA's rows to binary16 in shared memory
// and runs mma.sync over binary16 activations with f32 accumulation. This is the same
// arithmetic contract -- weights rounded ONCE to f16 after an f32 dequant, activations
// f16, f32 accumulate -- on Blackwell's own path:
//
//   warp 4        TMA producer. Raw Q4_K tiles (128 rows x one 144-byte super-block, a 2-D
//                 tensor map over the untouched ggml bytes) and activation tiles (NT tokens x
//                 64 k, 128-byte swizzle) land in shared memory, completion on mbarriers.
//   warps 6..13   dequant. Two threads per tile row (low-nibble / high-nibble sub-block): read the row's bytes, form
//                 w = (d sc) q - dmin m in f32 (one FFMA per weight on a nibble placed in a
//                 float's mantissa), rounds to f16 and stores the row's 128-byte k-block in
//                 the K-major SWIZZLE_128B layout tcgen05.mma reads.
//   warp 5        MMA issuer. One elected lane issues tcgen05.mma.cta_group::1.kind::f16,
//                 M = 128 rows, N = NT tokens, K = 16 per instruction, accumulators in
//                 TMEM (two buffers of NT columns, so a tile's epilogue overlaps the next
//                 tile's MMAs); tcgen05.commit releases shared-memory stages and publishes
//                 finished accumulators.
//   warps 0..3    epilogue. tcgen05.ld their 32-lane quarter of TMEM, undo the per-token
//                 activation scale, convert and store out[tok][row].
//
// Activations are converted once per call by act_to_f16_kernel: each token row is scaled by a
// power of two so its amax sits in [2^14, 2^15) (f16 then neither overflows nor flushes), and an
// f32 input is split x = hi + lo into two f16 rows whose products the epilogue adds, which keeps
// ~22 bits of the activation.
//
// Every wait on an mbarrier is bounded: when a limit runs out the kernel sets a status word,
// raises a CTA-wide abort flag that every role polls, frees its TMEM and returns.
#include "jl_internal.cuh"
#include "tma.cuh"

#define TC5_M 128           // weight rows per tile (the MMA's M)
#define TC5_KB 64           // k per shared-memory stage (128 bytes of f16: one swizzle atom)
#define TC5_RAW_BYTES (TC5_M * 144)
#define TC5_A_BYTES (TC5_M * TC5_KB * 2)
#define TC5_THREADS 448     // 14 warps: 4 epilogue, producer, MMA, 8 dequant
#define TC5_DQ_THREADS 256  // two threads per tile row: low-nibble half, high-nibble half

// ------------------------------------------------------------- activations

// One CTA per token row. dst rows: `split` ? (2 tok: hi, 2 tok + 1: lo) : tok.
__global__ void __launch_bounds__(256)
act_to_f16_kernel(const void *__restrict__ x, int x_dtype, __half *__restrict__ dst, float *__restrict__ inv_scale,
                  int k, int split) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float wmax[8];
    const int tok = blockIdx.x, tid = threadIdx.x;
    auto load = [&](int i) -> float {
        if (x_dtype == JL_DT_F32) return static_cast<const float *>(x)[(size_t)tok * k + i];
        if (x_dtype == JL_DT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(x)[(size_t)tok * k + i]);
        return __half2float(static_cast<const __half *>(x)[(size_t)tok * k + i]);
    };
    float amax = 0.f;
    for (int i = tid; i < k; i += 256) amax = fmaxf(amax, fabsf(load(i)));
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
    for (int i = tid; i < k; i += 256) {
        const float v = load(i) * scale;
        const __half h = __float2half_rn(v);
        hi[i] = h;
        if (split) lo[i] = __float2half_rn(v - __half2float(h));
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

// Bounded wait that also gives up when another role of the CTA has aborted.
__device__ __forceinline__ bool tc5_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < JL_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// The same, for a role that is not on the critical path: backs off between polls so that it
// does not take issue slots from the dequant warps it shares a scheduler with.
__device__ __forceinline__ bool tc5_wait_relaxed(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < (JL_SPIN_LIMIT >> 4); i++) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(256);
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// ------------------------------------------------------------------- kernel

struct tc5_params {
    int nrows, k, ntok, ntok_eff; // ntok_eff = MMA columns (2 x tokens when split)
    int split;                   // activations are hi/lo row pairs
    int row_tiles, tok_tiles;
    int out_dtype;
    void *out;                   // [ntok][nrows]
    const float *inv_scale;      // [ntok]
    int *status;
    int debug;                   // timing experiments: 1 = skip the dequant math, 2 = skip the MMAs
};

template <int NT, int STAGES>
struct tc5_smem {
    static constexpr int B_BYTES = NT * TC5_KB * 2;
    static constexpr int A_OFS = 0;
    static constexpr int B_OFS = STAGES * TC5_A_BYTES;
    static constexpr int RAW_OFS = B_OFS + STAGES * B_BYTES;
    static constexpr int BAR_OFS = RAW_OFS + 2 * TC5_RAW_BYTES;
    // barriers: a_full[S] b_full[S] empty[S] raw_full[2] raw_empty[2] acc_full[2] acc_empty[2]
    static constexpr int NBARS = 3 * STAGES + 8;
    static constexpr int MISC_OFS = BAR_OFS + NBARS * 8;   // tmem address, abort flag
    static constexpr int TOTAL = MISC_OFS + 16 + 1024;     // + slack to align the base to 1024
};

template <int NT, int STAGES>
__global__ void __launch_bounds__(TC5_THREADS, 1)
gemm_q4k_tc5_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                    const tc5_params p) {
    using L = tc5_smem<NT, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::BAR_OFS);
    uint64_t *a_full = bars, *b_full = bars + STAGES, *empty = bars + 2 * STAGES;
    uint64_t *raw_full = bars + 3 * STAGES, *raw_empty = raw_full + 2, *acc_full = raw_full + 4, *acc_empty = raw_full + 6;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::MISC_OFS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::MISC_OFS + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nsb = p.k / 256;               // super-blocks per row
    const int ntiles = p.row_tiles * p.tok_tiles;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(a_full + s), TC5_DQ_THREADS / 32);   // one arrival per dequant warp
            mbar_init(smem_u32(b_full + s), 1);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(smem_u32(raw_full + i), 1);
            mbar_init(smem_u32(raw_empty + i), TC5_DQ_THREADS / 32);
            mbar_init(smem_u32(acc_full + i), 1);
            mbar_init(smem_u32(acc_empty + i), 4);                      // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) tc5_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 2 * NT);
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // The activation rows come from the kernel in front (act_to_f16_kernel).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 4) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t kb_it = 0, raw_it = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x) {
                const int rt = tile / p.tok_tiles, tt = tile % p.tok_tiles;
                for (int sb = 0; sb < nsb; sb++, raw_it++) {
                    const uint32_t rs = raw_it & 1, rph = (raw_it >> 1) & 1;
                    if (raw_it >= 2 && !tc5_wait(smem_u32(raw_empty + rs), rph ^ 1, abort_flag)) break;
                    mbar_arrive_expect_tx(smem_u32(raw_full + rs), TC5_RAW_BYTES);
                    tma_load_2d(sbase + L::RAW_OFS + rs * TC5_RAW_BYTES, &wmap, sb * 144, rt * TC5_M,
                                smem_u32(raw_full + rs));
                    for (int j = 0; j < 4; j++, kb_it++) {
                        const uint32_t s = kb_it % STAGES, ph = (kb_it / STAGES) & 1;
                        if (kb_it >= STAGES && !tc5_wait(smem_u32(empty + s), ph ^ 1, abort_flag)) break;
                        mbar_arrive_expect_tx(smem_u32(b_full + s), L::B_BYTES);
                        tma_load_2d(sbase + L::B_OFS + s * L::B_BYTES, &xmap, sb * 256 + j * TC5_KB, tt * NT,
                                    smem_u32(b_full + s));
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = tc5_idesc(TC5_M, NT);
            uint32_t kb_it = 0, tile_it = 0;
            for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x, tile_it++) {
                const uint32_t ab = tile_it & 1, aph = (tile_it >> 1) & 1;
                if (tile_it >= 2 && !tc5_wait(smem_u32(acc_empty + ab), aph ^ 1, abort_flag)) break;
                tc5_fence_after();
                const uint32_t d_tmem = tmem_base + ab * NT;
                bool ok = true;
                for (int kb = 0; kb < nsb * 4 && ok; kb++, kb_it++) {
                    const uint32_t s = kb_it % STAGES, ph = (kb_it / STAGES) & 1;
                    ok = tc5_wait(smem_u32(a_full + s), ph, abort_flag) && tc5_wait(smem_u32(b_full + s), ph, abort_flag);
                    if (!ok) break;
                    tc5_fence_after();
                    const uint64_t adesc = tc5_smem_desc(sbase + L::A_OFS + s * TC5_A_BYTES);
                    const uint64_t bdesc = tc5_smem_desc(sbase + L::B_OFS + s * L::B_BYTES);
#pragma unroll
                    for (int j = 0; j < TC5_KB / 16; j++)  // 32 bytes of K per instruction: +2 in 16-byte units
                        if (!(p.debug & 2)) tc5_mma_f16(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | j) != 0);
                    tc5_commit(smem_u32(empty + s));      // stage reusable once these MMAs have read it
                }
                if (!ok) break;
                tc5_commit(smem_u32(acc_full + ab));      // accumulator complete
            }
        }
    } else if (warp >= 6) {
        // ------------------------------------------------ dequant: threads r and 128 + r own tile row r
        const int r = (tid - 192) & 127;
        const int nib = (tid - 192) >> 7;   // 0: low nibbles = sub-block 2j, 1: high nibbles = 2j+1
        const uint32_t swz = (uint32_t)(r & 7);
        uint32_t kb_it = 0, raw_it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok && !*abort_flag; tile += gridDim.x) {
            for (int sb = 0; sb < nsb && ok; sb++, raw_it++) {
                const uint32_t rs = raw_it & 1, rph = (raw_it >> 1) & 1;
                ok = tc5_wait(smem_u32(raw_full + rs), rph, abort_flag);
                if (!ok) break;
                const uint8_t *row = smem + L::RAW_OFS + rs * TC5_RAW_BYTES + r * 144;
                const uint4 h = *reinterpret_cast<const uint4 *>(row);
                const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
                // sc, m of the 8 sub-blocks (format/quant/dequant.go:360-365), four per word
                const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, m_lo = h.z & 0x3F3F3F3Fu;
                const uint32_t sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
                const uint32_t m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
#pragma unroll
                for (int j = 0; j < 4; j++, kb_it++) {   // k-block j = sub-blocks 2j (low nibbles), 2j+1 (high)
                    const uint32_t s = kb_it % STAGES, ph = (kb_it / STAGES) & 1;
                    const uint4 q0 = *reinterpret_cast<const uint4 *>(row + 16 + 32 * j);
                    const uint4 q1 = *reinterpret_cast<const uint4 *>(row + 32 + 32 * j);
                    const uint32_t scw = j < 2 ? sc_lo : sc_hi, mw = j < 2 ? m_lo : m_hi;
                    const int b0 = (2 * j) & 3;
                    // w = (16 d sc) (1 + q/16) - (16 d sc + dmin m): one FFMA on a nibble placed in the
                    // mantissa of 1.0; the products d sc and dmin m are exact in f32.
                    const float ds_e = 16.f * dd.x * (float)((scw >> (8 * b0)) & 0xFF);
                    const float ds_o = 16.f * dd.x * (float)((scw >> (8 * b0 + 8)) & 0xFF);
                    const float c_e = -(ds_e + dd.y * (float)((mw >> (8 * b0)) & 0xFF));
                    const float c_o = -(ds_o + dd.y * (float)((mw >> (8 * b0 + 8)) & 0xFF));
                    if (kb_it >= STAGES) ok = tc5_wait(smem_u32(empty + s), ph ^ 1, abort_flag);
                    if (!ok) break;
                    uint8_t *arow = smem + L::A_OFS + s * TC5_A_BYTES + r * 128;
                    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    const float ds = nib ? ds_o : ds_e, cc = nib ? c_o : c_e;
#pragma unroll
                    for (int cq = 0; cq < ((p.debug & 1) ? 0 : 4); cq++) {     // 16-byte chunk c = 4 nib + cq: k 8c..8c+7 of the k-block
                        uint32_t wa = w[2 * cq], wb = w[2 * cq + 1];
                        if (nib) { wa >>= 4; wb >>= 4; }
                        float f[8];                      // nibbles of bytes 0..3 -> mantissa bits 19..22
                        f[0] = __uint_as_float(((wa << 19) & 0x00780000u) | 0x3F800000u);
                        f[1] = __uint_as_float(((wa << 11) & 0x00780000u) | 0x3F800000u);
                        f[2] = __uint_as_float(((wa << 3) & 0x00780000u) | 0x3F800000u);
                        f[3] = __uint_as_float(((wa >> 5) & 0x00780000u) | 0x3F800000u);
                        f[4] = __uint_as_float(((wb << 19) & 0x00780000u) | 0x3F800000u);
                        f[5] = __uint_as_float(((wb << 11) & 0x00780000u) | 0x3F800000u);
                        f[6] = __uint_as_float(((wb << 3) & 0x00780000u) | 0x3F800000u);
                        f[7] = __uint_as_float(((wb >> 5) & 0x00780000u) | 0x3F800000u);
                        uint4 o;
                        __half2 h0 = __floats2half2_rn(fmaf(f[0], ds, cc), fmaf(f[1], ds, cc));
                        __half2 h1 = __floats2half2_rn(fmaf(f[2], ds, cc), fmaf(f[3], ds, cc));
                        __half2 h2 = __floats2half2_rn(fmaf(f[4], ds, cc), fmaf(f[5], ds, cc));
                        __half2 h3 = __floats2half2_rn(fmaf(f[6], ds, cc), fmaf(f[7], ds, cc));
                        o.x = *reinterpret_cast<uint32_t *>(&h0); o.y = *reinterpret_cast<uint32_t *>(&h1);
                        o.z = *reinterpret_cast<uint32_t *>(&h2); o.w = *reinterpret_cast<uint32_t *>(&h3);
                        *reinterpret_cast<uint4 *>(arow + (((uint32_t)(4 * nib + cq) ^ swz) << 4)) = o;
                    }
                    fence_async_smem();                   // generic writes -> visible to tcgen05.mma
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(a_full + s));
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(raw_empty + rs));
            }
        }
    } else {
        // ------------------------------------------------ epilogue: warp w reads TMEM lanes 32w..32w+31
        uint32_t tile_it = 0;
        for (int tile = blockIdx.x; tile < ntiles && !*abort_flag; tile += gridDim.x, tile_it++) {
            const int rt = tile / p.tok_tiles, tt = tile % p.tok_tiles;
            const uint32_t ab = tile_it & 1, aph = (tile_it >> 1) & 1;
            if (!tc5_wait_relaxed(smem_u32(acc_full + ab), aph, abort_flag)) break;
            tc5_fence_after();
            const int row = rt * TC5_M + warp * 32 + lane;
            const uint32_t taddr = tmem_base + ab * NT + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t v[32];
                tc5_ld32(taddr + c0, v);
                tc5_wait_ld();
                const int col0 = tt * NT + c0;
                // the per-token scales of these 32 columns: one load per lane, broadcast by shuffle
                const int mytok = p.split ? (col0 >> 1) + (lane & 15) : col0 + lane;
                const float myscale = mytok < p.ntok ? __ldg(p.inv_scale + mytok) : 0.f;
                if (p.split) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int tok = (col0 >> 1) + j;
                        const float sc = __shfl_sync(0xffffffffu, myscale, j);
                        if (row < p.nrows && tok < p.ntok) {
                            const float acc = (__uint_as_float(v[2 * j]) + __uint_as_float(v[2 * j + 1])) * sc;
                            const size_t o = (size_t)tok * p.nrows + row;
                            if (p.out_dtype == JL_DT_F32) static_cast<float *>(p.out)[o] = acc;
                            else if (p.out_dtype == JL_DT_BF16) static_cast<__nv_bfloat16 *>(p.out)[o] = __float2bfloat16_rn(acc);
                            else static_cast<__half *>(p.out)[o] = __float2half_rn(acc);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int tok = col0 + j;
                        const float sc = __shfl_sync(0xffffffffu, myscale, j);
                        if (row < p.nrows && tok < p.ntok) {
                            const float acc = __uint_as_float(v[j]) * sc;
                            const size_t o = (size_t)tok * p.nrows + row;
                            if (p.out_dtype == JL_DT_F32) static_cast<float *>(p.out)[o] = acc;
                            else if (p.out_dtype == JL_DT_BF16) static_cast<__nv_bfloat16 *>(p.out)[o] = __float2bfloat16_rn(acc);
                            else static_cast<__half *>(p.out)[o] = __float2half_rn(acc);
                        }
                    }
                }
            }
            tc5_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(acc_empty + ab));
        }
    }

    // teardown: everyone meets, the allocating warp frees TMEM
    tc5_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(p.status, 2);
    if (warp == 5) {
        tc5_fence_after();
        tc5_dealloc(tmem_base, 2 * NT);
    }
}

// --------------------------------------------------------------------- host

int jl_gemm_tc5_supported(uint32_t type, int nrows, int k, int ntok) {
    return type == JL_TYPE_Q4_K && k % 256 == 0 && nrows >= 1 && ntok >= 1;
}

static int tc5_pick_nt(int ntok_eff) { return ntok_eff > 128 ? 256 : (ntok_eff > 64 ? 128 : 64); }

int jl_gemm_tc5_choice(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out) {
    if (!jl_gemm_tc5_supported(type, nrows, k, ntok)) return JL_DECLINED;
    jl_choice c = {};
    int nt = tc5_pick_nt(ntok);
    c.kernel = JL_K_TC5; c.warps = TC5_THREADS / 32; c.rows_per_cta = TC5_M; c.split_k = 1;
    c.tile_m = TC5_M; c.tile_n = nt; c.tile_k = TC5_KB;
    int tiles = ((nrows + TC5_M - 1) / TC5_M) * ((ntok + nt - 1) / nt);
    int sms = ctx ? ctx->sm_count : 148;
    c.grid = tiles < sms ? tiles : sms;
    *out = c;
    return JL_OK;
}

size_t jl_gemm_tc5_scratch_bytes(int k, int ntok, int x_dtype) {
    size_t rows = (size_t)ntok * (x_dtype == JL_DT_F32 ? 2 : 1);
    return rows * (size_t)k * 2 + (size_t)ntok * 4 + 256;
}

template <int NT, int STAGES>
static int tc5_launch(jl_ctx *ctx, const CUtensorMap &wmap, const CUtensorMap &xmap, const tc5_params &p, int grid,
                      cudaStream_t s) {
    using L = tc5_smem<NT, STAGES>;
    JL_CUDA(ctx, cudaFuncSetAttribute(gemm_q4k_tc5_kernel<NT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      L::TOTAL));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(TC5_THREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_q4k_tc5_kernel<NT, STAGES>, wmap, xmap, p));
    return JL_OK;
}

int jl_launch_gemm_tc5(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, int expert,
                       const void *x_dev, int x_dtype, int ntok, cudaStream_t s) {
    const int nrows = w->nrows, k = w->k;
    if (!jl_gemm_tc5_supported(w->type, nrows, k, ntok))
        return jl_set_err(ctx, JL_DECLINED, "tcgen05 GEMM serves Q4_K with k %% 256 == 0");
    const int split = x_dtype == JL_DT_F32 ? 1 : 0;
    const int ntok_eff = ntok * (split ? 2 : 1);
    const size_t need = jl_gemm_tc5_scratch_bytes(k, ntok, x_dtype);
    if (ctx->scratch_cap < need)
        return jl_set_err(ctx, JL_ENOMEM, "GEMM scratch holds %zu bytes, %d tokens x %d need %zu (jl_reserve sizes it)",
                          ctx->scratch_cap, ntok, k, need);
    __half *xh = (__half *)ctx->scratch;
    float *inv_scale = (float *)((uint8_t *)ctx->scratch + (((size_t)ntok_eff * k * 2 + 255) & ~(size_t)255));

    // activations -> scaled f16 rows
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ntok); cfg.blockDim = dim3(256); cfg.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, act_to_f16_kernel, x_dev, x_dtype, xh, inv_scale, k, split));
        ctx->st.launches++;
    }

    const int nt = tc5_pick_nt(ntok_eff);
    CUtensorMap wmap, xmap;
    const uint8_t *wbase = w->data + (size_t)expert * nrows * jl_row_bytes(w->type, k);
    if (!jl_make_tmap_2d(&wmap, wbase, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, jl_row_bytes(w->type, k), (uint64_t)nrows,
                         jl_row_bytes(w->type, k), 144, TC5_M, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !jl_make_tmap_2d(&xmap, xh, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)k, (uint64_t)ntok_eff, (uint64_t)k * 2,
                         TC5_KB, nt, CU_TENSOR_MAP_SWIZZLE_128B))
        return jl_set_err(ctx, JL_DECLINED, "the driver refused a tensor map for this shape");

    tc5_params p;
    p.nrows = nrows; p.k = k; p.ntok = ntok; p.ntok_eff = ntok_eff; p.split = split;
    p.row_tiles = (nrows + TC5_M - 1) / TC5_M; p.tok_tiles = (ntok_eff + nt - 1) / nt;
    p.out_dtype = out_dtype; p.out = out_dev; p.inv_scale = inv_scale; p.status = ctx->dev_status;
    p.debug = (int)((ctx->opts.flags >> 16) & 3);
    const int tiles = p.row_tiles * p.tok_tiles;
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    int rc;
    if (nt == 256) rc = tc5_launch<256, 3>(ctx, wmap, xmap, p, grid, s);
    else if (nt == 128) rc = tc5_launch<128, 4>(ctx, wmap, xmap, p, grid, s);
    else rc = tc5_launch<64, 4>(ctx, wmap, xmap, p, grid, s);
    if (rc) return rc;
    ctx->st.launches++;
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}
