// Prefill GEMM: out[tok][row] = sum_k dequant(W)[row][k] * x[tok][k], Q4_K weights.
//
// The reference's prompt GEMM (jit/gpu/kernels/gemm70.go:99-131, chosen by f16Gemm,
// jit/gpu/tier/rows.go:1289-1327) dequantizes a CTA's rows to binary16 in shared memory
// and runs mma.sync over binary16 activations with f32 accumulation. This is the same
// arithmetic contract -- weights rounded ONCE to f16 after an f32 dequant, activations
// f16, f32 accumulate -- on Blackwell's own path:
//
//   warp 4        TMA producer. Activation tiles (NT tokens x 64 k, 128-byte swizzle) land in a
//                 deep shared-memory ring, completion on mbarriers.
//   warps 6..13   dequant. Thread r owns row r of the 256-row tile: reads its raw ggml bytes
//                 (128-bit loads, a super-block ahead of use) into registers, forms
//                 w = (d sc) q - dmin m in f32 (a PRMT places the code in a float's mantissa, one
//                 packed fma.rn.f32x2 per two weights), rounds to f16 and stores the row's 128-byte k-block in
//                 the K-major SWIZZLE_128B layout tcgen05.mma reads.
//   warp 5        MMA issuer. One elected lane issues tcgen05.mma.cta_group::1.kind::f16,
//                 M = 128 rows, N = NT tokens, K = 16 per instruction -- TWO per k step, one
//                 for each 128-row half of the tile against the same activation tile, which
//                 halves the activation bytes pulled through L2 per flop (the measured limit
//                 of a 128-row tile). Accumulators live in TMEM (2 x NT columns per tile);
//                 tcgen05.commit releases shared-memory stages and publishes accumulators.
//   warps 0..3    epilogue. tcgen05.ld their 32-lane quarter of TMEM, undo the per-token
//                 activation scale, convert and store out[tok][row].
//
// Activations are converted once per call by act_to_f16_kernel: each token row is scaled by a
// power of two so its amax sits in [2^14, 2^15) (f16 then neither overflows nor flushes), and an
// f32 input is split x = hi + lo into two f16 rows whose products the epilogue adds, which keeps
// ~22 bits of the activation.
//
// When a shape has fewer tiles than SMs the K range is split across CTAs; each split writes an
// f32 partial plane and tc5_reduce_kernel adds the planes in fixed order (bit-stable).
//
// Every wait on an mbarrier is bounded: when a limit runs out the kernel sets a status word,
// raises a CTA-wide abort flag that every role polls, frees its TMEM and returns.
#include "tc5.cuh"


// ------------------------------------------------------------------- kernel

struct tc5_params {
    int nrows, k, ntok, ntok_eff; // ntok_eff = MMA columns (2 x tokens when the activations are hi/lo pairs)
    int split;                    // activations are hi/lo row pairs
    int row_tiles, tok_tiles, ksplit;
    int out_dtype;
    void *out;                    // [ntok][nrows]
    float *partial;               // ksplit > 1: [ksplit][ntok][nrows] f32
    const float *inv_scale;       // [ntok]
    const uint8_t *w;             // Q4_K: raw rows of this weight (expert); Q8_0: its resident code plane [row][k]
    const uint16_t *w_d;          // Q8_0: f16 block scales [row][w_d_stride]
    int w_d_stride;
    int *status;                  // [0] timeout code, [1] wait limit in microseconds
};

template <int NT, int SA, int SB>
struct tc5_smem {
    static constexpr int ACC_COLS = TC5_MS * NT;                       // TMEM columns of one tile
    static constexpr int ACC_BUFS = ACC_COLS * 2 <= 512 ? 2 : 1;
    static constexpr int B_BYTES = NT * TC5_KB * 2;
    static constexpr int A_OFS = 0;                                    // [SA][MS] 128-row operands
    static constexpr int B_OFS = SA * TC5_MS * TC5_A_BYTES;            // [SB] activation tiles
    static constexpr int BAR_OFS = B_OFS + SB * B_BYTES;
    // barriers: a_full[SA] a_empty[SA] b_full[SB] b_empty[SB] acc_full[2] acc_empty[2]
    static constexpr int NBARS = 2 * SA + 2 * SB + 4;
    static constexpr int MISC_OFS = BAR_OFS + NBARS * 8;               // tmem address, abort flag
    static constexpr int TOTAL = MISC_OFS + 16 + 1024;                 // + slack to align the base to 1024
};

// Drains one finished tile from TMEM: lane quarter `q` (TMEM lanes 32q..32q+31 = tile rows), 32
// columns (tokens) at a time; undoes the per-token scale, converts, stores out[tok][row].
// part < 0: every 32-column job; part = 0,1,2: every third job (three warps share a quarter).
// One job of the drain: 32 accumulator columns of this lane's row, scaled per token and stored. KIND: 0 f32 (also the
// K-split partial planes), 1 bf16, 2 f16 -- decided once per call, not per element.
template <int KIND>
__device__ __forceinline__ void tc5_store32(const tc5_params &p, const uint32_t (&v)[32], void *base, int row, int col0, float myscale,
                                            int lane) {
    const int nj = p.split ? 16 : 32, tok0 = p.split ? col0 >> 1 : col0;
    const bool row_ok = row < p.nrows;
    size_t o = (size_t)tok0 * p.nrows + row;
#pragma unroll
    for (int j = 0; j < 32; j++) {
        if (j >= nj) break;
        const float sc = __shfl_sync(0xffffffffu, myscale, j);
        const float raw = p.split ? __uint_as_float(v[(2 * j) & 31]) + __uint_as_float(v[(2 * j + 1) & 31]) : __uint_as_float(v[j]);
        if (row_ok && tok0 + j < p.ntok) {
            const float acc = raw * sc;
            if (KIND == 0) static_cast<float *>(base)[o] = acc;
            else if (KIND == 1) static_cast<__nv_bfloat16 *>(base)[o] = __float2bfloat16_rn(acc);
            else static_cast<__half *>(base)[o] = __float2half_rn(acc);
        }
        o += p.nrows;
    }
}

template <int NT>
__device__ __forceinline__ void tc5_epilogue(const tc5_params &p, int u, uint32_t tmem_acc, int q, int lane, int part) {
    const int ks = u % p.ksplit, tt = (u / p.ksplit) % p.tok_tiles, rt = u / (p.ksplit * p.tok_tiles);
    float *partial = p.ksplit > 1 ? p.partial + (size_t)ks * p.ntok * p.nrows : nullptr;
    void *base = partial ? (void *)partial : p.out;
    const int kind = partial || p.out_dtype == JL_DT_F32 ? 0 : (p.out_dtype == JL_DT_BF16 ? 1 : 2);
    constexpr int NJ = TC5_MS * (NT / 32);                      // jobs of the tile: (128-row operand, 32 columns)
    // this warp's jobs: every job (part < 0) or every third one; the NEXT job's accumulators are asked for before
    // the current job is converted and stored, so the TMEM read's latency passes under the stores
    const int first = part < 0 ? 0 : part, step = part < 0 ? 1 : 3;
    auto taddr_of = [&](int job) { return tmem_acc + (job / (NT / 32)) * NT + ((uint32_t)(q * 32) << 16) + (job % (NT / 32)) * 32; };
    uint32_t va[32], vb[32];
    if (first < NJ) tc5_ld32(taddr_of(first), va);
#pragma unroll 1
    for (int job = first; job < NJ; job += 2 * step) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int jb = job + half * step;
            if (jb >= NJ) break;
            uint32_t (&cur)[32] = half ? vb : va;
            uint32_t (&nxt)[32] = half ? va : vb;
            const int ms = jb / (NT / 32), c0 = (jb % (NT / 32)) * 32;
            const int row = rt * TC5_ROWS + ms * TC5_M + q * 32 + lane, col0 = tt * NT + c0;
            // the per-token scales of these 32 columns: one load per lane, broadcast by shuffle
            const int mytok = p.split ? (col0 >> 1) + (lane & 15) : col0 + lane;
            const float myscale = mytok < p.ntok ? __ldg(p.inv_scale + mytok) : 0.f;
            tc5_wait_ld();
            if (jb + step < NJ) tc5_ld32(taddr_of(jb + step), nxt);
            if (kind == 0) tc5_store32<0>(p, cur, base, row, col0, myscale, lane);
            else if (kind == 1) tc5_store32<1>(p, cur, base, row, col0, myscale, lane);
            else tc5_store32<2>(p, cur, base, row, col0, myscale, lane);
        }
    }
}

// SA stages of dequantized weights, SB (deeper) stages of activations: an activation tile takes
// ~2 us to arrive from L2, a weight stage is produced locally.
// WT selects the weight format the dequant warps read: 0 = Q4_K (raw super-blocks), 1 = Q8_0 (resident
// code plane in 64-element span order + f16 scale plane). Everything else is shared.
#ifdef TC5_EXP_TRACE        // timing experiment: global-timer stamps of every CTA at seven points of its life
__device__ unsigned long long tc5_trace[160][8];
#define TC5_TR(i) do { tc5_trace[blockIdx.x][i] = jl_gtime_ns(); } while (0)
#else
#define TC5_TR(i) do { } while (0)
#endif
template <int WT, int NT, int SA, int SB>
__global__ void __launch_bounds__(TC5_GEMM_THREADS, 1)
gemm_q4k_tc5_kernel(const __grid_constant__ CUtensorMap xmap, const tc5_params p) {
    using L = tc5_smem<NT, SA, SB>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::BAR_OFS);
    uint64_t *a_full = bars, *a_empty = bars + SA, *b_full = bars + 2 * SA, *b_empty = b_full + SB;
    uint64_t *acc_full = b_empty + SB, *acc_empty = acc_full + 2;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::MISC_OFS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::MISC_OFS + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nsb = p.k / 256;               // super-blocks per row
    const int nunits = p.row_tiles * p.tok_tiles * p.ksplit;
    // unit u = (rt * tok_tiles + tt) * ksplit + ks; split ks covers super-blocks [sb0, sb1)
#define TC5_UNIT(u)                                                        \
    const int ks = (u) % p.ksplit, tt = ((u) / p.ksplit) % p.tok_tiles,    \
              rt = (u) / (p.ksplit * p.tok_tiles);                         \
    const int sb0 = (int)((long)ks * nsb / p.ksplit), sb1 = (int)((long)(ks + 1) * nsb / p.ksplit); \
    const int nsbu = sb1 - sb0, rot = (rt * 5 + tt * 3) % nsbu;                                     \
    (void)tt; (void)rt; (void)rot

    if (tid == 0) TC5_TR(0);
    if (tid == 0) {
        for (int s = 0; s < SA; s++) {
            mbar_init(smem_u32(a_full + s), TC5_DQ_THREADS / 32);   // one arrival per dequant warp
            mbar_init(smem_u32(a_empty + s), TC5_ISSUERS);          // one commit per MMA issuer
        }
        for (int s = 0; s < SB; s++) {
            mbar_init(smem_u32(b_full + s), 1);
            mbar_init(smem_u32(b_empty + s), TC5_ISSUERS);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(smem_u32(acc_full + i), TC5_ISSUERS);
            mbar_init(smem_u32(acc_empty + i), 4);                  // one arrival per epilogue warp
        }
        abort_flag[0] = 0;
        abort_flag[1] = p.status[1];                                // the wait limit, read once
        mbar_init_fence();
    }
    if (warp == 5) tc5_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), L::ACC_COLS * L::ACC_BUFS);
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0) TC5_TR(1);

    // The activation rows and their scales come from the kernel in front (act_to_f16_kernel): only
    // the roles that read them wait for it; the weights are converted meanwhile.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#define TC5_DEP_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")

    if (warp == 4) {
        // ------------------------------------------------ TMA producer: activation tiles
        TC5_DEP_WAIT();
        if (lane == 0) {
            uint32_t kb_it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
                TC5_UNIT(u);
                for (int i = 0; i < nsbu && ok; i++) {
                    const int sb = sb0 + (i + rot) % nsbu;   // every tile starts its K walk elsewhere
                    for (int j = 0; j < 4 && ok; j++, kb_it++) {
                        const uint32_t s = kb_it % SB, ph = (kb_it / SB) & 1;
                        if (kb_it >= (uint32_t)SB) ok = tc5_wait(smem_u32(b_empty + s), ph ^ 1, abort_flag);
                        if (!ok) break;
                        mbar_arrive_expect_tx(smem_u32(b_full + s), L::B_BYTES);
                        tma_load_2d(sbase + L::B_OFS + s * L::B_BYTES, &xmap, sb * 256 + j * TC5_KB, tt * NT,
                                    smem_u32(b_full + s));
                    }
                }
            }
        }
    } else if (warp == 5 || warp == TC5_MMA2_WARP) {
        // ------------------------------------------------ MMA issuers: each takes its 128-row operands of every stage
        // The whole warp runs the loop and an elected lane issues, so that what the instructions take is the same in
        // every lane; the next stage's barriers are probed before this stage's MMAs go out.
        constexpr uint32_t idesc = tc5_idesc(TC5_M, NT);
        const int wu = tc5_uniform(warp);
        const int ms_lo = TC5_ISSUERS == 2 ? (wu == 5 ? 0 : 1) : 0, ms_hi = TC5_ISSUERS == 2 ? ms_lo + 1 : TC5_MS;
        const bool leader = tc5_elect();
        const uint32_t tbase = (uint32_t)tc5_uniform((int)tmem_base), sb_u = (uint32_t)tc5_uniform((int)sbase);
        const uint32_t bars_u = sb_u + L::BAR_OFS;   // a_full +0, a_empty +SA, b_full +2SA, b_empty +2SA+SB, acc_full +2SA+2SB
        uint32_t kb_it = 0, unit_it = 0;
        bool ok = true, ready_a = false, ready_b = false;
        for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x, unit_it++) {
            if (tc5_uniform(*abort_flag)) break;
            TC5_UNIT(u);
            const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
            if (unit_it >= (uint32_t)L::ACC_BUFS)
                ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * (2 * SA + 2 * SB + 2 + ab), aph ^ 1, abort_flag));
            if (!ok) break;
            tc5_fence_after();
            const uint32_t d_tmem = tbase + ab * L::ACC_COLS;
            const int nkb = nsbu * 4;
            for (int kb = 0; kb < nkb && ok; kb++, kb_it++) {
                const uint32_t sa = kb_it % SA, pha = (kb_it / SA) & 1, s = kb_it % SB, ph = (kb_it / SB) & 1;
                if (!__all_sync(0xffffffffu, ready_a)) ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * sa, pha, abort_flag));
                if (ok && !__all_sync(0xffffffffu, ready_b))
                    ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * (2 * SA + s), ph, abort_flag));
                if (!ok) break;
                tc5_fence_after();
                if (kb_it == 0 && wu == 5 && leader) TC5_TR(2);
                ready_a = mbar_test_wait(bars_u + 8 * ((kb_it + 1) % SA), ((kb_it + 1) / SA) & 1);
                ready_b = mbar_test_wait(bars_u + 8 * (2 * SA + (kb_it + 1) % SB), ((kb_it + 1) / SB) & 1);
                if (leader) {
                    const uint64_t bdesc = tc5_smem_desc(sb_u + L::B_OFS + s * L::B_BYTES);
                    for (int ms = ms_lo; ms < ms_hi; ms++) {
                        const uint64_t adesc = tc5_smem_desc(sb_u + L::A_OFS + (sa * TC5_MS + ms) * TC5_A_BYTES);
#pragma unroll
                        for (int j = 0; j < TC5_KB / 16; j++)  // 32 bytes of K per instruction: +2 in 16-byte units
                            tc5_mma_f16(d_tmem + ms * NT, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | j) != 0);
                    }
                    tc5_commit(bars_u + 8 * (SA + sa));   // stages reusable once these MMAs have read them
                    tc5_commit(bars_u + 8 * (2 * SA + SB + s));
                }
            }
            if (!ok) break;
            if (leader) tc5_commit(bars_u + 8 * (2 * SA + 2 * SB + ab));      // accumulators complete
            if (wu == 5 && leader) TC5_TR(3);
        }
    } else if (warp >= 6) {
        // ------------------------------------------------ dequant: thread r owns tile row r
        // The row's raw bytes come straight from global memory into registers: while super-block i
        // is being converted, the 144 bytes of super-block i+1 are requested one 32-byte group per
        // k-block, so they are a full super-block period (~2 us) ahead of their use.
        const int r = tid - 192;
        const uint32_t swz = (uint32_t)(r & 7);
        const int a_row_ofs = (r >> 7) * TC5_A_BYTES + (r & 127) * 128;   // which 128-row operand, which row
        if constexpr (WT == 1) {
            // Q8_0: a "super-block" here is 256 k = four 64-element spans of the code plane (4 x 64 B) and
            // eight f16 scales (16 B). Span j of the NEXT super-block is requested into the registers of
            // span j as soon as span j of this one has been converted: four k-block periods ahead of use.
            uint32_t kb_it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
                TC5_UNIT(u);
                const int grow = min(rt * TC5_ROWS + r, p.nrows - 1);
                const uint8_t *crow = p.w + (size_t)grow * p.k;
                const uint8_t *drow = reinterpret_cast<const uint8_t *>(p.w_d + (size_t)grow * p.w_d_stride);
                uint4 q[4][4], dcur, dnxt = make_uint4(0, 0, 0, 0);
                {
                    const int sb = sb0 + rot % nsbu;
                    dcur = ldg_nc16(drow + (size_t)sb * 16);
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int t = 0; t < 4; t++) q[j][t] = ldg_nc16(crow + (size_t)sb * 256 + j * 64 + t * 16);
                }
                for (int i = 0; i < nsbu && ok; i++) {
                    const bool more = i + 1 < nsbu;
                    const int nsbi = sb0 + (i + 1 + rot) % nsbu;
                    const uint32_t dw[4] = {dcur.x, dcur.y, dcur.z, dcur.w};
#pragma unroll
                    for (int j = 0; j < 4; j++, kb_it++) {
                        const uint32_t s = kb_it % SA, ph = (kb_it / SA) & 1;
                        if (kb_it >= (uint32_t)SA) ok = tc5_wait(smem_u32(a_empty + s), ph ^ 1, abort_flag);
                        if (!ok) break;
                        uint8_t *arow = smem + L::A_OFS + s * TC5_MS * TC5_A_BYTES + a_row_ofs;
                        // the two block scales of this span, each broadcast to both halves of a half2
                        const uint32_t d0 = __byte_perm(dw[j], 0, 0x1010), d1 = __byte_perm(dw[j], 0, 0x3232);
                        const uint32_t bias = 0x64806480u;   // half2(1152, 1152): 1024 + the 128 that made the code unsigned
#pragma unroll
                        for (int c = 0; c < 8; c++) {       // 16-byte chunk c = k 8c..8c+7 of the span
                            const int wi = c >> 1, ta = 2 * (c & 1);
                            const uint4 pa = q[j][ta], pb = q[j][ta + 1];
                            const uint32_t wa = (wi == 0 ? pa.x : wi == 1 ? pa.y : wi == 2 ? pa.z : pa.w) ^ 0x80808080u;
                            const uint32_t wb = (wi == 0 ? pb.x : wi == 1 ? pb.y : wi == 2 ? pb.z : pb.w) ^ 0x80808080u;
                            const uint32_t dd = (c >> 2) ? d1 : d0;
                            // byte u -> f16 0x6400 | u = 1024 + u (exact), minus 1152 = the signed code (exact),
                            // times d: ONE rounding, to f16
                            uint4 o;
                            o.x = hmul2u(hsub2u(__byte_perm(wa, 0x64646464u, 0x4140), bias), dd);
                            o.y = hmul2u(hsub2u(__byte_perm(wa, 0x64646464u, 0x4342), bias), dd);
                            o.z = hmul2u(hsub2u(__byte_perm(wb, 0x64646464u, 0x4140), bias), dd);
                            o.w = hmul2u(hsub2u(__byte_perm(wb, 0x64646464u, 0x4342), bias), dd);
                            *reinterpret_cast<uint4 *>(arow + (((uint32_t)c ^ swz) << 4)) = o;
                        }
                        if (more) {
                            if (j == 0) dnxt = ldg_nc16(drow + (size_t)nsbi * 16);
#pragma unroll
                            for (int t = 0; t < 4; t++) q[j][t] = ldg_nc16(crow + (size_t)nsbi * 256 + j * 64 + t * 16);
                        }
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(a_full + s));
                    }
                    if (!ok) break;
                    dcur = dnxt;
                }
            }
        } else {
            const size_t row_bytes = (size_t)nsb * 144;
            uint32_t kb_it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
                TC5_UNIT(u);
                const int grow = min(rt * TC5_ROWS + r, p.nrows - 1);          // rows past the end repeat the last
                const uint8_t *wrow = p.w + (size_t)grow * row_bytes;
                uint4 hcur, hnxt = make_uint4(0, 0, 0, 0), qcur[8], qnxt[8];
                {
                    const uint8_t *b = wrow + (size_t)(sb0 + rot % nsbu) * 144;
                    hcur = ldg_nc16(b);
    #pragma unroll
                    for (int g = 0; g < 8; g++) qcur[g] = ldg_nc16(b + 16 + 16 * g);
                }
                for (int i = 0; i < nsbu && ok; i++) {
                    const bool more = i + 1 < nsbu;
                    const uint8_t *nb = wrow + (size_t)(sb0 + (i + 1 + rot) % nsbu) * 144;
                    const uint4 h = hcur;
                    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
                    // sc, m of the 8 sub-blocks (format/quant/dequant.go:360-365), four per word
                    const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, m_lo = h.z & 0x3F3F3F3Fu;
                    const uint32_t sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
                    const uint32_t m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    #pragma unroll
                    for (int j = 0; j < 4; j++, kb_it++) {   // k-block j = sub-blocks 2j (low nibbles), 2j+1 (high)
                        const uint32_t s = kb_it % SA, ph = (kb_it / SA) & 1;
                        const uint4 q0 = qcur[2 * j], q1 = qcur[2 * j + 1];
                        if (more) {       // next super-block: group j (and its header with j = 0)
                            if (j == 0) hnxt = ldg_nc16(nb);
                            qnxt[2 * j] = ldg_nc16(nb + 16 + 32 * j);
                            qnxt[2 * j + 1] = ldg_nc16(nb + 32 + 32 * j);
                        }
                        const uint32_t scw = j < 2 ? sc_lo : sc_hi, mw = j < 2 ? m_lo : m_hi;
                        const int b0 = (2 * j) & 3;
                        // w = (128 d sc) (1 + q/128) - (128 d sc + dmin m): one FMA on a code placed in the
                        // mantissa of 1.0; the products d sc and dmin m are exact in f32.
                        const float ds_e = 128.f * dd.x * (float)((scw >> (8 * b0)) & 0xFF);
                        const float ds_o = 128.f * dd.x * (float)((scw >> (8 * b0 + 8)) & 0xFF);
                        const float c_e = -(ds_e + dd.y * (float)((mw >> (8 * b0)) & 0xFF));
                        const float c_o = -(ds_o + dd.y * (float)((mw >> (8 * b0 + 8)) & 0xFF));
                        if (kb_it >= (uint32_t)SA) ok = tc5_wait(smem_u32(a_empty + s), ph ^ 1, abort_flag);
                        if (!ok) break;
                        uint8_t *arow = smem + L::A_OFS + s * TC5_MS * TC5_A_BYTES + a_row_ofs;
                        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    #pragma unroll
                        for (int c = 0; c < 8; c++) {    // 16-byte chunk c = k 8c..8c+7 of the k-block
                            const int nib = c >> 2, cq = c & 3;
                            const float ds = nib ? ds_o : ds_e, cc = nib ? c_o : c_e;
                            // four codes of a word -> bytes 0x80 | q: byte 2 of a float whose byte 3 is 0x3F,
                            // i.e. 1 + q/128, picked out by one PRMT per weight
                            const uint32_t ua = ((nib ? w[2 * cq] >> 4 : w[2 * cq]) & 0x0F0F0F0Fu) | 0x80808080u;
                            const uint32_t ub = ((nib ? w[2 * cq + 1] >> 4 : w[2 * cq + 1]) & 0x0F0F0F0Fu) | 0x80808080u;
                            float v[8];
                            tc5_fma2(v[0], v[1], tc5_code_float(ua, 0), tc5_code_float(ua, 1), ds, cc);
                            tc5_fma2(v[2], v[3], tc5_code_float(ua, 2), tc5_code_float(ua, 3), ds, cc);
                            tc5_fma2(v[4], v[5], tc5_code_float(ub, 0), tc5_code_float(ub, 1), ds, cc);
                            tc5_fma2(v[6], v[7], tc5_code_float(ub, 2), tc5_code_float(ub, 3), ds, cc);
                            uint4 o;
                            __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                            __half2 h2 = __floats2half2_rn(v[4], v[5]), h3 = __floats2half2_rn(v[6], v[7]);
                            o.x = *reinterpret_cast<uint32_t *>(&h0); o.y = *reinterpret_cast<uint32_t *>(&h1);
                            o.z = *reinterpret_cast<uint32_t *>(&h2); o.w = *reinterpret_cast<uint32_t *>(&h3);
                            *reinterpret_cast<uint4 *>(arow + (((uint32_t)c ^ swz) << 4)) = o;
                        }
                        fence_async_smem();   // generic writes -> visible to tcgen05.mma
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(a_full + s));
                    }
                    if (!ok) break;
                    hcur = hnxt;
    #pragma unroll
                    for (int g = 0; g < 8; g++) qcur[g] = qnxt[g];
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue: warp w reads TMEM lanes 32w..32w+31
        TC5_DEP_WAIT();
        uint32_t unit_it = 0;
        for (int u = blockIdx.x; u < nunits && !*abort_flag; u += gridDim.x, unit_it++) {
            const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
            if (!tc5_wait_relaxed(smem_u32(acc_full + ab), aph, abort_flag)) break;
            tc5_fence_after();
            if (tid == 0) TC5_TR(4);
            // the CTA's last unit is shared with the dequant warps, which have nothing left to do
            const bool last = u + (int)gridDim.x >= nunits;
            tc5_epilogue<NT>(p, u, tmem_base + ab * L::ACC_COLS, warp, lane, last ? 0 : -1);
            tc5_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(acc_empty + ab));
        }
    }
    if (warp >= 6 && warp < TC5_MMA2_WARP && !*abort_flag && (int)blockIdx.x < nunits) {
        // ------------------------------------------------ dequant warps help drain the last accumulators
        TC5_DEP_WAIT();
        const int n_mine = (nunits - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
        const uint32_t unit_it = (uint32_t)(n_mine - 1);
        const int u = (int)blockIdx.x + (n_mine - 1) * (int)gridDim.x;
        const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
        if (tc5_wait_relaxed(smem_u32(acc_full + ab), aph, abort_flag)) {
            tc5_fence_after();
            tc5_epilogue<NT>(p, u, tmem_base + ab * L::ACC_COLS, warp & 3, lane, 1 + ((warp - 6) >> 2));
        }
    }
#undef TC5_UNIT
#undef TC5_DEP_WAIT

    // teardown: everyone meets, the allocating warp frees TMEM
    if (tid == 0) TC5_TR(5);
    tc5_fence_before();
    __syncthreads();
    if (tid == 0) TC5_TR(6);
    if (tid == 0 && *abort_flag) atomicExch(p.status, 2);
    if (warp == 5) {
        tc5_fence_after();
        tc5_dealloc(tmem_base, L::ACC_COLS * L::ACC_BUFS);
    }
}

// out = sum over the K splits of their partial planes, in split order.
__global__ void __launch_bounds__(256)
tc5_reduce_kernel(const float *__restrict__ partial, void *__restrict__ out, int out_dtype, size_t n, int ksplit) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float acc = partial[i];
        for (int s = 1; s < ksplit; s++) acc += partial[(size_t)s * n + i];
        if (out_dtype == JL_DT_F32) static_cast<float *>(out)[i] = acc;
        else if (out_dtype == JL_DT_BF16) static_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(acc);
        else static_cast<__half *>(out)[i] = __float2half_rn(acc);
    }
}

// --------------------------------------------------------------------- host

int jl_gemm_tc5_supported(uint32_t type, int nrows, int k, int ntok) {
    return (type == JL_TYPE_Q4_K || type == JL_TYPE_Q8_0) && k % 256 == 0 && nrows >= 1 && ntok >= 1;
}

static int tc5_pick_nt(int ntok_eff) { return ntok_eff > 128 ? 256 : (ntok_eff > 64 ? 128 : 64); }

// How many CTAs share one tile's K range: only when the tiles alone would leave SMs idle.
static int tc5_ksplit(int nrows, int ntok_eff, int k, int sms) {
    const int nt = tc5_pick_nt(ntok_eff);
    const int units = ((nrows + TC5_ROWS - 1) / TC5_ROWS) * ((ntok_eff + nt - 1) / nt);
    int ks = sms / units;
    if (ks > 8) ks = 8;
    if (ks > k / 256) ks = k / 256;
    return ks < 2 ? 1 : ks;
}

// Answers for f32 activations (what jl_select is asked about: the decode-side entry points take f32), which
// occupy two MMA columns per token (hi + lo); 16-bit activations occupy one.
int jl_gemm_tc5_choice(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out) {
    if (!jl_gemm_tc5_supported(type, nrows, k, ntok)) return JL_DECLINED;
    jl_choice c = {};
    const int sms = ctx ? ctx->sm_count : 148;
    const int ntok_eff = 2 * ntok;
    const int nt = tc5_pick_nt(ntok_eff);
    c.kernel = JL_K_TC5; c.warps = TC5_GEMM_THREADS / 32; c.rows_per_cta = TC5_ROWS;
    c.split_k = tc5_ksplit(nrows, ntok_eff, k, sms);
    c.tile_m = TC5_M; c.tile_n = nt; c.tile_k = TC5_KB;
    const int units = ((nrows + TC5_ROWS - 1) / TC5_ROWS) * ((ntok_eff + nt - 1) / nt) * c.split_k;
    c.grid = units < sms ? units : sms;
    c.launches = 2 + (c.split_k > 1 ? 1 : 0);   // activation conversion, GEMM, and the split-K sum when K is split
    *out = c;
    return JL_OK;
}

size_t jl_gemm_tc5_scratch_bytes(int nrows, int k, int ntok, int x_dtype, int sms) {
    const int ntok_eff = ntok * (x_dtype == JL_DT_F32 ? 2 : 1);
    size_t b = (((size_t)ntok_eff * k * 2 + 255) & ~(size_t)255) + (((size_t)ntok * 4 + 255) & ~(size_t)255);
    const int ks = tc5_ksplit(nrows, ntok_eff, k, sms);
    if (ks > 1) b += (size_t)ks * ntok * nrows * 4;
    return b + 256;
}

template <int WT, int NT, int SA, int SB>
static int tc5_launch(jl_ctx *ctx, const CUtensorMap &xmap, const tc5_params &p, int grid,
                      cudaStream_t s) {
    using L = tc5_smem<NT, SA, SB>;
    static_assert(L::TOTAL <= 227 * 1024, "shared memory budget");
    JL_CUDA(ctx, cudaFuncSetAttribute(gemm_q4k_tc5_kernel<WT, NT, SA, SB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      L::TOTAL));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(TC5_GEMM_THREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_q4k_tc5_kernel<WT, NT, SA, SB>, xmap, p));
    return JL_OK;
}

// Where a producer writes the GEMM's activation operand for `ntok` f32-precision tokens of width w->k: rows
// [2 tok] = hi, [2 tok + 1] = lo (f16, k each) and one f32 1/scale per token. JL_DECLINED when the scratch is too small.
int jl_gemm_tc5_operand(jl_ctx *ctx, const jl_weight *w, int ntok, void **rows, float **inv_scale) {
    if (!jl_gemm_tc5_supported(w->type, w->nrows, w->k, ntok)) return JL_DECLINED;
    if (ctx->scratch_cap < jl_gemm_tc5_scratch_bytes(w->nrows, w->k, ntok, JL_DT_F32, ctx->sm_count)) return JL_DECLINED;
    uint8_t *sp = (uint8_t *)ctx->scratch;
    *rows = sp;
    *inv_scale = (float *)(sp + (((size_t)ntok * 2 * w->k * 2 + 255) & ~(size_t)255));
    return JL_OK;
}

int jl_launch_gemm_tc5(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, int expert,
                       const void *x_dev, int x_dtype, int ntok, cudaStream_t s) {
    const int nrows = w->nrows, k = w->k;
    if (!jl_gemm_tc5_supported(w->type, nrows, k, ntok))
        return jl_set_err(ctx, JL_DECLINED, "tcgen05 GEMM serves Q4_K and Q8_0 with k %% 256 == 0");
    // x_dev == NULL: the f16 hi/lo rows and the per-token scales are in the scratch already (a producer kernel wrote
    // them where jl_gemm_tc5_operand said, in the layout of f32 activations): no conversion launch
    const bool prepared = x_dev == nullptr;
    if (prepared) x_dtype = JL_DT_F32;
    const int split = x_dtype == JL_DT_F32 ? 1 : 0;
    const int ntok_eff = ntok * (split ? 2 : 1);
    const size_t need = jl_gemm_tc5_scratch_bytes(nrows, k, ntok, x_dtype, ctx->sm_count);
    if (ctx->scratch_cap < need)
        return jl_set_err(ctx, JL_ENOMEM, "GEMM scratch holds %zu bytes, %d tokens x %d x %d need %zu (jl_reserve sizes it)",
                          ctx->scratch_cap, ntok, nrows, k, need);
    uint8_t *sp = (uint8_t *)ctx->scratch;
    __half *xh = (__half *)sp;
    sp += ((size_t)ntok_eff * k * 2 + 255) & ~(size_t)255;
    float *inv_scale = (float *)sp;
    sp += ((size_t)ntok * 4 + 255) & ~(size_t)255;
    float *partial = (float *)sp;

    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    const int nattr = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    if (!prepared) {   // activations -> scaled f16 rows
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ntok); cfg.blockDim = dim3(256); cfg.stream = s;
        cfg.attrs = at; cfg.numAttrs = nattr;
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, act_to_f16_kernel, x_dev, x_dtype, xh, inv_scale, k, split, (const int *)nullptr, 0));
        ctx->st.launches++;
    }

    const int nt = tc5_pick_nt(ntok_eff);
    CUtensorMap xmap;
    const bool q8 = w->type == JL_TYPE_Q8_0;
    const uint8_t *wbase = w->data + (size_t)expert * nrows * (q8 ? (size_t)k : jl_row_bytes(w->type, k));
    if (!jl_make_tmap_2d(&xmap, xh, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)k, (uint64_t)ntok_eff, (uint64_t)k * 2,
                         TC5_KB, nt, CU_TENSOR_MAP_SWIZZLE_128B))
        return jl_set_err(ctx, JL_DECLINED, "the driver refused a tensor map for this shape");

    tc5_params p;
    p.nrows = nrows; p.k = k; p.ntok = ntok; p.ntok_eff = ntok_eff; p.split = split;
    p.row_tiles = (nrows + TC5_ROWS - 1) / TC5_ROWS; p.tok_tiles = (ntok_eff + nt - 1) / nt;
    p.ksplit = tc5_ksplit(nrows, ntok_eff, k, ctx->sm_count);
    p.out_dtype = out_dtype; p.out = out_dev; p.partial = partial; p.inv_scale = inv_scale; p.w = wbase; p.status = ctx->dev_status;
    p.w_d = q8 ? reinterpret_cast<const uint16_t *>(w->scales) + (size_t)expert * nrows * w->scale_stride : nullptr;
    p.w_d_stride = w->scale_stride;
    const int units = p.row_tiles * p.tok_tiles * p.ksplit;
    const int grid = units < ctx->sm_count ? units : ctx->sm_count;
    int rc;
    // Ring depths: the weight stages are produced locally (3 deep is enough) and every KB of shared memory not
    // taken is L1 for the dequant warps' raw-weight loads -- with 224 KB of rings (A 4 deep, B 3 deep) the 256-token
    // tile ran 7 % slower than with 160 KB (A 3, B 2); 128 KB (A 2, B 2) is on par.
    if (q8) {
        if (nt == 256) rc = tc5_launch<1, 256, 3, 2>(ctx, xmap, p, grid, s);
        else if (nt == 128) rc = tc5_launch<1, 128, 3, 6>(ctx, xmap, p, grid, s);
        else rc = tc5_launch<1, 64, 3, 8>(ctx, xmap, p, grid, s);
    } else {
        if (nt == 256) rc = tc5_launch<0, 256, 3, 2>(ctx, xmap, p, grid, s);
        else if (nt == 128) rc = tc5_launch<0, 128, 3, 6>(ctx, xmap, p, grid, s);
        else rc = tc5_launch<0, 64, 3, 8>(ctx, xmap, p, grid, s);
    }
    if (rc) return rc;
    ctx->st.launches++;
    if (p.ksplit > 1) {
        const size_t n = (size_t)ntok * nrows;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((n + 1023) / 1024 < 1184 ? (n + 1023) / 1024 : 1184)); cfg.blockDim = dim3(256);
        cfg.stream = s; cfg.attrs = at; cfg.numAttrs = nattr;
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, tc5_reduce_kernel, (const float *)partial, out_dev, out_dtype, n, p.ksplit));
        ctx->st.launches++;
    }
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}

#ifdef TC5_EXP_TRACE
JL_EXPORT int jl_exp_tc5_trace(unsigned long long *host) { return (int)cudaMemcpyFromSymbol(host, tc5_trace, sizeof(tc5_trace)); }
#endif
