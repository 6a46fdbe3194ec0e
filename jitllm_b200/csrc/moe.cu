// Mixture-of-experts layer: State.moeBatch (engine/model/moe.go:502-760).
//
//   route    softmax over the router logits, lexicographic top-k (ties to the lowest id, a NaN
//            never eligible), weights = score / (sum in SELECTION order + 1e-20) * scale
//            (engine/nn/moetopk.go:316-385, internal/oracle/moe.go:197-359)
//   sort     stable counting sort of the (token, slot) pairs by expert: the per-expert token
//            lists, on the device, with no host round trip (the reference reads one word home
//            per chunk to size its grouped launches, jit/gpu/tier/moegroup.go:10-19; here the
//            grids are sized by the static worst case and surplus work units exit)
//   gather   token rows -> expert order, as scaled f16 rows (act_to_f16_kernel with a row map)
//   gate|up  grouped tcgen05 GEMM over the token lists: a 256-row tile is 128 gate rows + 128
//            up rows of one expert against the same activation tile, so the epilogue holds g
//            and u of one (row, token) in one thread and writes act(g, u)
//   down     grouped tcgen05 GEMM, y = down_e act
//   combine  out[token] += w_e y_e over the token's experts in ASCENDING expert id
//            (engine/model/moe.go:127-134): a fixed order, so the result is bit-stable
//
// MXFP4 weights are exact in f16 (e2m1 times a power of two), activations are split hi + lo into
// two f16 rows, accumulation is f32: the only rounding left is the f32 -> (hi, lo) split.
#include "tc5.cuh"

#include <math.h>
#include <string.h>

// ------------------------------------------------------------------ route

// One token by one warp. n_expert <= 256.
__device__ __forceinline__ void moe_route_token(const float *__restrict__ logits, const float *__restrict__ router_bias,
                                                const float *__restrict__ sel_bias, int tok, int lane, int n_expert, int top_k,
                                                int norm, float scale, int32_t *sel, float *wt) {
    float lg[8], pr[8];
    double mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        lg[i] = e < n_expert ? logits[(size_t)tok * n_expert + e] + (router_bias ? router_bias[e] : 0.f) : -INFINITY;
        if (lg[i] == lg[i]) mx = fmax(mx, (double)lg[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    double ex[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        ex[i] = (lane + 32 * i < n_expert) ? exp((double)lg[i] - mx) : 0.0;
        sum += ex[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int i = 0; i < 8; i++) pr[i] = (float)(ex[i] / sum);   // a NaN logit stays a NaN score
    // the scores the SELECTION ranks: the gated scores plus the selection-only bias; the weights below
    // come from the unbiased scores (internal/oracle/moe.go:204-262)
    float rk[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        rk[i] = (sel_bias && e < n_expert) ? pr[i] + sel_bias[e] : pr[i];
    }

    // k rounds of "largest score, lowest index"; picked entries are retired
    bool taken[8] = {false, false, false, false, false, false, false, false};
    float wsum = 0.f;
    float mywt = 0.f;     // lane j keeps the j-th selected weight
    int mysel = -1;
    for (int j = 0; j < top_k; j++) {
        float best = -INFINITY, bw = 0.f;            // ranking score and the unbiased score that goes with it
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int e = lane + 32 * i;
            if (e < n_expert && !taken[i] && rk[i] == rk[i] && (bi == 0x7fffffff || rk[i] > best)) { best = rk[i]; bw = pr[i]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const float ow = __shfl_xor_sync(0xffffffffu, bw, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bw = ow; bi = oi; }
        }
        if (bi == 0x7fffffff) break;                 // nothing eligible is left
#pragma unroll
        for (int i = 0; i < 8; i++) if (lane + 32 * i == bi) taken[i] = true;
        wsum += bw;                                  // selection order, one addition at a time
        if (lane == j) { mywt = bw; mysel = bi; }
    }
    const float div = norm ? wsum + 1e-20f : 1.f;
    if (lane < top_k) {
        float w = mywt / div;
        if (scale != 0.f && scale != 1.f) w *= scale;
        sel[(size_t)tok * top_k + lane] = mysel;
        wt[(size_t)tok * top_k + lane] = w;
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float *__restrict__ logits, const float *__restrict__ router_bias,
                 const float *__restrict__ sel_bias, int ntok, int n_expert, int top_k, int norm, float scale,
                 int32_t *__restrict__ sel, float *__restrict__ wt) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tok = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (tok >= ntok) return;
    moe_route_token(logits, router_bias, sel_bias, tok, lane, n_expert, top_k, norm, scale, sel, wt);
}

// ------------------------------------------------------------------- sort

// Stable counting sort of the pairs by expert, one CTA of 256 threads.
//   cnt[e], off[e] (exclusive), perm_tok[pos] = token of sorted position pos,
//   pos_of[tok * k + slot] = sorted position of that pair (or -1 for an unfilled slot)
// Counts by shared-memory atomics; placement by ONE warp walking the pairs 32 at a time in
// order, ranking equal ids inside a chunk with __match_any_sync, so positions keep token order.
#define MOE_SORT_STAGE 4096
__device__ __forceinline__ void moe_sort_cta(const int32_t *sel, int npairs, int top_k, int n_expert, int *__restrict__ cnt,
                                             int *__restrict__ off, int *__restrict__ perm_tok, int *__restrict__ pos_of) {
    __shared__ int s_cnt[256], s_base[257];
    // the ids of a batch of up to MOE_SORT_STAGE pairs stay in shared memory for the placement walk below: read from
    // global memory there, each of its 32-pair steps waited for its own L2 round trip (10 of the kernel's 12 us)
    __shared__ int s_sel[MOE_SORT_STAGE];
    const bool staged = npairs <= MOE_SORT_STAGE;
    const int tid = threadIdx.x;
    for (int i = tid; i < 256; i += blockDim.x) s_cnt[i] = 0;
    __syncthreads();
    for (int i = tid; i < npairs; i += blockDim.x) {
        const int id = __ldcg(sel + i);
        if (staged) s_sel[i] = id;
        if (id >= 0 && id < n_expert) atomicAdd(&s_cnt[id], 1);
        else pos_of[i] = -1;
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int i = 0; i < n_expert; i++) { s_base[i] = acc; acc += s_cnt[i]; }
        s_base[n_expert] = acc;
    }
    __syncthreads();
    for (int i = tid; i <= n_expert; i += blockDim.x) off[i] = s_base[i];
    for (int i = tid; i < n_expert; i += blockDim.x) cnt[i] = s_cnt[i];
    __syncthreads();                                   // off[] is read back below by every thread
    if (tid < 32) {
        // one generic pointer, shared or global: a per-step choice between the two would issue the global load as well
        const int *src = staged ? static_cast<const int *>(s_sel) : sel;
        for (int c = 0; c < npairs; c += 32) {
            const int i = c + tid;
            const int id = i < npairs ? src[i] : -1;
            const bool ok = id >= 0 && id < n_expert;
            const unsigned same = __match_any_sync(0xffffffffu, ok ? id : -1 - tid);   // invalid ids match nobody
            if (ok) {
                const int rank = __popc(same & ((1u << tid) - 1));
                const int p = s_base[id] + rank;
                perm_tok[p] = i / top_k;
                pos_of[i] = p;
            }
            __syncwarp();
            if (ok && (same & ((1u << tid) - 1)) == 0) s_base[id] += __popc(same);     // the chunk's first lane of this id
            __syncwarp();
        }
    }
    // Pairs without an expert (a row of NaN logits fills fewer than top_k slots; an id out of range) leave the last
    // positions of the list unused: name token 0 there, so that the gather that walks all npairs positions reads a
    // real row (nothing consumes those positions).
    for (int i = off[n_expert] + tid; i < npairs; i += blockDim.x) perm_tok[i] = 0;
}

__global__ void __launch_bounds__(256)
moe_sort_kernel(const int32_t *__restrict__ sel, int npairs, int top_k, int n_expert, int *__restrict__ cnt,
                int *__restrict__ off, int *__restrict__ perm_tok, int *__restrict__ pos_of) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    moe_sort_cta(sel, npairs, top_k, n_expert, cnt, off, perm_tok, pos_of);
}

// ---------------------------------------------------------------- combine

// out[tok][d] += sum over the token's experts, ascending id, of wt * y[pos][d].
__global__ void __launch_bounds__(256)
moe_combine_kernel(float *__restrict__ out, const float *__restrict__ y, const int32_t *__restrict__ sel,
                   const float *__restrict__ wt, const int *__restrict__ pos_of, int ntok, int top_k, int hidden) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int tok = blockIdx.x;
    __shared__ int s_pos[32];
    __shared__ float s_w[32];
    __shared__ int s_id0[32], s_pos0[32];
    __shared__ float s_w0[32];
    if (threadIdx.x < top_k) {          // the token's slots, all loads in flight at once
        s_id0[threadIdx.x] = sel[(size_t)tok * top_k + threadIdx.x];
        s_pos0[threadIdx.x] = pos_of[(size_t)tok * top_k + threadIdx.x];
        s_w0[threadIdx.x] = wt[(size_t)tok * top_k + threadIdx.x];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // insertion sort of the slots by expert id (top_k <= 32)
        int ids[32], n = 0;
        for (int j = 0; j < top_k; j++) {
            const int id = s_id0[j];
            if (id < 0) continue;
            int q = n++;
            while (q > 0 && ids[q - 1] > id) { ids[q] = ids[q - 1]; s_pos[q] = s_pos[q - 1]; s_w[q] = s_w[q - 1]; q--; }
            ids[q] = id; s_pos[q] = s_pos0[j]; s_w[q] = s_w0[j];
        }
        for (int j = n; j < 32; j++) s_pos[j] = -1;
    }
    __syncthreads();
    int n = 0;
    while (n < top_k && s_pos[n] >= 0) n++;
    float4 *o4 = reinterpret_cast<float4 *>(out + (size_t)tok * hidden);   // hidden is a multiple of 64
    for (int d = threadIdx.x; d < hidden / 4; d += blockDim.x) {
        float4 acc = o4[d];
        for (int j = 0; j < n; j++) {                                       // ascending expert id
            const float4 v = __ldg(reinterpret_cast<const float4 *>(y + (size_t)s_pos[j] * hidden) + d);
            const float w = s_w[j];
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        o4[d] = acc;
    }
}

// ------------------------------------------------------------ grouped GEMM

#define MOE_PF 4   // k-blocks of raw codes a dequant thread keeps in flight
#define MOE_KH 2   // 64-wide k-blocks per shared-memory stage
#define MOE_ISSUERS 2                                    // MMA issuer warps: 5 (first 128 rows of a tile), 14 (second 128)
#define MOE_THREADS (TC5_THREADS + 32 * (MOE_ISSUERS - 1))
struct moe_gemm_params {
    int mode;                    // 0: gate|up -> act(g, u);  1: down
    int n_expert, rows, k;       // rows, k of ONE expert matrix (mode 0: ffn x hidden; mode 1: hidden x ffn)
    int row_tiles, max_tok_tiles, split, act;
    const uint8_t *c0, *c1;      // code planes [E][rows][k/32][16]: mode 0 gate, up; mode 1 down, -
    const uint8_t *e0, *e1;      // e8m0 planes [E][rows][e_stride]
    int e_stride;
    const float *b0, *b1;        // biases [E][rows] or NULL
    const int *cnt, *off;        // pairs per expert, exclusive offsets (device)
    const float *inv_scale;      // [npairs] scale of each gathered activation row
    float *outp;                 // [npairs][rows] f32
    const int *out_rowmap;       // mode 1: row of outp that sorted position pos is written to (NULL: pos)
    int npairs;
    int bitdq;                   // every block scale byte is in [104, 128]: the conversion-free dequant applies
    int *status;
    const uint8_t *sfb;          // block-scaled arm: ue8m0 scales of the activation rows, [npairs][sfb_stride]
    int sfb_stride;              // a multiple of 4: one 32-bit word per 128-element stage
};

// Two e2m1 codes of one byte -> two f16 (low nibble first).
__device__ __forceinline__ uint32_t e2m1x2_to_h2(uint32_t byte) {
    uint32_t r;
    asm("{\n\t.reg .b8 lo, hi;\n\t.reg .b16 t;\n\t"
        "cvt.u16.u32 t, %1;\n\t"
        "mov.b16 {lo, hi}, t;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, lo;\n\t}"
        : "=r"(r)
        : "r"(byte));
    return r;
}
// 2^(e - 127) as an f16 pair (e in [104, 140]: exact, subnormal below 113).
__device__ __forceinline__ uint32_t e8m0_to_h2(uint32_t e) {
    e = min(max(e, 104u), 140u);   // only an all-zero block can be outside (the upload checked the others)
    const uint32_t h = e >= 113 ? (e - 112) << 10 : 1u << (e - 103);
    return h | (h << 16);
}
__device__ __forceinline__ float moe_act(int kind, float g, float u) {
    if (kind == JL_ACT_SWIGLU_OAI) {   // jit/gpu/kernels/actkind.go:13-39
        const float x = fminf(g, 7.f), y = fmaxf(fminf(u, 7.f), -7.f);
        return __fdividef(x, 1.f + __expf(-1.702f * x)) * (y + 1.f);
    }
    // SiLU gate. The fast exponential and division (a few ulp) on purpose: the four epilogue warps share their
    // schedulers with the MMA issuers, and with expf and an IEEE division the drain of a unit cost ~35 instructions
    // per element (37 us of a 172 us layer, measured by leaving the drain out).
    return __fdividef(g, 1.f + __expf(-g)) * u;
}

#include "moe_bs.cuh"

template <int NT, int SA, int SB>
struct moe_smem {
    static constexpr int ACC_COLS = TC5_MS * NT;
    static constexpr int ACC_BUFS = ACC_COLS * 2 <= 512 ? 2 : 1;
    // A stage holds MOE_KH 64-wide halves of k (each a 128-byte swizzle atom wide): one barrier handshake per 128 k
    static constexpr int BH_BYTES = NT * TC5_KB * 2;            // one half of an activation stage
    static constexpr int B_BYTES = MOE_KH * BH_BYTES;
    static constexpr int AH_BYTES = TC5_MS * TC5_A_BYTES;       // one half of a weight stage
    static constexpr int A_BYTES = MOE_KH * AH_BYTES;
    static constexpr int A_OFS = 0;
    static constexpr int B_OFS = SA * A_BYTES;
    static constexpr int BAR_OFS = B_OFS + SB * B_BYTES;
    static constexpr int NBARS = 2 * SA + 2 * SB + 4;
    static constexpr int MISC_OFS = BAR_OFS + NBARS * 8;
    static constexpr int CNT_OFS = MISC_OFS + 16;               // the experts' list offsets: 257 ints (a length is a difference)
    static constexpr int TOTAL = CNT_OFS + 1040 + 1024;         // kept small on purpose: see the note at moe_launch
};

// Same roles as the dense prefill GEMM (gemm_tc5.cu): warps 0..3 epilogue, 4 TMA producer
// (activation tiles of the expert's token list), 5 MMA issuer, 6..13 dequant (thread r owns tile
// row r). A work unit is (expert, row tile, token tile); units past an expert's list exit.
template <int NT, int SA, int SB>
__global__ void __launch_bounds__(MOE_THREADS, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const moe_gemm_params p) {
    using L = moe_smem<NT, SA, SB>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::BAR_OFS);
    uint64_t *a_full = bars, *a_empty = bars + SA, *b_full = bars + 2 * SA, *b_empty = b_full + SB;
    uint64_t *acc_full = b_empty + SB, *acc_empty = acc_full + 2;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::MISC_OFS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::MISC_OFS + 4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n64 = p.k / TC5_KB;                       // 64-wide k-blocks of a row
    const int nkb = (n64 + MOE_KH - 1) / MOE_KH;        // stages (the last one may hold a single half)
    const int mult = p.split ? 2 : 1;
    int *s_off = reinterpret_cast<int *>(smem + L::CNT_OFS);

    if (tid == 0) {
        for (int s = 0; s < SA; s++) { mbar_init(smem_u32(a_full + s), TC5_DQ_THREADS / 32); mbar_init(smem_u32(a_empty + s), MOE_ISSUERS); }
        for (int s = 0; s < SB; s++) { mbar_init(smem_u32(b_full + s), 1); mbar_init(smem_u32(b_empty + s), MOE_ISSUERS); }
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(acc_full + i), MOE_ISSUERS); mbar_init(smem_u32(acc_empty + i), 4); }
        abort_flag[0] = 0;
        abort_flag[1] = p.status[1];                                // the wait limit, read once
        mbar_init_fence();
    }
    if (warp == 5) tc5_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), L::ACC_COLS * L::ACC_BUFS);
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");   // token lists and activation rows come from the kernels in front
    // list lengths and offsets once into shared memory (every role asks for them at every unit, live or not); the walk
    // over the units ends at the longest list's last token tile
    if (tid <= p.n_expert) s_off[tid] = p.off[tid];      // off[n_expert] = the number of listed pairs
    __syncthreads();
    int longest = 0;
    for (int e = 0; e < p.n_expert; e++) longest = max(longest, (s_off[e + 1] - s_off[e]));
    const int nunits = p.n_expert * p.row_tiles * min(p.max_tok_tiles, (longest * mult + NT - 1) / NT);

    // unit -> (expert, row tile, token tile); live iff the token tile starts inside the expert's list
#define MOE_UNIT(u)                                                                   \
    const int tt = (u) / (p.n_expert * p.row_tiles);   /* slowest: the live units (first token    \
                                                          tiles) are contiguous, spread over CTAs */ \
    const int e = ((u) / p.row_tiles) % p.n_expert, rt = (u) % p.row_tiles;           \
    const int m_eff = (s_off[e + 1] - s_off[e]) * mult, col0 = s_off[e] * mult + tt * NT;              \
    const bool live = tt * NT < m_eff;                                                \
    (void)rt; (void)col0; (void)m_eff

    if (warp == 4) {
        if (lane == 0) {
            uint32_t kb_it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
                MOE_UNIT(u);
                if (!live) continue;
                for (int kb = 0; kb < nkb && ok; kb++, kb_it++) {
                    const uint32_t s = kb_it % SB, ph = (kb_it / SB) & 1;
                    if (kb_it >= (uint32_t)SB) ok = tc5_wait(smem_u32(b_empty + s), ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(smem_u32(b_full + s), L::B_BYTES);      // a half beyond k arrives as zeros
#pragma unroll
                    for (int h = 0; h < MOE_KH; h++)
                        tma_load_2d(sbase + L::B_OFS + s * L::B_BYTES + h * L::BH_BYTES, &xmap, (kb * MOE_KH + h) * TC5_KB, col0,
                                    smem_u32(b_full + s));
                }
            }
        }
    } else if (warp == 5 || warp == TC5_THREADS / 32) {
        // ---- MMA issuers. Each takes one 128-row operand of every stage (its own accumulators), so that one warp's
        //      barrier waits and commits pass while the other's MMAs execute. The whole warp runs the loop and an
        //      elected lane issues: what the instructions take is then the same in every lane (values from memory by
        //      a broadcast). The next stage's barriers are probed before this stage's MMAs go out.
        constexpr uint32_t idesc = tc5_idesc(TC5_M, NT);
        const int wu = tc5_uniform(warp);
        const int ms_lo = MOE_ISSUERS == 2 ? (wu == 5 ? 0 : 1) : 0, ms_hi = MOE_ISSUERS == 2 ? ms_lo + 1 : TC5_MS;
        const bool leader = tc5_elect();
        const uint32_t tbase = (uint32_t)tc5_uniform((int)tmem_base), sb_u = (uint32_t)tc5_uniform((int)sbase);
        const uint32_t bars_u = sb_u + L::BAR_OFS;   // a_full +0, a_empty +SA, b_full +2SA, b_empty +2SA+SB, acc_full +2SA+2SB
        uint32_t kb_it = 0, unit_it = 0;
        bool ok = true, ready_a = false, ready_b = false;
        for (int u = blockIdx.x; u < nunits && ok; u += gridDim.x) {
            if (tc5_uniform(*abort_flag)) break;
            const int e = (u / p.row_tiles) % p.n_expert, tt = u / (p.n_expert * p.row_tiles);
            if (tt * NT >= tc5_uniform((s_off[e + 1] - s_off[e])) * mult) continue;                   // not a live unit
            const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
            if (unit_it >= (uint32_t)L::ACC_BUFS)
                ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * (2 * SA + 2 * SB + 2 + ab), aph ^ 1, abort_flag));
            if (!ok) break;
            tc5_fence_after();
            const uint32_t d_tmem = tbase + ab * L::ACC_COLS;
            for (int kb = 0; kb < nkb && ok; kb++, kb_it++) {
                const uint32_t sa = kb_it % SA, pha = (kb_it / SA) & 1, s = kb_it % SB, ph = (kb_it / SB) & 1;
                if (!__all_sync(0xffffffffu, ready_a)) ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * sa, pha, abort_flag));
                if (ok && !__all_sync(0xffffffffu, ready_b))
                    ok = __all_sync(0xffffffffu, tc5_wait(bars_u + 8 * (2 * SA + s), ph, abort_flag));
                if (!ok) break;
                tc5_fence_after();
                ready_a = mbar_test_wait(bars_u + 8 * ((kb_it + 1) % SA), ((kb_it + 1) / SA) & 1);
                ready_b = mbar_test_wait(bars_u + 8 * (2 * SA + (kb_it + 1) % SB), ((kb_it + 1) / SB) & 1);
                if (leader) {
#pragma unroll
                    for (int h = 0; h < MOE_KH; h++) {
                        if (kb * MOE_KH + h >= n64) break;
                        const uint64_t bdesc = tc5_smem_desc(sb_u + L::B_OFS + s * L::B_BYTES + h * L::BH_BYTES);
                        for (int ms = ms_lo; ms < ms_hi; ms++) {
                            const uint64_t adesc = tc5_smem_desc(sb_u + L::A_OFS + sa * L::A_BYTES + h * L::AH_BYTES + ms * TC5_A_BYTES);
#pragma unroll
                            for (int j = 0; j < TC5_KB / 16; j++)
                                tc5_mma_f16(d_tmem + ms * NT, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | h | j) != 0);
                        }
                    }
                    tc5_commit(bars_u + 8 * (SA + sa));
                    tc5_commit(bars_u + 8 * (2 * SA + SB + s));
                }
            }
            if (!ok) break;
            if (leader) tc5_commit(bars_u + 8 * (2 * SA + 2 * SB + ab));
            unit_it++;
        }
    } else if (warp >= 6 && warp < TC5_THREADS / 32) {
        // ---- dequant: thread r owns tile row r. mode 0: rows 0..127 gate, 128..255 up (same row index);
        //      mode 1: 256 consecutive rows of down.
        const int r = tid - 192;
        const uint32_t swz = (uint32_t)(r & 7);
        const int a_row_ofs = (r >> 7) * TC5_A_BYTES + (r & 127) * 128;
        const int nblk = p.k / 32;
        uint32_t kb_it = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < nunits && ok && !*abort_flag; u += gridDim.x) {
            MOE_UNIT(u);
            if (!live) continue;
            const bool second = p.mode == 0 && r >= 128;
            const int row = p.mode == 0 ? min(rt * TC5_M + (r & 127), p.rows - 1) : min(rt * TC5_ROWS + r, p.rows - 1);
            const size_t grow = (size_t)e * p.rows + row;
            const uint8_t *codes = (second ? p.c1 : p.c0) + grow * nblk * 16;
            const uint8_t *ebytes = (second ? p.e1 : p.e0) + grow * p.e_stride;
            // raw codes run MOE_PF k-blocks (64 k = 32 B of the row each) ahead of their use, in registers: slot j is
            // refilled with k-block kb+MOE_PF the moment k-block kb has been copied out of it
            uint4 q[2 * MOE_PF];
            uint32_t ec[MOE_PF];
#pragma unroll
            for (int j = 0; j < MOE_PF; j++) {
                q[2 * j] = q[2 * j + 1] = make_uint4(0, 0, 0, 0); ec[j] = 0x7F7F;
                if (j < n64) {
                    q[2 * j] = ldg_nc16(codes + (size_t)j * 32);
                    q[2 * j + 1] = ldg_nc16(codes + (size_t)j * 32 + 16);
                    ec[j] = *reinterpret_cast<const uint16_t *>(ebytes + 2 * j);
                }
            }
            static_assert(MOE_PF % MOE_KH == 0, "a stage's halves are consecutive slots of the prefetch ring");
            for (int kb0 = 0; kb0 < n64 && ok; kb0 += MOE_PF) {
#pragma unroll
              for (int j = 0; j < MOE_PF; j++) {
                const int kb = kb0 + j;                 // 64-wide k-block; half j % MOE_KH of stage kb / MOE_KH
                if (kb >= n64) break;
                const int half = j % MOE_KH;
                const uint32_t s = kb_it % SA, ph = (kb_it / SA) & 1;
                const uint4 c0 = q[2 * j], c1 = q[2 * j + 1];
                const uint32_t e_lo = ec[j] & 0xFF, e_hi = ec[j] >> 8;
                if (half == 0 && kb_it >= (uint32_t)SA) ok = tc5_wait(smem_u32(a_empty + s), ph ^ 1, abort_flag);
                if (!ok) break;
                uint8_t *arow = smem + L::A_OFS + s * L::A_BYTES + half * L::AH_BYTES + a_row_ofs;
#pragma unroll
                for (int b = 0; b < 2; b++) {           // block b of the k-block: k 32b..32b+31
                    const uint4 cw = b ? c1 : c0;
                    const uint32_t eb = b ? e_hi : e_lo;
                    const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
                    uint32_t lo[8], hi[8];              // f16 pairs: elements 2i,2i+1 (low nibbles) and 16+2i,16+2i+1
                    if (p.bitdq) {
                        // An e2m1 code s|e1 e0|m IS the top of an f16 with exponent field e1 e0 and mantissa m...:
                        // high byte s<<7 | (e1 e0 m)<<1 reads as value * 2^-14, subnormals included (0, 0.5). One
                        // packed multiply by 2^14 * 2^(e-127) finishes the weight -- no conversion instruction,
                        // whose unit the eight dequant warps saturate.
                        // 2^(e - 113), e in [104, 128]: exponent field 6..30 (an all-zero block may carry any byte: clamp)
                        const uint32_t mh = (min(max(eb, 104u), 128u) - 98u) << 10;
                        const uint32_t mult = mh | (mh << 16);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const uint32_t v = w[q], vl = v << 4;
                            const uint32_t hh = ((v & 0x70707070u) >> 3) | (v & 0x80808080u);     // elements 16+4q..16+4q+3
                            const uint32_t hl = ((vl & 0x70707070u) >> 3) | (vl & 0x80808080u);   // elements 4q..4q+3
                            lo[2 * q] = hmul2u(__byte_perm(hl, 0u, 0x1404), mult);
                            lo[2 * q + 1] = hmul2u(__byte_perm(hl, 0u, 0x3424), mult);
                            hi[2 * q] = hmul2u(__byte_perm(hh, 0u, 0x1404), mult);
                            hi[2 * q + 1] = hmul2u(__byte_perm(hh, 0u, 0x3424), mult);
                        }
                    } else {
                        const uint32_t sc = e8m0_to_h2(eb);
#pragma unroll
                        for (int i = 0; i < 8; i++) {       // bytes 2i, 2i+1: byte j holds element j (low) and j+16 (high)
                            const uint32_t wv = w[i >> 1] >> (16 * (i & 1));
                            const uint32_t a = e2m1x2_to_h2(wv & 0xFF), bb = e2m1x2_to_h2((wv >> 8) & 0xFF);
                            lo[i] = hmul2u(__byte_perm(a, bb, 0x5410), sc);
                            hi[i] = hmul2u(__byte_perm(a, bb, 0x7632), sc);
                        }
                    }
                    // chunks 4b..4b+3: elements 0-7, 8-15 (low nibbles), 16-23, 24-31 (high nibbles)
                    *reinterpret_cast<uint4 *>(arow + (((uint32_t)(4 * b + 0) ^ swz) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    *reinterpret_cast<uint4 *>(arow + (((uint32_t)(4 * b + 1) ^ swz) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                    *reinterpret_cast<uint4 *>(arow + (((uint32_t)(4 * b + 2) ^ swz) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(arow + (((uint32_t)(4 * b + 3) ^ swz) << 4)) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                }
                if (half == MOE_KH - 1 || kb == n64 - 1) {     // the stage is complete (the last one may be short)
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(a_full + s));
                    kb_it++;
                }
                // The slot is refilled AFTER the fence: a proxy fence waits for the thread's loads in flight, so a
                // prefetch issued in front of it put a DRAM round trip into every stage.
                if (kb + MOE_PF < n64) {
                    q[2 * j] = ldg_nc16(codes + (size_t)(kb + MOE_PF) * 32);
                    q[2 * j + 1] = ldg_nc16(codes + (size_t)(kb + MOE_PF) * 32 + 16);
                    ec[j] = *reinterpret_cast<const uint16_t *>(ebytes + 2 * (kb + MOE_PF));
                }
              }
            }
        }
    } else {
        // ---- epilogue: warp w reads TMEM lanes 32w..32w+31 (tile rows), 32 token columns at a time
        uint32_t unit_it = 0;
        for (int u = blockIdx.x; u < nunits && !*abort_flag; u += gridDim.x) {
            MOE_UNIT(u);
            if (!live) continue;
            const uint32_t ab = unit_it % L::ACC_BUFS, aph = (unit_it / L::ACC_BUFS) & 1;
            if (!tc5_wait_relaxed(smem_u32(acc_full + ab), aph, abort_flag)) break;
            tc5_fence_after();
            const uint32_t tacc = tmem_base + ab * L::ACC_COLS + ((uint32_t)(warp * 32) << 16);
            const int pos_end = s_off[e] + (s_off[e + 1] - s_off[e]);
            const int nj = p.split ? 16 : 32;
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
                const int pos0 = (col0 + c0) / mult;
                const int mypos = pos0 + (p.split ? (lane & 15) : lane);
                const float myscale = mypos < pos_end ? __ldg(p.inv_scale + mypos) : 0.f;
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
                        if (j >= nj) break;
                        const int pos = pos0 + j;
                        const float sc = __shfl_sync(0xffffffffu, myscale, j);
                        const float g = (p.split ? __uint_as_float(vg[(2 * j) & 31]) + __uint_as_float(vg[(2 * j + 1) & 31])
                                                 : __uint_as_float(vg[j])) * sc + bg;
                        const float uu = (p.split ? __uint_as_float(vu[(2 * j) & 31]) + __uint_as_float(vu[(2 * j + 1) & 31])
                                                  : __uint_as_float(vu[j])) * sc + bu;
                        if (row < p.rows && pos < pos_end) p.outp[(size_t)pos * p.rows + row] = moe_act(p.act, g, uu);
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
                            if (j >= nj) break;
                            const int pos = pos0 + j;
                            const float sc = __shfl_sync(0xffffffffu, myscale, j);
                            const float y = (p.split ? __uint_as_float(v[(2 * j) & 31]) + __uint_as_float(v[(2 * j + 1) & 31])
                                                     : __uint_as_float(v[j])) * sc + bd;
                            if (row < p.rows && pos < pos_end)
                                p.outp[(size_t)(p.out_rowmap ? p.out_rowmap[pos] : pos) * p.rows + row] = y;
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
#undef MOE_UNIT
    tc5_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(p.status, 3);
    if (warp == 5) {
        tc5_fence_after();
        tc5_dealloc(tmem_base, L::ACC_COLS * L::ACC_BUFS);
    }
}

// --------------------------------------------------------------------- host

static size_t al256(size_t n) { return (n + 255) & ~(size_t)255; }

size_t jl_moe_scratch_bytes(int ntok, int n_expert, int top_k, int hidden, int ffn) {
    const size_t np = (size_t)ntok * top_k;
    return al256(np * 4) * 4 + al256((size_t)(n_expert + 1) * 4) * 2 +          // sel wt perm pos_of, cnt off
           al256(np * 2 * hidden * 2) + al256(np * 4) * 2 +                       // xs (hi/lo), two scale arrays
           al256(np * ffn * 4) + al256(np * 2 * ffn * 2) + al256(np * hidden * 4) + 4096;
}

template <int NT, int SA, int SB>
static int moe_launch(jl_ctx *ctx, const CUtensorMap &xmap, const moe_gemm_params &p, cudaStream_t s, int nattr,
                      cudaLaunchAttribute *at) {
    using L = moe_smem<NT, SA, SB>;
    static_assert(L::TOTAL <= 227 * 1024, "shared memory budget");
    // Measured: the <128,2,2> form sits just under a step of the shared-memory carve-out (with the per-CTA reserve,
    // 196 KB); 2 KB more shared memory move it over the step, the L1 the dequant warps' raw loads lean on shrinks,
    // and the layer goes from 347 to 447 us.
    static_assert(L::TOTAL + 1024 <= 196 * 1024, "stay under the 196 KB carve-out step: the raw loads need the L1 beside it");
    JL_CUDA(ctx, cudaFuncSetAttribute(moe_gemm_kernel<NT, SA, SB>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    const int units = p.n_expert * p.row_tiles * p.max_tok_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(units < ctx->sm_count ? units : ctx->sm_count); cfg.blockDim = dim3(MOE_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s; cfg.attrs = at; cfg.numAttrs = nattr;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, moe_gemm_kernel<NT, SA, SB>, xmap, p));
    ctx->st.launches++;
    return JL_OK;
}

// One grouped GEMM over the sorted activation rows `xs` ([npairs * mult][k] f16).
static int moe_grouped(jl_ctx *ctx, moe_gemm_params p, const __half *xs, int ntok, cudaStream_t s, int nattr,
                       cudaLaunchAttribute *at) {
    const int mult = p.split ? 2 : 1;
    const int nt = p.split ? 128 : 64;
    p.max_tok_tiles = (ntok * mult + nt - 1) / nt;
    CUtensorMap xmap;
    if (!jl_make_tmap_2d(&xmap, xs, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)p.k, (uint64_t)p.npairs * mult,
                         (uint64_t)p.k * 2, TC5_KB, nt, CU_TENSOR_MAP_SWIZZLE_128B))
        return jl_set_err(ctx, JL_DECLINED, "the driver refused a tensor map for the mixture's activations");
    // shallow rings: shared memory not taken is L1 for the dequant warps' raw-weight loads (5-deep A rings: 576 us
    // per layer against 348 us)
    // (a 2-deep activation ring for the first form, which puts it under the next lower carve-out step: 337 against 341 us)
    return p.split ? moe_launch<128, 2, 2>(ctx, xmap, p, s, nattr, at) : moe_launch<64, 2, 3>(ctx, xmap, p, s, nattr, at);
}

// The block-scaled arm's grouped GEMM over the sorted e4m3 activation rows `xq` ([npairs][k] bytes).
template <int NT, int T, int DIG>
static int moe_grouped_bs(jl_ctx *ctx, moe_gemm_params p, const uint8_t *xq, int ntok, cudaStream_t s, int nattr,
                          cudaLaunchAttribute *at) {
    constexpr int SA = BS_SA, SB = BS_SB;
    using L = moe_bs_smem<NT, SA, SB>;
    static_assert(L::TOTAL <= 227 * 1024, "shared memory budget");
    static_assert(DIG * T <= NT && T % 8 == 0, "a tile's digit columns fit the MMAs' N; digit planes start on a swizzle atom");
    p.max_tok_tiles = (ntok + T - 1) / T;
    p.split = 0;
    CUtensorMap xmap;     // the DIG digit planes of the e4m3 rows, one below the other; a box is one plane's T rows
    if (!jl_make_tmap_2d(&xmap, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)p.k, (uint64_t)p.npairs * DIG, (uint64_t)p.k, BS_KB, T,
                         CU_TENSOR_MAP_SWIZZLE_128B))
        return jl_set_err(ctx, JL_DECLINED, "the driver refused a tensor map for the mixture's e4m3 activations");
    // The weight planes as packed 4-bit tensors: 16 codes per 8 bytes in HBM, 16 bytes (8 of them a gap) in shared
    // memory. The inner extent has to be a multiple of 128 codes: a row of k codes is declared ceil(k / 128) * 128
    // long at its true pitch, so a row's last box runs into the first bytes of the next row (or the slack behind
    // the plane): codes the activation side multiplies by its own zero fill, in stages whose MMAs are not issued.
    const uint64_t kpad = (uint64_t)((p.k + BS_KB - 1) / BS_KB) * BS_KB, nrows_all = (uint64_t)p.n_expert * p.rows;
    CUtensorMap amap0, amap1;
    bool tma_a = p.k % 64 == 0 &&
                 jl_make_tmap_2d(&amap0, p.c0, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 1, kpad, nrows_all, (uint64_t)p.k / 2, BS_KB, TC5_M,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
    if (tma_a) tma_a = jl_make_tmap_2d(&amap1, p.c1 ? p.c1 : p.c0, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 1, kpad, nrows_all,
                                       (uint64_t)p.k / 2, BS_KB, TC5_M, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!tma_a) amap0 = amap1 = xmap;
    const int units = p.n_expert * p.row_tiles * p.max_tok_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(units < ctx->sm_count ? units : ctx->sm_count); cfg.blockDim = dim3(BS_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = s; cfg.attrs = at; cfg.numAttrs = nattr;
    if (tma_a) {
        JL_CUDA(ctx, cudaFuncSetAttribute(moe_gemm_bs_kernel<NT, T, DIG, SA, SB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, moe_gemm_bs_kernel<NT, T, DIG, SA, SB, true>, xmap, amap0, amap1, p));
    } else {
        JL_CUDA(ctx, cudaFuncSetAttribute(moe_gemm_bs_kernel<NT, T, DIG, SA, SB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, moe_gemm_bs_kernel<NT, T, DIG, SA, SB, false>, xmap, amap0, amap1, p));
    }
    ctx->st.launches++;
    ctx->moe_bs_tma = tma_a ? 1 : 0;
    return JL_OK;
}

// given_ids != NULL: no router and no combine -- row i goes through expert given_ids[i] and
// out_dev[i] = down(act(gate h_i, up h_i)) is WRITTEN in the caller's row order (the expert-parallel
// path: rows arrive from other ranks already routed). Otherwise the whole layer, ADDED into out_dev.
#ifdef MOE_EXP_SKIP_GEMM          // timing experiment: the layer without its two grouped GEMMs
#define MOE_EXP_GEMM(call) 0
#else
#define MOE_EXP_GEMM(call) (call)
#endif
static int moe_dev_locked(jl_ctx *ctx, float *out_dev, const void *h_dev, int h_dtype, const float *logits_dev, int ntok,
                          const jl_moe_desc *d, int32_t *sel_out, float *wt_out, cudaStream_t s,
                          const int32_t *given_ids = nullptr) {
    const jl_weight *wg = (const jl_weight *)d->gate, *wu = (const jl_weight *)d->up, *wd = (const jl_weight *)d->down;
    const int E = d->n_expert, K = given_ids ? 1 : d->top_k, H = d->hidden, F = d->ffn;
    if (!wg || !wu || !wd || d->type != JL_TYPE_MXFP4 || wg->type != JL_TYPE_MXFP4 || wu->type != JL_TYPE_MXFP4 ||
        wd->type != JL_TYPE_MXFP4)
        return jl_set_err(ctx, JL_DECLINED, "the mixture layer serves MXFP4 expert banks");
    if (E < 1 || E > 256 || K < 1 || K > 32 || K > E || H % 64 || F % 64 || ntok < 1)
        return jl_set_err(ctx, JL_DECLINED, "mixture shape not served: %d experts, top %d, hidden %d, ffn %d", E, K, H, F);
    if (wg->n_expert != E || wu->n_expert != E || wd->n_expert != E || wg->nrows != F || wg->k != H || wu->nrows != F ||
        wu->k != H || wd->nrows != H || wd->k != F)
        return jl_set_err(ctx, JL_EINVAL, "expert banks do not match the descriptor's shape");
    if (d->arm != JL_MOE_ARM_EXACT && d->arm != JL_MOE_ARM_BLOCK_SCALED && d->arm != JL_MOE_ARM_BLOCK_SCALED_X3)
        return jl_set_err(ctx, JL_EINVAL, "jl_moe_desc.arm %d is not a known arm", d->arm);
    if (d->arm != JL_MOE_ARM_EXACT && (H > BS_MAX_KB * BS_KB || F > BS_MAX_KB * BS_KB))
        return jl_set_err(ctx, JL_DECLINED, "the block-scaled arm serves hidden and ffn up to %d", BS_MAX_KB * BS_KB);
    if (d->arm == JL_MOE_ARM_EXACT &&
        (wg->emin < 104 || wg->emax > 140 || wu->emin < 104 || wu->emax > 140 || wd->emin < 104 || wd->emax > 140))
        return jl_set_err(ctx, JL_DECLINED, "an MXFP4 block scale lies outside 2^-23..2^13, where f16 holds the weights exactly");
    const size_t need = jl_moe_scratch_bytes(ntok, E, K, H, F);
    if (ctx->scratch_cap < need)
        return jl_set_err(ctx, JL_ENOMEM, "mixture scratch holds %zu bytes, this layer needs %zu (jl_moe_reserve sizes it)",
                          ctx->scratch_cap, need);
    const int np = ntok * K;
    uint8_t *sp = (uint8_t *)ctx->scratch;
    auto take = [&](size_t n) { uint8_t *r = sp; sp += al256(n); return r; };
    int32_t *sel = (int32_t *)take((size_t)np * 4);
    float *wt = (float *)take((size_t)np * 4);
    int *perm = (int *)take((size_t)np * 4), *pos_of = (int *)take((size_t)np * 4);
    int *cnt = (int *)take((size_t)(E + 1) * 4), *off = (int *)take((size_t)(E + 1) * 4);
    __half *xs = (__half *)take((size_t)np * 2 * H * 2);
    float *xs_scale = (float *)take((size_t)np * 4), *as_scale = (float *)take((size_t)np * 4);
    float *act = (float *)take((size_t)np * F * 4);
    __half *as = (__half *)take((size_t)np * 2 * F * 2);
    float *y = (float *)take((size_t)np * H * 4);
    if (sel_out) sel = sel_out;
    if (wt_out) wt = wt_out;
    if (given_ids) sel = const_cast<int32_t *>(given_ids);

    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    const int nattr = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    auto cfg_of = [&](dim3 g, dim3 b) { cudaLaunchConfig_t c = {}; c.gridDim = g; c.blockDim = b; c.stream = s; c.attrs = at; c.numAttrs = nattr; return c; };
    {
        // (Router and sort as ONE launch were built twice and measured slower: a single CTA routing all tokens, +65 us
        // per layer -- the f64 softmax of 256 tokens on one SM; and the router's last CTA, by ticket, sorting, +7 us.
        // With programmatic dependent launch the boundary between the two costs less than either fusion.)
        cudaLaunchConfig_t c = cfg_of(dim3((ntok + 3) / 4), dim3(128));
        if (!given_ids) {
            JL_CUDA(ctx, cudaLaunchKernelEx(&c, moe_route_kernel, logits_dev, d->router_bias, d->sel_bias, ntok, E, K, d->norm, d->scale, sel, wt));
            ctx->st.launches++;
        }
        c = cfg_of(dim3(1), dim3(256));
        JL_CUDA(ctx, cudaLaunchKernelEx(&c, moe_sort_kernel, (const int32_t *)sel, np, K, E, cnt, off, perm, pos_of));
        ctx->st.launches++;
    }
    if (d->arm != JL_MOE_ARM_EXACT) {
        // The block-scaled arms: activations to e4m3 + ue8m0 per 32 (twice: the routed rows, then the gated
        // intermediates), one digit or three, weights and their scales as they are. The e4m3 planes and scale rows
        // live where the exact arm keeps its f16 rows (4 bytes per element there: room for three planes and the scales).
        // Digits: one for the one-digit arm. The parity arm takes three (12 significant bits), except for bf16 input rows,
        // whose 8 significant bits two digits hold (the second digit is an integer of at most 8 units of the first
        // one's last place; only an element below ~2^-10 of its block's largest loses bits, to e4m3's subnormal
        // step: under 2^-17 of the block's largest): 64 tokens per tile instead of 40, so that no expert of the 256-token batch needs a
        // second pass over its weights. The gated intermediates are f32: three.
        const int ndig2 = d->arm == JL_MOE_ARM_BLOCK_SCALED_X3 ? 3 : 1;
        const int ndig1 = ndig2 == 3 && h_dtype == JL_DT_BF16 ? 2 : ndig2;
        const int sfs1 = (H + BS_KB - 1) / BS_KB * 4, sfs2 = (F + BS_KB - 1) / BS_KB * 4;
        uint8_t *q1 = (uint8_t *)xs, *sf1 = q1 + (size_t)ndig1 * np * H;
        uint8_t *q2 = (uint8_t *)as, *sf2 = q2 + (size_t)ndig2 * np * F;
        const int src_rows = given_ids ? ntok : ntok;
        auto grouped = [&](const moe_gemm_params &pp, const uint8_t *xq, int ndig) {
            return ndig == 3   ? moe_grouped_bs<128, 40, 3>(ctx, pp, xq, ntok, s, nattr, at)
                   : ndig == 2 ? moe_grouped_bs<128, 64, 2>(ctx, pp, xq, ntok, s, nattr, at)
                               : moe_grouped_bs<64, 64, 1>(ctx, pp, xq, ntok, s, nattr, at);
        };
        cudaLaunchConfig_t c = cfg_of(dim3(np), dim3(256));
        JL_CUDA(ctx, cudaLaunchKernelEx(&c, act_to_mx8_kernel, h_dev, h_dtype, q1, sf1, H, sfs1, (const int *)perm, src_rows, ndig1,
                                        (size_t)np * H));
        ctx->st.launches++;
        moe_gemm_params p = {};
        p.n_expert = E; p.cnt = cnt; p.off = off; p.npairs = np; p.status = ctx->dev_status; p.act = d->act;
        p.mode = 0; p.rows = F; p.k = H; p.row_tiles = (F + TC5_M - 1) / TC5_M;
        p.c0 = wg->data; p.c1 = wu->data; p.e0 = wg->scales; p.e1 = wu->scales; p.e_stride = wg->scale_stride;
        p.b0 = d->gate_bias; p.b1 = d->up_bias; p.outp = act; p.sfb = sf1; p.sfb_stride = sfs1;
        int rc = MOE_EXP_GEMM(grouped(p, q1, ndig1));
        if (rc) return rc;
        c = cfg_of(dim3(np), dim3(256));
        JL_CUDA(ctx, cudaLaunchKernelEx(&c, act_to_mx8_kernel, (const void *)act, (int)JL_DT_F32, q2, sf2, F, sfs2, (const int *)nullptr, 0,
                                        ndig2, (size_t)np * F));
        ctx->st.launches++;
        p.mode = 1; p.rows = H; p.k = F; p.row_tiles = (H + TC5_ROWS - 1) / TC5_ROWS;
        p.c0 = wd->data; p.c1 = nullptr; p.e0 = wd->scales; p.e1 = nullptr; p.e_stride = wd->scale_stride;
        p.b0 = d->down_bias; p.b1 = nullptr; p.outp = y; p.sfb = sf2; p.sfb_stride = sfs2;
        if (given_ids) { p.outp = out_dev; p.out_rowmap = perm; }
        if ((rc = MOE_EXP_GEMM(grouped(p, q2, ndig2)))) return rc;
        if (!given_ids) {
            c = cfg_of(dim3(ntok), dim3(256));
            JL_CUDA(ctx, cudaLaunchKernelEx(&c, moe_combine_kernel, out_dev, (const float *)y, (const int32_t *)sel, (const float *)wt,
                                            (const int *)pos_of, ntok, K, H));
            ctx->st.launches++;
        }
        JL_CUDA(ctx, cudaGetLastError());
        return JL_OK;
    }
    const int hsplit = h_dtype == JL_DT_F32 ? 1 : 0;
    {
        cudaLaunchConfig_t c = cfg_of(dim3(np), dim3(256));
        JL_CUDA(ctx, cudaLaunchKernelEx(&c, act_to_f16_kernel, h_dev, h_dtype, xs, xs_scale, H, hsplit, (const int *)perm, ntok));
        ctx->st.launches++;
    }
    moe_gemm_params p = {};
    p.n_expert = E; p.cnt = cnt; p.off = off; p.npairs = np; p.status = ctx->dev_status; p.act = d->act;
    p.bitdq = wg->emax <= 128 && wu->emax <= 128;
    // gate | up -> act
    p.mode = 0; p.rows = F; p.k = H; p.row_tiles = (F + TC5_M - 1) / TC5_M; p.split = hsplit;
    p.c0 = wg->data; p.c1 = wu->data; p.e0 = wg->scales; p.e1 = wu->scales; p.e_stride = wg->scale_stride;
    p.b0 = d->gate_bias; p.b1 = d->up_bias; p.inv_scale = xs_scale; p.outp = act;
    int rc = MOE_EXP_GEMM(moe_grouped(ctx, p, xs, ntok, s, nattr, at));
    if (rc) return rc;
    {
        cudaLaunchConfig_t c = cfg_of(dim3(np), dim3(256));
        JL_CUDA(ctx, cudaLaunchKernelEx(&c, act_to_f16_kernel, (const void *)act, (int)JL_DT_F32, as, as_scale, F, 1, (const int *)nullptr, 0));
        ctx->st.launches++;
    }
    // down
    p.mode = 1; p.rows = H; p.k = F; p.row_tiles = (H + TC5_ROWS - 1) / TC5_ROWS; p.split = 1;
    p.bitdq = wd->emax <= 128;
    p.c0 = wd->data; p.c1 = nullptr; p.e0 = wd->scales; p.e1 = nullptr; p.e_stride = wd->scale_stride;
    p.b0 = d->down_bias; p.b1 = nullptr; p.inv_scale = as_scale; p.outp = y;
    if (given_ids) { p.outp = out_dev; p.out_rowmap = perm; }   // top_k = 1: perm[pos] is the caller's row
    if ((rc = MOE_EXP_GEMM(moe_grouped(ctx, p, as, ntok, s, nattr, at)))) return rc;
    if (!given_ids) {
        cudaLaunchConfig_t c = cfg_of(dim3(ntok), dim3(256));
        JL_CUDA(ctx, cudaLaunchKernelEx(&c, moe_combine_kernel, out_dev, (const float *)y, (const int32_t *)sel, (const float *)wt,
                                        (const int *)pos_of, ntok, K, H));
        ctx->st.launches++;
    }
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}

// jl_moe_desc grew by a field (sel_bias): a caller built against the shorter struct says so in struct_size.
static size_t desc_size(const jl_moe_desc *d) {
    return d->struct_size >= 64 && d->struct_size < sizeof(jl_moe_desc) ? d->struct_size : sizeof(jl_moe_desc);
}
// The caller's descriptor as the current struct (fields it does not know are zero).
static jl_moe_desc desc_local(const jl_moe_desc *d) {
    jl_moe_desc out = {};
    memcpy(&out, d, desc_size(d));
    return out;
}

// The host-pointer call's device staging: grows only, and only here.
static int moe_grow_stage(jl_ctx *ctx, size_t need) {
    if (ctx->moe_stage_cap >= need) return JL_OK;
    cudaStreamSynchronize(ctx->stream);
    if (ctx->moe_stage) { cudaFree(ctx->moe_stage); ctx->moe_stage = nullptr; ctx->moe_stage_cap = 0; }
    cudaError_t e = cudaMalloc(&ctx->moe_stage, need);
    if (e != cudaSuccess) { cudaGetLastError(); return jl_set_err(ctx, JL_ENOMEM, "cudaMalloc(%zu): %s", need, cudaGetErrorString(e)); }
    ctx->moe_stage_cap = need;
    return JL_OK;
}

#ifdef BS_EXP_TRACE
JL_EXPORT int jl_exp_bs_trace(long long *host) { return (int)cudaMemcpyFromSymbol(host, bs_trace, sizeof(bs_trace)); }
JL_EXPORT int jl_exp_bs_cta(unsigned long long *host) { return (int)cudaMemcpyFromSymbol(host, bs_cta_t, sizeof(bs_cta_t)); }
#endif
JL_EXPORT int jl_moe_bs_weights_by_tma(jl_ctx *ctx) { return ctx ? ctx->moe_bs_tma : 0; }

JL_EXPORT int jl_moe_reserve(jl_ctx *ctx, int ntok, int n_expert, int top_k, int hidden, int ffn) {
    if (!ctx || ntok < 1 || n_expert < 1 || top_k < 1 || hidden < 1 || ffn < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    // the host-pointer call's staging with every optional operand present
    const size_t np = (size_t)ntok * top_k;
    const size_t stage = al256((size_t)ntok * hidden * 4) * 2 + al256((size_t)ntok * n_expert * 4) + al256(np * 4) * 2 +
                         al256((size_t)n_expert * ffn * 4) * 2 + al256((size_t)n_expert * hidden * 4) +
                         al256((size_t)n_expert * 4) * 2;
    int rc = moe_grow_stage(ctx, stage);
    if (rc) return rc;
    return jl_grow_scratch(ctx, jl_moe_scratch_bytes(ntok, n_expert, top_k, hidden, ffn));
}

JL_EXPORT int jl_moe_dev(jl_ctx *ctx, float *out_dev, const void *h_dev, int h_dtype, const float *logits_dev, int ntok,
                         const jl_moe_desc *desc, int32_t *sel_out_dev, float *wt_out_dev, void *stream) {
    if (!ctx || !out_dev || !h_dev || !logits_dev || !desc) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->unhealthy) return jl_set_err(ctx, JL_ECUDA, "context is unhealthy after an earlier CUDA error");
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    const jl_moe_desc dl = desc_local(desc);
    int rc = moe_dev_locked(ctx, out_dev, h_dev, h_dtype, logits_dev, ntok, &dl, sel_out_dev, wt_out_dev, (cudaStream_t)stream);
    if (rc == JL_OK) ctx->st.served++;
    return rc;
}

JL_EXPORT int jl_moe_route_dev(jl_ctx *ctx, const float *logits_dev, int ntok, const jl_moe_desc *desc,
                               int32_t *sel_out_dev, float *wt_out_dev, void *stream) {
    if (!ctx || !logits_dev || !desc || !sel_out_dev || !wt_out_dev || ntok < 1) return JL_EINVAL;
    if (desc->n_expert < 1 || desc->n_expert > 256 || desc->top_k < 1 || desc->top_k > 32 || desc->top_k > desc->n_expert)
        return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    const jl_moe_desc dl = desc_local(desc);
    moe_route_kernel<<<(ntok + 3) / 4, 128, 0, (cudaStream_t)stream>>>(logits_dev, dl.router_bias, dl.sel_bias, ntok,
                                                                     dl.n_expert, dl.top_k, dl.norm, dl.scale,
                                                                     sel_out_dev, wt_out_dev);
    ctx->st.launches++;
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}

JL_EXPORT int jl_moe_experts_dev(jl_ctx *ctx, float *y_dev, const void *h_dev, int h_dtype, const int32_t *expert_ids_dev,
                                 int nrows, const jl_moe_desc *desc, void *stream) {
    if (!ctx || !y_dev || !h_dev || !expert_ids_dev || !desc) return JL_EINVAL;
    if (nrows < 1) return JL_OK;
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->unhealthy) return jl_set_err(ctx, JL_ECUDA, "context is unhealthy after an earlier CUDA error");
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    const jl_moe_desc dl = desc_local(desc);
    int rc = moe_dev_locked(ctx, y_dev, h_dev, h_dtype, nullptr, nrows, &dl, nullptr, nullptr, (cudaStream_t)stream,
                            expert_ids_dev);
    if (rc == JL_OK) ctx->st.served++;
    return rc;
}

// Host buffers in and out; the banks are uploaded (and kept, keyed on their host address) on first use.
JL_EXPORT int jl_moe(jl_ctx *ctx, float *out, const void *h, int h_dtype, const float *logits, int ntok,
                     const jl_moe_desc *desc, int32_t *sel_out, float *wt_out) {
    if (!ctx || !out || !h || !logits || !desc) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->unhealthy) return jl_set_err(ctx, JL_ECUDA, "context is unhealthy after an earlier CUDA error");
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    const jl_moe_desc dcopy = desc_local(desc);
    desc = &dcopy;
    const int E = desc->n_expert, K = desc->top_k, H = desc->hidden, F = desc->ffn;
    if (desc->type != JL_TYPE_MXFP4 || E < 1 || K < 1 || H < 64 || F < 64 || H % 64 || F % 64 || ntok < 1)
        return jl_set_err(ctx, JL_DECLINED, "the mixture layer serves MXFP4 banks with hidden and ffn multiples of 64");
    jl_drain_graveyard(ctx);
    jl_weight *wg = nullptr, *wu = nullptr, *wd = nullptr;
    // the three banks stay pinned while they are fetched: fetching one never evicts another
    int rc = jl_resident_bank(ctx, desc->type, desc->gate, desc->gate_bytes, E, F, H, &wg);
    if (!rc) rc = jl_resident_bank(ctx, desc->type, desc->up, desc->up_bytes, E, F, H, &wu);
    if (!rc) rc = jl_resident_bank(ctx, desc->type, desc->down, desc->down_bytes, E, H, F, &wd);
    jl_resident_unpin(ctx);   // ctx->mu is held to the end of this call
    if (rc) return rc;
    if ((rc = jl_grow_scratch(ctx, jl_moe_scratch_bytes(ntok, E, K, H, F)))) return rc;

    const size_t hb = (size_t)ntok * H * (h_dtype == JL_DT_F32 ? 4 : 2), ob = (size_t)ntok * H * 4;
    const size_t np = (size_t)ntok * K;
    // one staging block of the context: h | logits | out | sel | wt | biases. It only grows (jl_moe_reserve
    // pre-sizes it), so a steady-state call allocates nothing.
    const size_t nb_g = desc->gate_bias ? (size_t)E * F * 4 : 0, nb_u = desc->up_bias ? (size_t)E * F * 4 : 0;
    const size_t nb_d = desc->down_bias ? (size_t)E * H * 4 : 0, nb_r = desc->router_bias ? (size_t)E * 4 : 0;
    const size_t nb_s = desc->sel_bias ? (size_t)E * 4 : 0;
    const size_t total = al256(hb) + al256((size_t)ntok * E * 4) + al256(ob) + al256(np * 4) * 2 + al256(nb_g) +
                         al256(nb_u) + al256(nb_d) + al256(nb_r) + al256(nb_s);
    if ((rc = moe_grow_stage(ctx, total))) return rc;
    uint8_t *sp = (uint8_t *)ctx->moe_stage;
    auto take = [&](size_t n) { uint8_t *r = sp; sp += al256(n); return r; };
    void *h_d = take(hb);
    float *lg_d = (float *)take((size_t)ntok * E * 4), *out_d = (float *)take(ob);
    int32_t *sel_d = (int32_t *)take(np * 4);
    float *wt_d = (float *)take(np * 4);
    float *bg = (float *)take(nb_g), *bu = (float *)take(nb_u), *bd = (float *)take(nb_d), *br = (float *)take(nb_r);
    float *bs = (float *)take(nb_s);
    cudaStream_t s = ctx->stream;
    cudaError_t ce = cudaMemcpyAsync(h_d, h, hb, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(lg_d, logits, (size_t)ntok * E * 4, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(out_d, out, ob, cudaMemcpyHostToDevice, s);   // the layer ADDS into out
    if (ce == cudaSuccess && nb_g) ce = cudaMemcpyAsync(bg, desc->gate_bias, nb_g, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess && nb_u) ce = cudaMemcpyAsync(bu, desc->up_bias, nb_u, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess && nb_d) ce = cudaMemcpyAsync(bd, desc->down_bias, nb_d, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess && nb_r) ce = cudaMemcpyAsync(br, desc->router_bias, nb_r, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess && nb_s) ce = cudaMemcpyAsync(bs, desc->sel_bias, nb_s, cudaMemcpyHostToDevice, s);
    rc = JL_OK;
    if (ce == cudaSuccess) {
        jl_moe_desc dd = *desc;
        dd.gate = wg; dd.up = wu; dd.down = wd;
        dd.gate_bias = nb_g ? bg : nullptr; dd.up_bias = nb_u ? bu : nullptr; dd.down_bias = nb_d ? bd : nullptr;
        dd.router_bias = nb_r ? br : nullptr; dd.sel_bias = nb_s ? bs : nullptr;
        rc = moe_dev_locked(ctx, out_d, h_d, h_dtype, lg_d, ntok, &dd, sel_d, wt_d, s);
    }
    if (ce == cudaSuccess && rc == JL_OK) ce = cudaMemcpyAsync(out, out_d, ob, cudaMemcpyDeviceToHost, s);
    if (ce == cudaSuccess && rc == JL_OK && sel_out) ce = cudaMemcpyAsync(sel_out, sel_d, np * 4, cudaMemcpyDeviceToHost, s);
    if (ce == cudaSuccess && rc == JL_OK && wt_out) ce = cudaMemcpyAsync(wt_out, wt_d, np * 4, cudaMemcpyDeviceToHost, s);
    if (ce != cudaSuccess) {
        cudaStreamSynchronize(s);
        ctx->unhealthy = true;
        return jl_set_err(ctx, JL_ECUDA, "mixture layer: %s", cudaGetErrorString(ce));
    }
    const int rs = jl_read_status(ctx, s);   // synchronises the stream
    if (rc) return rc;
    if (rs) return rs;
    ctx->st.served++;
    return JL_OK;
}
