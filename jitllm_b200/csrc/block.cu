// Whole decoder blocks as ONE persistent kernel per token: the reference's LayerDevice seam
// (engine/nn/device.go:1096-1176: PrepLayer uploads a block's weights, Layers runs blocks [lo, hi)
// as one submission without the residual stream leaving the device, an optional Head continues the
// same submission with the output norm and the vocabulary projection; EmbedDevice fills the
// residual row from a token id on the card, :1178-1191).
//
// A decode step at batch 1 is a chain of small dependent matvecs (Llama-3-8B: 9.4 .. 66 MB of
// Q4_K weights each). Launched one by one each pays a launch, a ramp and a tail, and HBM idles
// between them. Here one cooperative launch of one CTA per SM walks a list of PHASES,
//     qkv -> attention -> o -> gate|up -> down      (per block),   head,   argmax
// handing each phase's output vector to the next through memory. What makes it fast:
//   * every warp owns a TMA ring of weight tiles (16 rows x one 144-byte super-block per copy) that
//     runs ACROSS phases: weights do not depend on activations, so while a CTA waits at a barrier
//     its warps' rings are already filling with the next phase's tiles and HBM never idles;
//   * the glue between matvecs lives in the phases' prologues and epilogues: residual add +
//     RMSNorm + conversion of the activation row into the decode operand (every CTA redoes the
//     16 KB row: cheaper than a phase of its own), SiLU(gate)*up in the gate|up epilogue (a tile
//     is 8 gate rows + 8 matching up rows: the reference's Gate2, jit/gpu/kernels/matvec.go:283-290),
//     RoPE and the KV-cache append inside the attention phase, argmax after the head;
//   * no grid barrier between phases: every vector that crosses a phase boundary (q|k|v, the attention output,
//     the o and down partial sums, SiLU*up) is stored as (value, sequence number) pairs in single 8-byte
//     stores, and a consumer simply re-reads a pair until it carries the sequence number of the producing
//     phase. The handoff costs one trip through L2 instead of a fence, an atomic and a poll, and a CTA waits
//     only for the data it reads. (A phase's prologue reads the WHOLE vector, so it still orders a CTA after
//     every producer, which is what makes the single-buffered reuse of the vectors safe.)
//   * tensor parallel ranks exchange the row-parallel partial sums the same way: the o and down epilogues
//     store their pairs into every rank's slot buffer over NVLink with plain peer stores, and the next
//     prologue sums the ranks' planes in rank order (bit-stable). No collective call, no system-wide fence.
// Every wait (ring slot, data pair, the one grid barrier in front of the argmax) is bounded by the GPU's
// global timer; when one
// runs out the kernel records a code, raises an abort word that every other wait polls, waits
// (bounded) for its own copies in flight and returns.
#include "jl_internal.cuh"
#include "tma.cuh"
#include "q4k_dot.cuh"

#include <string.h>

#define BK_WARPS 16
#define BK_THREADS (BK_WARPS * 32)
#define BK_STAGES 4
#define BK_TILE 2304                 // 16 rows x 144 B
#define BK_MAX_NSB 64                // longest activation row: 64 super-blocks = 16384 elements
#define BK_ROUND_TASKS 256           // warp-tasks whose partial sums one round keeps in shared memory
#define BK_ATT_CHUNK 32              // cache positions per attention task
#define BK_ATT_D 128
#define BK_MAX_G 4                   // query heads per kv head
#define BK_MAX_WORLD 8
#define BK_ATT_SUB_BYTES 13824       // shared memory of one 128-thread attention group

enum { BK_MATVEC = 0, BK_ATTN = 1, BK_FINAL = 2 };
enum { BK_PRO_NORM = 0, BK_PRO_PLAIN = 1 };
enum { BK_EPI_STORE = 0, BK_EPI_GATE2 = 1, BK_EPI_ARGMAX = 2 };

// Status codes of the waits. Diagnostic builds (BK_DIAG) append the site and, through bk_diag_phase, the phase and CTA.
#ifdef BK_DIAG
#define BK_CODE(code, site) ((code) * 10 + (site))
static __device__ int bk_diag_phase[256];   // the phase each CTA is in
static __device__ unsigned bk_diag_iter[256];   // polls of the wait that gave up, in thousands
#define BK_DIAG_WHERE(code) ((code) + 100 * bk_diag_phase[blockIdx.x] + 100000 * (int)min(bk_diag_iter[blockIdx.x] >> 10, 20000u))
#define BK_DIAG_ITER(i) (bk_diag_iter[blockIdx.x] = (i))
#else
#define BK_DIAG_WHERE(code) (code)
#define BK_DIAG_ITER(i) ((void)0)
#define BK_CODE(code, site) (code)
#endif
typedef uint2 bk_ll;    // {float bits, sequence number of the phase that produced it}: one 8-byte store, atomic

struct alignas(16) bk_phase {
    int kind;
    // ---- matvec
    int map;            // index of the weight's tensor map: box 144 B x 16 rows (GATE2: x 8 rows)
    int nrows;          // output values (GATE2: ffn = the rows of the gate half)
    int nsb;            // super-blocks per row
    int prologue, epilogue;
    int up_row0;        // GATE2: first row of the up half inside the map
    int exchange;       // outputs go to every rank's slot buffer
    int nplanes;        // NORM: partial planes added to the residual row (0 = none)
    int from_emb;       // NORM: the residual row starts as the embedding of *tok
    const bk_ll *planes;   // NORM: [nplanes][hidden]
    const float *norm_w;   // NORM: [hidden]
    const bk_ll *vsrc;     // PLAIN: the activation row
    bk_ll *out;            // STORE / GATE2: output vector
    float *out_f32;        // ARGMAX: the logits, plain f32
    bk_ll *peer_out[BK_MAX_WORLD];   // exchange: this rank's plane inside every rank's slot buffer
    // ---- attention
    const bk_ll *qkv;      // [(hq + 2 hkv) * 128]
    bk_ll *att;            // [hq * 128]
    void *k_cache, *v_cache;   // bf16 [hkv][max_len][128]
    unsigned *tickets;     // [hkv], zero at launch
};

struct bk_params {
    const bk_phase *phases;
    int nphases;
    const CUtensorMap *maps;
    int hidden, hq, hkv, max_len;
    float eps;
    const float *cos_t, *sin_t;          // [max_len][64]
    const __nv_bfloat16 *emb;            // [vocab_total][hidden]
    long long *tok, *pos;
    int advance;                         // FINAL: *tok = argmax, *pos += 1
    long long *next_tok;                 // FINAL: argmax goes here too (may be NULL)
    float *part;                         // attention partials
    float *cand_val; int *cand_idx;      // [grid] per-CTA argmax candidates
    unsigned *bar;                       // grid barrier counter, zero at launch
    int *abort_word;                     // zero at launch
    int *status;                         // [0] code, [1] limit in microseconds
    int rank, world;
    unsigned *seq;                       // sequence numbers used up by earlier launches (nphases per launch)
    unsigned long long *trace;           // optional [2][nphases][4] global-timer stamps of the first and the last CTA
};

// ------------------------------------------------------------------ small helpers

__device__ __forceinline__ unsigned bk_ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int bk_ld_volatile(const int *p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void bk_subbar(int id) {   // the 128 threads of one attention group
    asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}
__device__ __forceinline__ void bk_bf16x8(const uint4 &v, float *f) {
    const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

// Between two polls of a value that has not arrived: every waiting thread of every CTA re-reads L2, and those reads
// queue in front of the loads of the CTAs that still produce.
#ifndef BK_POLL_SLEEP_NS
#define BK_POLL_SLEEP_NS 0
#endif
#if BK_POLL_SLEEP_NS > 0
#define BK_POLL_PAUSE() __nanosleep(BK_POLL_SLEEP_NS)
#else
#define BK_POLL_PAUSE() do { } while (0)
#endif
__device__ __forceinline__ uint4 bk_ld_vol16(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void bk_ll_store(bk_ll *p, float v, unsigned seq) {
    asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
struct bk_params;
__device__ __forceinline__ bool bk_ll_giveup(const bk_params &P, uint64_t t0, uint64_t limit_ns, int code);
// Two / four consecutive values of a vector another CTA (or another GPU) produces in phase `seq`: re-read until
// every pair carries `seq`. p is 16- / 32-byte aligned. False when the wait was given up (abort or timeout).
__device__ __forceinline__ bool bk_ll_read2(const bk_ll *p, unsigned seq, float2 &out, const bk_params &P, uint64_t limit_ns, int code) {
    uint4 a = bk_ld_vol16(p);
    if (a.y != seq || a.w != seq) {
        const uint64_t t0 = jl_gtime_ns();
        for (uint32_t i = 0;; i++) {
            BK_POLL_PAUSE();
            a = bk_ld_vol16(p);
            if (a.y == seq && a.w == seq) break;
            if ((i & 7u) == 7u) { BK_DIAG_ITER(i); if (bk_ll_giveup(P, t0, limit_ns, code)) return false; }
        }
    }
    out = make_float2(__uint_as_float(a.x), __uint_as_float(a.z));
    return true;
}
__device__ __forceinline__ bool bk_ll_read4(const bk_ll *p, unsigned seq, float4 &out, const bk_params &P, uint64_t limit_ns, int code) {
    uint4 a = bk_ld_vol16(p), b = bk_ld_vol16(p + 2);
    if (a.y != seq || a.w != seq || b.y != seq || b.w != seq) {
        const uint64_t t0 = jl_gtime_ns();
        for (uint32_t i = 0;; i++) {
            BK_POLL_PAUSE();
            a = bk_ld_vol16(p); b = bk_ld_vol16(p + 2);
            if (a.y == seq && a.w == seq && b.y == seq && b.w == seq) break;
            if ((i & 7u) == 7u) { BK_DIAG_ITER(i); if (bk_ll_giveup(P, t0, limit_ns, code)) return false; }
        }
    }
    out = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
    return true;
}

// N reads at once: every load is issued before the first flag is looked at, so a batch costs one trip to L2 instead of
// N. A null pointer skips its slot (the output is zero).
template <int N>
__device__ __forceinline__ bool bk_ll_read4_n(const bk_ll *const (&p)[N], unsigned seq, float4 (&out)[N], const bk_params &P,
                                              uint64_t limit_ns, int code) {
    uint4 a[N], b[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        a[i] = b[i] = make_uint4(0u, seq, 0u, seq);
        if (p[i]) { a[i] = bk_ld_vol16(p[i]); b[i] = bk_ld_vol16(p[i] + 2); }
    }
    bool ok = true;
#pragma unroll
    for (int i = 0; i < N; i++) {
        if (a[i].y != seq || a[i].w != seq || b[i].y != seq || b[i].w != seq) ok = bk_ll_read4(p[i], seq, out[i], P, limit_ns, code) && ok;
        else out[i] = make_float4(__uint_as_float(a[i].x), __uint_as_float(a[i].z), __uint_as_float(b[i].x), __uint_as_float(b[i].z));
    }
    return ok;
}
template <int N>
__device__ __forceinline__ bool bk_ll_read2_n(const bk_ll *const (&p)[N], unsigned seq, float2 (&out)[N], const bk_params &P,
                                              uint64_t limit_ns, int code) {
    uint4 a[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        a[i] = make_uint4(0u, seq, 0u, seq);
        if (p[i]) a[i] = bk_ld_vol16(p[i]);
    }
    bool ok = true;
#pragma unroll
    for (int i = 0; i < N; i++) {
        if (a[i].y != seq || a[i].w != seq) ok = bk_ll_read2(p[i], seq, out[i], P, limit_ns, code) && ok;
        else out[i] = make_float2(__uint_as_float(a[i].x), __uint_as_float(a[i].z));
    }
    return ok;
}

__device__ __forceinline__ bool bk_mbar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 16; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_ns(bar, parity, limit_ns);
}

__device__ __forceinline__ bool bk_ll_giveup(const bk_params &P, uint64_t t0, uint64_t limit_ns, int code) {
    if (bk_ld_volatile(P.abort_word)) return true;
    if (jl_gtime_ns() - t0 > limit_ns) {
        atomicCAS(P.status, 0, BK_DIAG_WHERE(code));       // the first wait that ran out names the cause; later ones are its consequences
        atomicExch(P.abort_word, 1);
        return true;
    }
    return false;
}

// Spins until *p >= target (p: a counter other CTAs or other GPUs advance). False on abort or timeout.
template <bool SYS>
__device__ __forceinline__ bool bk_wait_ge(const unsigned *p, unsigned target, const bk_params &P, uint64_t limit_ns, int code) {
    const uint64_t t0 = jl_gtime_ns();
    for (uint32_t i = 0;; i++) {
        const unsigned v = bk_ld_acquire_gpu(p);
        if (v >= target) return true;
        if ((i & 15u) == 15u) {
            if (bk_ld_volatile(P.abort_word)) return false;
            if (jl_gtime_ns() - t0 > limit_ns) {
                atomicCAS(P.status, 0, BK_DIAG_WHERE(code));       // the first wait that ran out names the cause; later ones are its consequences
                atomicExch(P.abort_word, 1);
                return false;
            }
        }
    }
}

// All CTAs of the grid meet. `done` counts the barriers this launch has passed. Writes made before the barrier by
// any CTA are visible (through L2: read them with ld.cg / ld.volatile, never through L1) after it.
__device__ __forceinline__ bool bk_grid_sync(const bk_params &P, int &done, uint64_t limit_ns) {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        // release: the CTA's writes (ordered before this thread by the barrier above) become visible before the count
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.bar) : "memory");
        s_ok = bk_wait_ge<false>(P.bar, (unsigned)(done + 1) * gridDim.x, P, limit_ns, BK_CODE(4, 4)) ? 1 : 0;   // acquire loads
    }
    __syncthreads();
    done++;
    return s_ok != 0;
}

// ------------------------------------------------------------------ the warp's stream of weight tiles
//
// A CTA owns a contiguous range of a matvec phase's 16-row groups; it walks them in rounds of as many row groups
// as BK_ROUND_TASKS warp-tasks cover; inside a round warp w takes tasks w, w + 16, ... (task = row group x
// super-block, super-block fastest). The fetch side (TMA requests) and the consume side walk the same sequence;
// the fetch side runs BK_STAGES tasks ahead and simply continues into the following matvec phases.
// What the hot loop needs to know about a phase, staged in shared memory once per launch (the phase list itself
// lives in global memory: reading it from the fetch path cost more than the fetch).
struct bk_pinfo {
    int kind, map, nsb, epi;
    int rg0, rg1, up_row0, rpr;   // this CTA's row groups [rg0, rg1); row groups per round
};
#define BK_MAX_PHASES 512

struct bk_cursor {
    int p;        // phase index (nphases = exhausted)
    int rg1;      // end of the CTA's row groups in this phase
    int rbase;    // first row group of the current round
    int nr;       // row groups in the current round
    int rgl, sb;  // this warp's task inside the round: row group (relative to rbase) and super-block
    int nsb, rpr;
};

__device__ __forceinline__ int bk_phase_nrg(const bk_phase &ph) {
    return ph.epilogue == BK_EPI_GATE2 ? (ph.nrows + 7) / 8 : (ph.nrows + 15) / 16;
}
__device__ __forceinline__ int bk_rounds_rgs(int nsb) {
    const int r = BK_ROUND_TASKS / nsb;
    return r < 1 ? 1 : r;
}
// The warp's first task of a round: task index `warp`, if the round has that many.
__device__ __forceinline__ bool bk_cursor_round(bk_cursor &c, int warp) {
    if (warp >= c.nr * c.nsb) return false;
    c.rgl = warp / c.nsb; c.sb = warp % c.nsb;
    return true;
}
// Positions the cursor on the warp's first task of the first matvec phase >= p that has one.
__device__ __forceinline__ void bk_cursor_seek(bk_cursor &c, const bk_pinfo *pi, int nphases, int p, int warp) {
    for (; p < nphases; p++) {
        const bk_pinfo f = pi[p];
        if (f.kind != BK_MATVEC) continue;
        c.rg1 = f.rg1; c.nsb = f.nsb; c.rpr = f.rpr;
        for (c.rbase = f.rg0; c.rbase < c.rg1; c.rbase += c.rpr) {
            c.nr = min(c.rpr, c.rg1 - c.rbase);
            if (bk_cursor_round(c, warp)) { c.p = p; return; }
        }
    }
    c.p = nphases;
}
__device__ __forceinline__ void bk_cursor_next(bk_cursor &c, const bk_pinfo *pi, int nphases, int warp) {
    c.sb += BK_WARPS;                       // task index + 16, super-block fastest
    while (c.sb >= c.nsb) { c.sb -= c.nsb; c.rgl++; }
    if (c.rgl < c.nr) return;
    for (c.rbase += c.rpr; c.rbase < c.rg1; c.rbase += c.rpr) {
        c.nr = min(c.rpr, c.rg1 - c.rbase);
        if (bk_cursor_round(c, warp)) return;
    }
    bk_cursor_seek(c, pi, nphases, c.p + 1, warp);
}
// Requests the cursor's tile into a ring stage (one elected lane calls this).
__device__ __forceinline__ void bk_fetch(const bk_cursor &c, const bk_pinfo *pi, const CUtensorMap *maps, uint32_t tile_smem,
                                         uint32_t bar) {
    const bk_pinfo f = pi[c.p];
    const int rg = c.rbase + c.rgl, sb = c.sb;
    const CUtensorMap *map = maps + f.map;
    mbar_arrive_expect_tx(bar, BK_TILE);
    if (f.epi == BK_EPI_GATE2) {
        tma_load_2d(tile_smem, map, sb * 144, rg * 8, bar);                            // 8 gate rows
        tma_load_2d(tile_smem + 8 * 144, map, sb * 144, f.up_row0 + rg * 8, bar);      // the matching 8 up rows
    } else {
        tma_load_2d(tile_smem, map, sb * 144, rg * 16, bar);
    }
}

// ------------------------------------------------------------------ prologues

// Builds the decode operand of the phase's activation row in shared memory (every CTA, the whole row). Warp w owns
// super-block w (NORM: rows of at most BK_WARPS super-blocks) or super-blocks w, w + 16, ... (PLAIN).
//   NORM   the residual row lives in registers for the whole launch (xres: warp w's lanes hold the eight values of
//          super-block w each): xres (+)= the planes of the previous o / down phase in rank order, then
//          RMSNorm(xres) * norm_w becomes the operand. Every CTA keeps its own copy and gets the same bits.
//   PLAIN  the operand of the previous phase's output vector as it is (attention output, SiLU*up).
// seq: the sequence number the producing phase stamped on its values. False when a wait was given up.
#define BK_PRO_IT (BK_MAX_NSB / BK_WARPS)
#ifdef BK_FINE_TRACE
#define BK_PT(i) do { ft[i] = clock64(); } while (0)
#define BK_PT_ARG , long long *ft
#else
#define BK_PT(i) do { } while (0)
#define BK_PT_ARG
#endif
__device__ __forceinline__ bool bk_prologue(const bk_params &P, const bk_phase &ph, uint8_t *xop, float *ssq, float4 (&xres)[2],
                                            unsigned seq, uint64_t limit_ns BK_PT_ARG) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nsb = ph.nsb;
    bool ok = true;
    BK_PT(0);
    if (ph.prologue == BK_PRO_NORM) {
        const bool mine = warp < nsb;
        float4 gw[2];
        if (mine) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int i4 = warp * 64 + hf * 32 + lane;
                gw[hf] = ph.norm_w ? __ldg(reinterpret_cast<const float4 *>(ph.norm_w) + i4) : make_float4(1.f, 1.f, 1.f, 1.f);
                if (ph.from_emb) {
                    const long long tok = *P.tok;
                    const uint2 u = __ldg(reinterpret_cast<const uint2 *>(P.emb + (size_t)tok * P.hidden) + i4);
                    const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&u);
                    const float2 lo = __bfloat1622float2(b2[0]), hi = __bfloat1622float2(b2[1]);
                    xres[hf] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
            for (int r = 0; r < ph.nplanes; r += 2) {                 // two planes per batch of loads
                const bk_ll *pp[4];
                float4 d[4];
#pragma unroll
                for (int q = 0; q < 4; q++)
                    pp[q] = r + (q >> 1) < ph.nplanes
                                ? ph.planes + (size_t)(r + (q >> 1)) * P.hidden + (size_t)(warp * 64 + (q & 1) * 32 + lane) * 4 : nullptr;
                ok = bk_ll_read4_n<4>(pp, seq, d, P, limit_ns, BK_CODE(5, 5)) && ok;
#pragma unroll
                for (int q = 0; q < 4; q++) {                           // rank order: the same sum on every CTA and every rank
                    float4 &x = xres[q & 1];
                    x.x += d[q].x; x.y += d[q].y; x.z += d[q].z; x.w += d[q].w;
                }
            }
        }
        float ss = 0.f;
        if (mine) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const float4 a = xres[hf];
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        BK_PT(1);
        if (lane == 0) ssq[warp] = ss;
        __syncthreads();
        BK_PT(2);
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < BK_WARPS; i++) tot += ssq[i];      // fixed order: every CTA gets the same bits
        const float r = rsqrtf(tot / (float)P.hidden + P.eps);
        if (mine) {
            float4 v[2];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const float4 a = xres[hf], g4 = gw[hf];
                v[hf] = make_float4(a.x * r * g4.x, a.y * r * g4.y, a.z * r * g4.z, a.w * r * g4.w);
            }
            q4k_prep_sb_vals(v[0], v[1], xop + (size_t)warp * Q4K_XP_SB_BYTES, lane);
        }
    } else {
        float4 v[BK_PRO_IT][2];
#pragma unroll
        for (int it = 0; it < BK_PRO_IT; it += 2) {
            const bk_ll *pp[4];
            float4 d[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int sb = warp + (it + (q >> 1)) * BK_WARPS;
                pp[q] = sb < nsb ? ph.vsrc + (size_t)sb * 256 + (q & 1) * 128 + lane * 4 : nullptr;
            }
            ok = bk_ll_read4_n<4>(pp, seq, d, P, limit_ns, BK_CODE(4, 1)) && ok;
            v[it][0] = d[0]; v[it][1] = d[1]; v[it + 1][0] = d[2]; v[it + 1][1] = d[3];
        }
        BK_PT(1);
        BK_PT(2);
#pragma unroll
        for (int it = 0; it < BK_PRO_IT; it++) {
            const int sb = warp + it * BK_WARPS;
            if (sb < nsb) q4k_prep_sb_vals(v[it][0], v[it][1], xop + (size_t)sb * Q4K_XP_SB_BYTES, lane);
        }
    }
    BK_PT(3);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    BK_PT(4);
    return ok;
}

// Pulls the next matvec phase's norm weights (and, for the first phase, nothing else) towards L2 while the current phase
// streams: the weights of a step are far larger than L2, so without this every prologue would wait on HBM for 16 KB.
__device__ __forceinline__ void bk_prefetch_norm(const bk_params &P, int p_from) {
    for (int q = p_from; q < P.nphases; q++) {
        const bk_phase &n = P.phases[q];
        if (n.kind != BK_MATVEC || n.prologue != BK_PRO_NORM) continue;
        if (n.norm_w) {
            const int lines = P.hidden * 4 / 128;
            for (int i = threadIdx.x; i < lines; i += BK_THREADS)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(n.norm_w) + (size_t)i * 128));
        }
        return;
    }
}

// ------------------------------------------------------------------ attention phase
//
// A CTA-task is (kv head, block of four chunks of BK_ATT_CHUNK cache positions); each of the CTA's four 128-thread
// groups takes one chunk, all G query heads of the kv head at once. K and V rows go from global memory straight
// into registers (a thread owns 64 bytes of one K row and 16 bytes of four V rows; the lines were pulled into L2
// before the preceding grid barrier). q and the new k are rotated here (adjacent-pair RoPE) and rounded to bf16 as
// the cache stores them; the thread that owns the new position builds its k / v piece from the q|k|v row instead of
// loading it, and appends it to the cache. The four groups' partial (max, sum, weighted V) meet in shared memory;
// one record per CTA goes to `part`, and the CTA that takes the last ticket of its kv head merges the records in
// block order (bit-stable).
#define BK_QS_STRIDE 36     // floats between the four 32-dim quarters of a q row: keeps the quarter reads off one bank

struct bk_att_smem {        // one group's shared memory
    float qs[BK_MAX_G][4 * BK_QS_STRIDE];
    float sc[BK_MAX_G][BK_ATT_CHUNK];
    float mred[4][BK_MAX_G], lred[4][BK_MAX_G];
    float red4[4][BK_MAX_G][BK_ATT_D];
    float gp_o[BK_MAX_G][BK_ATT_D];
    float gp_m[BK_MAX_G], gp_l[BK_MAX_G];
    uint32_t kf[BK_ATT_D / 2], vf[BK_ATT_D / 2];   // the new position's key (rotated) and value as bf16 pairs
};
static_assert(sizeof(bk_att_smem) <= BK_ATT_SUB_BYTES, "attention group smem");

__device__ __forceinline__ int bk_att_nblk(int len) { return (len + 4 * BK_ATT_CHUNK - 1) / (4 * BK_ATT_CHUNK); }

// Before the grid barrier in front of an attention phase: the CTA's first task's K and V lines, towards L2.
__device__ __forceinline__ void bk_attention_prefetch(const bk_params &P, const void *k_cache, const void *v_cache) {
    const long long pos = *P.pos;
    if (pos < 0 || pos >= P.max_len) return;
    const int nblk = bk_att_nblk((int)pos + 1);
    const int ct = blockIdx.x;
    if (ct >= P.hkv * nblk) return;
    const int kv = ct / nblk, j = ct % nblk, sub = threadIdx.x >> 7, t = threadIdx.x & 127;
    const int s0 = (4 * j + sub) * BK_ATT_CHUNK;
    const int row = s0 + (t & 63) / 2;                           // two 128-byte lines per 256-byte row
    if (row >= (int)pos) return;
    const uint8_t *base = static_cast<const uint8_t *>(t < 64 ? k_cache : v_cache);
    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + ((size_t)kv * P.max_len + row) * 256 + (t & 1) * 128));
}

#ifdef BK_FINE_TRACE
#define BK_AT(i) do { if (at && threadIdx.x == 0) at[i] = jl_gtime_ns(); } while (0)
#define BK_AT_ARG , unsigned long long *at
#else
#define BK_AT(i) do { } while (0)
#define BK_AT_ARG
#endif
template <int G>
__device__ bool bk_attention(const bk_params &P, const bk_phase &ph, uint8_t *work, unsigned seq_r, unsigned seq_w,
                             uint64_t limit_ns BK_AT_ARG) {
    constexpr int HDR = (2 * G + 3) & ~3;
    constexpr int STRIDE = HDR + G * BK_ATT_D;
    const int tid = threadIdx.x, sub = tid >> 7, t = tid & 127, warp = t >> 5, lane = t & 31;
    bk_att_smem *S = reinterpret_cast<bk_att_smem *>(work + (size_t)sub * BK_ATT_SUB_BYTES);
    auto group = [&](int g4) { return reinterpret_cast<const bk_att_smem *>(work + (size_t)g4 * BK_ATT_SUB_BYTES); };
    __shared__ unsigned s_last;
    const int bid = 1 + sub;
    const long long pos = *P.pos;
    if (pos < 0 || pos >= P.max_len) return true;
    bool ok = true;
    const int len = (int)pos + 1;
    const int nchunk = (len + BK_ATT_CHUNK - 1) / BK_ATT_CHUNK;
    const int nblk = bk_att_nblk(len), nblk_max = bk_att_nblk(P.max_len);
    __nv_bfloat16 *kc = static_cast<__nv_bfloat16 *>(ph.k_cache), *vc = static_cast<__nv_bfloat16 *>(ph.v_cache);
    const float *cs = P.cos_t + (size_t)pos * (BK_ATT_D / 2), *sn = P.sin_t + (size_t)pos * (BK_ATT_D / 2);
    const int p1 = t >> 2, qd = t & 3;          // scores: four threads per position, 32 dims each
    const int dg = t & 15, pg = t >> 4;         // weighted V: 16 threads per row (8 dims each), 8 position groups
    BK_AT(0);
    for (int ct = blockIdx.x; ct < P.hkv * nblk; ct += gridDim.x) {
        const int kv = ct / nblk, j = ct % nblk;
        const int chunk = 4 * j + sub;
        const int s0 = chunk * BK_ATT_CHUNK;
        const int cnt = chunk < nchunk ? min(BK_ATT_CHUNK, len - s0) : 0;
        uint4 kreg[4], vreg[4];
        {   // K: this thread's 64 bytes of row p1; V: 16 bytes of rows pg, pg + 8, pg + 16, pg + 24
            const int krow = s0 + p1;
            const uint4 *kg = reinterpret_cast<const uint4 *>(kc + ((size_t)kv * P.max_len + krow) * BK_ATT_D) + qd * 4;
#pragma unroll
            for (int c = 0; c < 4; ++c) kreg[c] = krow < (int)pos ? kg[c] : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int vrow = s0 + pg + 8 * i;
                vreg[i] = vrow < (int)pos ? reinterpret_cast<const uint4 *>(vc + ((size_t)kv * P.max_len + vrow) * BK_ATT_D)[dg]
                                          : make_uint4(0, 0, 0, 0);
            }
        }
        const bool fresh = (int)pos >= s0 && (int)pos < s0 + BK_ATT_CHUNK;
        // this thread's rotation pair (the same for the new key and for both of its q pairs: 128 = 2 x 64), asked for
        // before the polls below: after them it would be one more round trip between "q has arrived" and the scores
        const float rot_c = cs[t & 63], rot_s = sn[t & 63];
        if (fresh) {
            // the new position's key (rotated) and value: one pair per thread, rounded to bf16, appended to the cache and
            // handed through shared memory to the threads that own that row's pieces
            const int jp = t & 63;
            const bk_ll *src[1] = {ph.qkv + (size_t)(t < 64 ? P.hq + kv : P.hq + P.hkv + kv) * BK_ATT_D + 2 * jp};
            float2 ab[1];
            ok = bk_ll_read2_n<1>(src, seq_r, ab, P, limit_ns, BK_CODE(4, 2)) && ok;
            __nv_bfloat162 o;
            if (t < 64) {
                const float cc = rot_c, ss = rot_s;
                o = __floats2bfloat162_rn(ab[0].x * cc - ab[0].y * ss, ab[0].x * ss + ab[0].y * cc);
                S->kf[jp] = *reinterpret_cast<const uint32_t *>(&o);
                reinterpret_cast<__nv_bfloat162 *>(kc + ((size_t)kv * P.max_len + pos) * BK_ATT_D)[jp] = o;
            } else {
                o = __floats2bfloat162_rn(ab[0].x, ab[0].y);
                S->vf[jp] = *reinterpret_cast<const uint32_t *>(&o);
                reinterpret_cast<__nv_bfloat162 *>(vc + ((size_t)kv * P.max_len + pos) * BK_ATT_D)[jp] = o;
            }
        }
        {
            const int nq = G * (BK_ATT_D / 2);                            // q: rotate, round to bf16, scale; <= 2 pairs per thread
            const bk_ll *src[2];
            float2 ab[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int pi = t + 128 * u;
                src[u] = pi < nq ? ph.qkv + (size_t)(kv * G + (pi >> 6)) * BK_ATT_D + 2 * (pi & 63) : nullptr;
            }
            ok = bk_ll_read2_n<2>(src, seq_r, ab, P, limit_ns, BK_CODE(4, 3)) && ok;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int pi = t + 128 * u;
                if (pi < nq) {
                    const int h = pi >> 6, jp = pi & 63;
                    const float c = rot_c, s_ = rot_s;
                    const __nv_bfloat162 o = __floats2bfloat162_rn(ab[u].x * c - ab[u].y * s_, ab[u].x * s_ + ab[u].y * c);
                    const float2 f = __bfloat1622float2(o);
                    const int d0 = 2 * jp;                                // dims d0, d0 + 1: quarter d0 / 32
                    S->qs[h][(d0 >> 5) * BK_QS_STRIDE + (d0 & 31)] = f.x * 0.08838834764831845f;
                    S->qs[h][(d0 >> 5) * BK_QS_STRIDE + (d0 & 31) + 1] = f.y * 0.08838834764831845f;
                }
            }
        }
        bk_subbar(bid);
        BK_AT(1);
        if (fresh) {                            // the owners of the new row's pieces take them from shared memory
            if (s0 + p1 == (int)pos) {
#pragma unroll
                for (int c = 0; c < 4; ++c) kreg[c] = reinterpret_cast<const uint4 *>(S->kf)[qd * 4 + c];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (s0 + pg + 8 * i == (int)pos) vreg[i] = reinterpret_cast<const uint4 *>(S->vf)[dg];
        }
        float s[G];
#pragma unroll
        for (int h = 0; h < G; ++h) s[h] = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float f[8];
            bk_bf16x8(kreg[c], f);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float4 q0 = *reinterpret_cast<const float4 *>(&S->qs[h][qd * BK_QS_STRIDE + c * 8]);
                const float4 q1 = *reinterpret_cast<const float4 *>(&S->qs[h][qd * BK_QS_STRIDE + c * 8 + 4]);
                s[h] = fmaf(f[0], q0.x, s[h]); s[h] = fmaf(f[1], q0.y, s[h]); s[h] = fmaf(f[2], q0.z, s[h]); s[h] = fmaf(f[3], q0.w, s[h]);
                s[h] = fmaf(f[4], q1.x, s[h]); s[h] = fmaf(f[5], q1.y, s[h]); s[h] = fmaf(f[6], q1.z, s[h]); s[h] = fmaf(f[7], q1.w, s[h]);
            }
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
            s[h] += __shfl_xor_sync(0xffffffffu, s[h], 1);
            s[h] += __shfl_xor_sync(0xffffffffu, s[h], 2);
            if (p1 >= cnt) s[h] = -INFINITY;
            float m = s[h];
            for (int o = 16; o >= 4; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (lane == 0) S->mred[warp][h] = m;
        }
        bk_subbar(bid);
        float Mh[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
            Mh[h] = fmaxf(fmaxf(S->mred[0][h], S->mred[1][h]), fmaxf(S->mred[2][h], S->mred[3][h]));
            float p = (p1 < cnt && qd == 0) ? __expf(s[h] - Mh[h]) : 0.f;
            if (qd == 0) S->sc[h][p1] = p;
            for (int o = 16; o; o >>= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
            if (lane == 0) S->lred[warp][h] = p;
        }
        bk_subbar(bid);
        float acc[G][8];
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = pg + 8 * i;                                     // rows past cnt hold zeros and weight 0
            float f[8];
            bk_bf16x8(vreg[i], f);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float w = S->sc[h][p];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(w, f[e], acc[h][e]);
            }
        }
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], 16);   // the warp's two position groups
        if (lane < 16) {
#pragma unroll
            for (int h = 0; h < G; ++h) {
                *reinterpret_cast<float4 *>(&S->red4[warp][h][dg * 8]) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
                *reinterpret_cast<float4 *>(&S->red4[warp][h][dg * 8 + 4]) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
            }
        }
        bk_subbar(bid);
#pragma unroll
        for (int h = 0; h < G; ++h) S->gp_o[h][t] = (S->red4[0][h][t] + S->red4[1][h][t]) + (S->red4[2][h][t] + S->red4[3][h][t]);
        if (t < G) {
            S->gp_m[t] = fmaxf(fmaxf(S->mred[0][t], S->mred[1][t]), fmaxf(S->mred[2][t], S->mred[3][t]));
            S->gp_l[t] = (S->lred[0][t] + S->lred[1][t]) + (S->lred[2][t] + S->lred[3][t]);
        }
        __syncthreads();
        // the CTA's record: the four groups in chunk order
        float *my = P.part + ((size_t)kv * nblk_max + j) * STRIDE;
        {
            const int h = tid >> 7, d = tid & 127;
            if (h < G) {
                float M = -INFINITY;
#pragma unroll
                for (int g4 = 0; g4 < 4; ++g4) M = fmaxf(M, group(g4)->gp_m[h]);
                float o = 0.f, l = 0.f;
#pragma unroll
                for (int g4 = 0; g4 < 4; ++g4) {
                    const float mg = group(g4)->gp_m[h];
                    const float w = mg == -INFINITY ? 0.f : __expf(mg - M);
                    o = fmaf(w, group(g4)->gp_o[h][d], o);
                    l = fmaf(w, group(g4)->gp_l[h], l);
                }
                my[HDR + h * BK_ATT_D + d] = o;
                if (d == 0) { my[h] = M; my[G + h] = l; }
            }
        }
        BK_AT(2);
        __threadfence();
        if (!__syncthreads_and(ok ? 1 : 0)) return false;
        BK_AT(3);
        if (tid == 0) s_last = atomicAdd(&ph.tickets[kv], 1u) == (unsigned)(nblk - 1) ? 1u : 0u;
        __syncthreads();
        if (s_last) {
            __threadfence();
            const float *base = P.part + (size_t)kv * nblk_max * STRIDE;
            const int h = tid >> 7, d = tid & 127;
            // ONE trip to L2 for the whole merge: the kv head's records are contiguous, so the CTA copies them (as many
            // as fit: 26 at G = 4, i.e. 3328 positions) into the groups' now free shared memory with every load in
            // flight at once, and merges from there. Dependent loads in a loop would cost a trip each.
            float *rs = reinterpret_cast<float *>(work);
            const int nrec = min(nblk, (int)(4 * BK_ATT_SUB_BYTES / 4) / STRIDE);
            static_assert(STRIDE % 4 == 0, "records are copied 16 bytes at a time");
            {   // 16-byte loads: at 2048 positions the 16 records are 2096 of them, about four per thread, one batch
                const float4 *b4 = reinterpret_cast<const float4 *>(base);
                float4 *r4 = reinterpret_cast<float4 *>(rs);
#pragma unroll 8
                for (int i = tid; i < nrec * (STRIDE / 4); i += BK_THREADS) r4[i] = __ldcg(b4 + i);
            }
            __syncthreads();
            BK_AT(6);
            if (h < G) {
                // Two loops each, one over the records in shared memory and one over the rest in global memory. As ONE
                // loop choosing per record, every step also issued the global-memory side's loads and waited for them
                // (3.5 us for 16 records, all of them in shared memory).
                float M = -INFINITY;
                for (int b2 = 0; b2 < nrec; ++b2) M = fmaxf(M, rs[b2 * STRIDE + h]);
                for (int b2 = nrec; b2 < nblk; ++b2) M = fmaxf(M, __ldcg(base + (size_t)b2 * STRIDE + h));
                float o = 0.f, l = 0.f;
                for (int b2 = 0; b2 < nrec; ++b2) {                       // ascending block order: bit-stable
                    const float *rec = rs + b2 * STRIDE;
                    const float mb = rec[h];
                    const float w = mb == -INFINITY ? 0.f : __expf(mb - M);
                    o = fmaf(w, rec[HDR + h * BK_ATT_D + d], o);
                    l = fmaf(w, rec[G + h], l);
                }
                for (int b2 = nrec; b2 < nblk; ++b2) {
                    const float *rec = base + (size_t)b2 * STRIDE;
                    const float mb = __ldcg(rec + h);
                    const float w = mb == -INFINITY ? 0.f : __expf(mb - M);
                    o = fmaf(w, __ldcg(rec + HDR + h * BK_ATT_D + d), o);
                    l = fmaf(w, __ldcg(rec + G + h), l);
                }
                bk_ll_store(ph.att + (size_t)(kv * G + h) * BK_ATT_D + d, l > 0.f ? o / l : 0.f, seq_w);
            }
            BK_AT(7);
        }
        __syncthreads();                                                  // the groups' shared memory is free again
        BK_AT(4);
    }
    BK_AT(5);
    return true;
}

// ------------------------------------------------------------------ the kernel

#define BK_RING_BYTES (BK_WARPS * BK_STAGES * BK_TILE)
#define BK_XOP_BYTES (BK_MAX_NSB * Q4K_XP_SB_BYTES)
#define BK_RED_BYTES (BK_ROUND_TASKS * 16 * 4)
#define BK_WORK_BYTES (4 * BK_ATT_SUB_BYTES > BK_XOP_BYTES + BK_RED_BYTES ? 4 * BK_ATT_SUB_BYTES : BK_XOP_BYTES + BK_RED_BYTES)
static_assert(sizeof(bk_pinfo) % 16 == 0, "the phase table is followed by 16-byte aligned descriptors");
#define BK_PHASE_BYTES ((sizeof(bk_phase) + 15) / 16 * 16)
#define BK_SMEM_BYTES (BK_RING_BYTES + BK_WORK_BYTES + Q4K_XP_ZERO_BYTES + BK_WARPS * BK_STAGES * 8 + 64 * 4 + BK_MAX_PHASES * sizeof(bk_pinfo) + 3 * BK_PHASE_BYTES + 128)

__global__ void __launch_bounds__(BK_THREADS, 1) jl_block_kernel(const __grid_constant__ bk_params P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // [rings | work: operand + round partials, or the four attention groups | zero fragment | barriers | misc]
    uint8_t *tiles = smem + (size_t)warp * BK_STAGES * BK_TILE;
    uint8_t *work = smem + BK_RING_BYTES;
    uint8_t *xop = work;
    float *red = reinterpret_cast<float *>(work + BK_XOP_BYTES);
    uint8_t *zero = work + BK_WORK_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(zero + Q4K_XP_ZERO_BYTES) + warp * BK_STAGES;
    float *misc = reinterpret_cast<float *>(zero + Q4K_XP_ZERO_BYTES + BK_WARPS * BK_STAGES * 8);   // 64 floats
    bk_pinfo *pinfo = reinterpret_cast<bk_pinfo *>(misc + 64);
    // Full phase descriptors, copied from global memory one phase ahead of their use into a ring of three; a barrier
    // at the top of every phase (right after the copy) orders the copy against both its readers and the readers
    // of the copy it replaces.
    uint8_t *phase_sm = reinterpret_cast<uint8_t *>(pinfo + BK_MAX_PHASES);
    auto stage_phase = [&](int q) {
        if (q < P.nphases && tid < (int)(BK_PHASE_BYTES / 16))
            reinterpret_cast<uint4 *>(phase_sm + (size_t)(q % 3) * BK_PHASE_BYTES)[tid] = __ldg(reinterpret_cast<const uint4 *>(P.phases + q) + tid);
    };
    stage_phase(0);
    const uint64_t limit_ns = jl_wait_limit_ns(P.status);
    const int nphases = P.nphases;
    const CUtensorMap *maps = P.maps;

    for (int i = tid; i < nphases; i += BK_THREADS) {
        const bk_phase &q = P.phases[i];
        bk_pinfo f;
        f.kind = q.kind; f.map = q.map; f.nsb = q.nsb; f.epi = q.epilogue; f.up_row0 = q.up_row0;
        f.rg0 = f.rg1 = 0; f.rpr = 1;
        if (q.kind == BK_MATVEC) {
            const int nrg = bk_phase_nrg(q);
            f.rg0 = (int)((long long)blockIdx.x * nrg / gridDim.x);
            f.rg1 = (int)((long long)(blockIdx.x + 1) * nrg / gridDim.x);
            f.rpr = bk_rounds_rgs(q.nsb);
        }
        pinfo[i] = f;
    }

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < BK_STAGES; s++) mbar_init(smem_u32(bars + s), 1);
        mbar_init_fence();
    }
    if (tid < Q4K_XP_ZERO_BYTES / 4) reinterpret_cast<uint32_t *>(zero)[tid] = 0u;
    __syncthreads();                    // the phase table is complete
    // The ring runs ahead of everything else: the first BK_STAGES tiles of this warp are requested now.
    bk_cursor fc;                       // fetch side
    uint32_t fetched = 0, consumed = 0;
    bk_cursor_seek(fc, pinfo, nphases, 0, warp);
    for (int s = 0; s < BK_STAGES && fc.p < nphases; s++) {
        if (lane == 0) bk_fetch(fc, pinfo, maps, smem_u32(tiles + s * BK_TILE), smem_u32(bars + s));
        bk_cursor_next(fc, pinfo, nphases, warp);
        fetched++;
    }

    int barriers_done = 0;
    // Phase p stamps its outputs with seq_base + p + 1; its inputs carry the previous phase's number, seq_base + p.
    const unsigned seq_base = bk_ld_acquire_gpu(P.seq);
    float4 xres[2];                     // the residual row: warp w's lanes hold super-block w's values
    xres[0] = xres[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    bool alive = true;
    float best_val = -INFINITY;
    int best_idx = 0x7fffffff;

    // per-phase time stamps (phase start, prologue done, work done, barrier passed) of the first and last CTA
    const int tr_cta = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x - 1 ? 1 : -1);
#ifdef BK_FINE_TRACE
    // experimental builds only: every CTA's stamps, after the other regions
#define BK_TRACE(slot)                                                                      \
    do {                                                                                    \
        if (P.trace && tid == 0) {                                                          \
            const unsigned long long now_ = jl_gtime_ns();                                  \
            if (tr_cta >= 0) P.trace[((size_t)tr_cta * P.nphases + p) * 4 + (slot)] = now_; \
            P.trace[(size_t)2 * P.nphases * 4 + (size_t)P.nphases * 12 + (size_t)gridDim.x * 8 + ((size_t)blockIdx.x * P.nphases + p) * 4 + (slot)] = now_; \
        }                                                                                   \
    } while (0)
#else
#define BK_TRACE(slot)                                                                      \
    do {                                                                                    \
        if (P.trace && tr_cta >= 0 && tid == 0) P.trace[((size_t)tr_cta * P.nphases + p) * 4 + (slot)] = jl_gtime_ns(); \
    } while (0)
#endif

#ifdef BK_FINE_TRACE
    // experimental builds only: clock64 spent between marks 0..6 of the consume loop, first CTA's first warp, per phase
    long long ft_acc[7], ft_last = 0;
#define BK_FT(i) do { const long long c_ = clock64(); if ((i) > 0) ft_acc[i] += c_ - ft_last; ft_last = c_; } while (0)
#else
#define BK_FT(i) do { } while (0)
#endif
    for (int p = 0; p < P.nphases && alive; p++) {
        const bk_phase &ph = *reinterpret_cast<const bk_phase *>(phase_sm + (size_t)(p % 3) * BK_PHASE_BYTES);
        const int p_kind = pinfo[p].kind, p_epi = pinfo[p].epi;   // from the immutable table, not from the ring
#ifdef BK_DIAG
        if (tid == 0) bk_diag_phase[blockIdx.x] = p;
#endif
        stage_phase(p + 1);
        // Every thread passes this barrier between the staging of phase p + 1's descriptor and its first use, and
        // between its last look at phase p - 2's copy and the overwrite above. Without it a CTA that has no work
        // item in an attention phase crosses that phase without any barrier, and a warp could read the FOLLOWING
        // phase's descriptor before warp 0 had stored it: it then waited for the inputs of the phase that had used
        // the slot three phases earlier (seen as a bounded-wait timeout about once in 250,000 attention phases).
        __syncthreads();
#ifdef BK_FINE_TRACE
        for (int i = 0; i < 7; i++) ft_acc[i] = 0;
#endif
        BK_TRACE(0);
        const unsigned seq_r = seq_base + (unsigned)p, seq_w = seq_r + 1u;
        if ((int)blockIdx.x == (p + 1) % (int)gridDim.x) bk_prefetch_norm(P, p + 1);
        if (p + 1 < nphases && pinfo[p + 1].kind == BK_ATTN)          // the next phase's K and V lines, towards L2
            bk_attention_prefetch(P, P.phases[p + 1].k_cache, P.phases[p + 1].v_cache);
        if (p_kind == BK_MATVEC) {
#ifdef BK_FINE_TRACE
            long long pt[5] = {0, 0, 0, 0, 0};
            alive = bk_prologue(P, ph, xop, misc, xres, seq_r, limit_ns, pt);
            if (P.trace && blockIdx.x == 0 && tid == 0)
                for (int i = 1; i < 5; i++) P.trace[(size_t)2 * P.nphases * 4 + (size_t)P.nphases * 8 + (size_t)p * 4 + i - 1] = (unsigned long long)(pt[i] - pt[i - 1]);
#else
            alive = bk_prologue(P, ph, xop, misc, xres, seq_r, limit_ns);
#endif
            BK_TRACE(1);
            if (!alive) break;
            const int nsb = pinfo[p].nsb, rg0 = pinfo[p].rg0, rg1 = pinfo[p].rg1, rpr = pinfo[p].rpr;
            for (int rbase = rg0; rbase < rg1 && alive; rbase += rpr) {
                const int nr = min(rpr, rg1 - rbase), ntask = nr * nsb;
                for (int tk = warp; tk < ntask; tk += BK_WARPS) {
                    const int sb = tk % nsb;
                    const uint32_t s = consumed % BK_STAGES, parity = (consumed / BK_STAGES) & 1u;
                    BK_FT(0);
                    if (!__all_sync(0xffffffffu, bk_mbar_wait(smem_u32(bars + s), parity, limit_ns))) {
                        if (lane == 0) { atomicCAS(P.status, 0, BK_DIAG_WHERE(BK_CODE(1, 6))); atomicExch(P.abort_word, 1); }
                        alive = false;
                        break;
                    }
                    BK_FT(1);
                    const q4k_lane_tile w = q4k_lane_load(tiles + s * BK_TILE, g, t);
                    consumed++;
                    __syncwarp();        // every lane holds its share: the stage may be refilled
                    if (fc.p < nphases) {
                        if (lane == 0) bk_fetch(fc, pinfo, maps, smem_u32(tiles + s * BK_TILE), smem_u32(bars + s));
                        bk_cursor_next(fc, pinfo, nphases, warp);
                        fetched++;
                    }
                    BK_FT(2);
                    float accA = 0.f, accB = 0.f;
                    q4k_dot_task(w, xop + (size_t)sb * Q4K_XP_SB_BYTES, zero, g, t, accA, accB);
                    accA += __shfl_xor_sync(0xffffffffu, accA, 1);
                    accA += __shfl_xor_sync(0xffffffffu, accA, 2);
                    accB += __shfl_xor_sync(0xffffffffu, accB, 1);
                    accB += __shfl_xor_sync(0xffffffffu, accB, 2);
                    if (t == 0) {
                        red[tk * 16 + g] = accA;
                        red[tk * 16 + g + 8] = accB;
                    }
                    BK_FT(3);
                }
                BK_FT(4);
                alive = __syncthreads_and(alive ? 1 : 0) != 0;
                BK_FT(5);
                if (!alive) break;
                // the round's row groups: super-blocks in ascending order (run-to-run bit-stable)
                if (p_epi == BK_EPI_GATE2) {
                    if (tid < nr * 8) {
                        const int rgl = tid >> 3, r = tid & 7;
                        float sg = 0.f, su = 0.f;
                        for (int sb = 0; sb < nsb; sb++) {
                            sg += red[(rgl * nsb + sb) * 16 + r];
                            su += red[(rgl * nsb + sb) * 16 + r + 8];
                        }
                        const int o = (rbase + rgl) * 8 + r;
                        if (o < ph.nrows) bk_ll_store(ph.out + o, sg / (1.f + __expf(-sg)) * su, seq_w);     // SiLU(gate) * up
                    }
                } else if (tid < nr * 16) {
                    const int rgl = tid >> 4, r = tid & 15;
                    float sum = 0.f;
                    for (int sb = 0; sb < nsb; sb++) sum += red[(rgl * nsb + sb) * 16 + r];
                    const int row = (rbase + rgl) * 16 + r;
                    if (row < ph.nrows) {
                        if (p_epi == BK_EPI_ARGMAX) {
                            ph.out_f32[row] = sum;
                            if (sum > best_val || (sum == best_val && row < best_idx)) { best_val = sum; best_idx = row; }
                        } else if (ph.exchange) {
#pragma unroll 1
                            for (int pr = 0; pr < P.world; pr++) bk_ll_store(ph.peer_out[pr] + row, sum, seq_w);   // over NVLink for pr != rank
                        } else {
                            bk_ll_store(ph.out + row, sum, seq_w);
                        }
                    }
                }
                __syncthreads();         // the round's partials are consumed
                BK_FT(6);
            }
            if (alive && p_epi == BK_EPI_ARGMAX) {
                // the CTA's candidate: largest value, lowest row on a tie
                for (int o = 16; o; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best_val, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
                    if (ov > best_val || (ov == best_val && oi < best_idx)) { best_val = ov; best_idx = oi; }
                }
                int *misc_i = reinterpret_cast<int *>(misc + 32);
                if (lane == 0) { misc[warp] = best_val; misc_i[warp] = best_idx; }
                __syncthreads();
                if (tid == 0) {
                    float bv = misc[0]; int bi = misc_i[0];
                    for (int i = 1; i < BK_WARPS; i++)
                        if (misc[i] > bv || (misc[i] == bv && misc_i[i] < bi)) { bv = misc[i]; bi = misc_i[i]; }
                    P.cand_val[blockIdx.x] = bv; P.cand_idx[blockIdx.x] = bi;
                }
            }
        } else if (p_kind == BK_ATTN) {
            const int G = P.hq / P.hkv;
#ifdef BK_FINE_TRACE
            unsigned long long *at = (P.trace && p == 6) ? P.trace + (size_t)2 * P.nphases * 4 + (size_t)P.nphases * 12 + (size_t)blockIdx.x * 8 : nullptr;
            if (G == 4) alive = bk_attention<4>(P, ph, work, seq_r, seq_w, limit_ns, at);
            else if (G == 2) alive = bk_attention<2>(P, ph, work, seq_r, seq_w, limit_ns, at);
            else alive = bk_attention<1>(P, ph, work, seq_r, seq_w, limit_ns, at);
#else
            if (G == 4) alive = bk_attention<4>(P, ph, work, seq_r, seq_w, limit_ns);
            else if (G == 2) alive = bk_attention<2>(P, ph, work, seq_r, seq_w, limit_ns);
            else alive = bk_attention<1>(P, ph, work, seq_r, seq_w, limit_ns);
#endif
        } else {   // BK_FINAL: CTA 0 picks the winner among the CTAs' candidates
            if (blockIdx.x == 0 && warp == 0) {
                float bv = -INFINITY; int bi = 0x7fffffff;
                for (int i = lane; i < (int)gridDim.x; i += 32) {
                    const float v = __ldcg(P.cand_val + i); const int ix = __ldcg(P.cand_idx + i);
                    if (v > bv || (v == bv && ix < bi)) { bv = v; bi = ix; }
                }
                for (int o = 16; o; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                }
                if (lane == 0) {
                    const long long nxt = bi == 0x7fffffff ? 0 : bi;
                    if (P.next_tok) *P.next_tok = nxt;
                    if (P.advance) { *P.tok = nxt; *P.pos = *P.pos + 1; }
                }
            }
        }
        BK_TRACE(2);
#ifdef BK_FINE_TRACE
        if (P.trace && blockIdx.x == 0 && tid == 0)
            for (int i = 1; i < 7; i++) P.trace[(size_t)2 * P.nphases * 4 + (size_t)p * 8 + i] = (unsigned long long)ft_acc[i];
#endif
        if (!alive || p + 1 >= P.nphases) break;
        // The only grid-wide meeting of a launch: the argmax reads every CTA's candidate.
        if (pinfo[p + 1].kind == BK_FINAL) alive = bk_grid_sync(P, barriers_done, limit_ns);
        BK_TRACE(3);
    }
#undef BK_TRACE
#undef BK_FT
    // The launch's sequence numbers are used up (also after an abort, so that the ranks' counters stay in step). Every
    // CTA read the counter before it produced anything CTA 0's last phases depend on.
    if (blockIdx.x == 0 && tid == 0) *P.seq = seq_base + (unsigned)P.nphases;
    // Copies still in flight into this CTA's shared memory must land before the CTA may exit.
    for (; consumed < fetched; consumed++) {
        const uint32_t s = consumed % BK_STAGES, parity = (consumed / BK_STAGES) & 1u;
        mbar_wait_ns(smem_u32(bars + s), parity, limit_ns);
    }
}

// ------------------------------------------------------------------ host

struct jl_layers {
    jl_ctx *ctx;
    int n_layer, hidden, hq, hkv, ffn, vocab, max_len, rank, world, grid;
    uint8_t *buf;          // phases, tensor maps and every scratch vector of the step: one allocation
    uint8_t *slot;         // partial-sum planes of o and down for every rank + the exchange flags (peers write here)
    size_t slot_bytes;
    bk_phase *phases_dev;
    std::vector<bk_phase> phases;
    float *logits;
    size_t zero_bytes;           // barrier counter, abort word and attention tickets: cleared in front of every launch
    unsigned long long *trace;   // [2][nphases][4]
    bk_params P;
    bool attached;
};

static size_t bk_al(size_t n) { return (n + 255) & ~(size_t)255; }
static size_t bk_slot_bytes(int world, int hidden) { return 2 * bk_al((size_t)world * hidden * sizeof(bk_ll)); }

// PrepLayer for every block plus the head (engine/nn/device.go:1099-1102): checks that each weight has a
// kernel here, builds the phase list and sizes all scratch. Declines (JL_DECLINED) instead of running a
// shape the block kernel does not serve; the caller then keeps its per-matvec path.
JL_EXPORT int jl_layers_prep(jl_ctx *ctx, const jl_layers_desc *d, jl_layers **out) {
    if (!ctx || !d || !out || !d->blocks) return JL_EINVAL;
    *out = nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    const int L = d->n_layer, H = d->hidden, hq = d->n_head, hkv = d->n_kv, F = d->ffn, V = d->vocab;
    const int world = d->world < 1 ? 1 : d->world, rank = d->rank;
    if (L < 1 || H < 256 || H % 256 || d->head_dim != BK_ATT_D || hq < 1 || hkv < 1 || hq % hkv || F < 256 || F % 256 ||
        (hq * BK_ATT_D) % 256 || d->max_len < 1 || world > BK_MAX_WORLD || rank < 0 || rank >= world)
        return jl_set_err(ctx, JL_DECLINED, "block kernel: shape not served (hidden %d, heads %d/%d x %d, ffn %d, world %d)", H, hq,
                          hkv, d->head_dim, F, world);
    const int G = hq / hkv;
    if (G != 1 && G != 2 && G != 4)
        return jl_set_err(ctx, JL_DECLINED, "block kernel: %d query heads per kv head (1, 2 or 4 are served)", G);
    if (H / 256 > BK_WARPS || F / 256 > BK_MAX_NSB || hq * BK_ATT_D / 256 > BK_MAX_NSB)
        return jl_set_err(ctx, JL_DECLINED, "block kernel: hidden above %d or a row longer than %d elements", BK_WARPS * 256,
                          BK_MAX_NSB * 256);
    if (!d->cos_t || !d->sin_t) return JL_EINVAL;
    auto okw = [&](const jl_weight *w, int rows, int k) {
        return w && w->type == JL_TYPE_Q4_K && w->n_expert == 1 && w->nrows == rows && w->k == k && w->has_map_sb16;
    };
    for (int l = 0; l < L; l++) {
        const jl_layers_block &b = d->blocks[l];
        if (!okw(b.qkv, (hq + 2 * hkv) * BK_ATT_D, H) || !okw(b.o, H, hq * BK_ATT_D) || !okw(b.gate_up, 2 * F, H) ||
            !okw(b.down, H, F) || !b.k_cache || !b.v_cache)
            return jl_set_err(ctx, JL_DECLINED, "block %d: every projection must be a resident Q4_K matrix of the block's shape", l);
    }
    if (d->head && !okw(d->head, V, H)) return jl_set_err(ctx, JL_DECLINED, "head: not a resident Q4_K matrix %d x %d", V, H);
    if (5 * L + 2 > BK_MAX_PHASES) return jl_set_err(ctx, JL_DECLINED, "block kernel: more than %d blocks", (BK_MAX_PHASES - 2) / 5);

    int occ = 0;
    JL_CUDA(ctx, cudaFuncSetAttribute(jl_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BK_SMEM_BYTES));
    JL_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, jl_block_kernel, BK_THREADS, BK_SMEM_BYTES));
    if (occ < 1) return jl_set_err(ctx, JL_DECLINED, "block kernel does not fit an SM");

    jl_layers *S = new jl_layers();
    S->ctx = ctx; S->n_layer = L; S->hidden = H; S->hq = hq; S->hkv = hkv; S->ffn = F; S->vocab = V; S->max_len = d->max_len;
    S->rank = rank; S->world = world; S->grid = ctx->sm_count; S->attached = world == 1; S->buf = nullptr; S->slot = nullptr;
    const int nmaps = 4 * L + (d->head ? 1 : 0);
    const int nph = 5 * L + (d->head ? 2 : 0);
    const int nchunk_max = (d->max_len + 4 * BK_ATT_CHUNK - 1) / (4 * BK_ATT_CHUNK);   // records: one per block of four chunks
    const size_t stride = (size_t)(((2 * G + 3) & ~3) + G * BK_ATT_D);
    size_t off = 0;
    auto take = [&](size_t n) { size_t o = off; off += bk_al(n); return o; };
    const size_t o_ph = take((size_t)nph * sizeof(bk_phase)), o_maps = take((size_t)nmaps * sizeof(CUtensorMap));
    const size_t o_qkv = take((size_t)(hq + 2 * hkv) * BK_ATT_D * sizeof(bk_ll));
    const size_t o_att = take((size_t)hq * BK_ATT_D * sizeof(bk_ll)), o_a = take((size_t)F * sizeof(bk_ll));
    const size_t o_logits = take((size_t)(V > 0 ? V : 1) * 4);
    const size_t o_part = take((size_t)hkv * nchunk_max * stride * 4);
    const size_t o_cv = take((size_t)S->grid * 4), o_ci = take((size_t)S->grid * 4), o_seq = take(16);
    // zeroed in front of every launch: the grid barrier's counter, the abort word, every attention phase's tickets
    S->zero_bytes = 16 + (size_t)L * hkv * 4;
    const size_t o_bar = take(S->zero_bytes);
#ifdef BK_FINE_TRACE
    const size_t o_trace = take((size_t)2 * nph * 4 * 8 + (size_t)nph * 12 * 8 + (size_t)S->grid * 8 * 8 + (size_t)S->grid * nph * 4 * 8);
#else
    const size_t o_trace = take((size_t)2 * nph * 4 * 8 + (size_t)nph * 12 * 8 + (size_t)S->grid * 8 * 8);
#endif
    S->slot_bytes = bk_slot_bytes(world, H);
    cudaError_t e = cudaMalloc(&S->buf, off);
    if (e == cudaSuccess) e = cudaMalloc(&S->slot, S->slot_bytes);
    if (e == cudaSuccess) e = cudaMemset(S->buf, 0, off);
    if (e == cudaSuccess) e = cudaMemset(S->slot, 0, S->slot_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (S->buf) cudaFree(S->buf);
        if (S->slot) cudaFree(S->slot);
        delete S;
        return jl_set_err(ctx, JL_ENOMEM, "block kernel scratch (%zu bytes): %s", off, cudaGetErrorString(e));
    }
    uint8_t *B = S->buf;
    bk_ll *qkv = (bk_ll *)(B + o_qkv), *att = (bk_ll *)(B + o_att), *abuf = (bk_ll *)(B + o_a);
    bk_ll *planesO = (bk_ll *)S->slot, *planesD = (bk_ll *)(S->slot + bk_al((size_t)world * H * sizeof(bk_ll)));
    unsigned *tickets = (unsigned *)(B + o_bar + 16);
    S->logits = (float *)(B + o_logits);
    S->trace = (unsigned long long *)(B + o_trace);
    S->phases_dev = (bk_phase *)(B + o_ph);

    std::vector<CUtensorMap> maps(nmaps);
    bool maps_ok = true;
    auto map16 = [&](const jl_weight *w) { return w->map_sb16; };
    auto map8 = [&](const jl_weight *w, CUtensorMap *m) {
        const size_t rb = jl_row_bytes(w->type, w->k);
        return jl_make_tmap_2d(m, w->data, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rb, (uint64_t)w->nrows, rb, 144, 8,
                               CU_TENSOR_MAP_SWIZZLE_NONE);
    };
    S->phases.assign(nph, bk_phase());
    int pi = 0;
    for (int l = 0; l < L; l++) {
        const jl_layers_block &b = d->blocks[l];
        maps[4 * l + 0] = map16(b.qkv); maps[4 * l + 1] = map16(b.o);
        maps_ok = maps_ok && map8(b.gate_up, &maps[4 * l + 2]);
        maps[4 * l + 3] = map16(b.down);
        bk_phase q = {};
        q.kind = BK_MATVEC; q.map = 4 * l; q.nrows = (hq + 2 * hkv) * BK_ATT_D; q.nsb = H / 256; q.prologue = BK_PRO_NORM;
        q.epilogue = BK_EPI_STORE; q.from_emb = l == 0; q.planes = planesD; q.nplanes = l == 0 ? 0 : world;
        q.norm_w = b.attn_norm; q.out = qkv;
        S->phases[pi++] = q;
        bk_phase a = {};
        a.kind = BK_ATTN; a.qkv = qkv; a.att = att; a.k_cache = b.k_cache; a.v_cache = b.v_cache; a.tickets = tickets + (size_t)l * hkv;
        S->phases[pi++] = a;
        bk_phase o = {};
        o.kind = BK_MATVEC; o.map = 4 * l + 1; o.nrows = H; o.nsb = hq * BK_ATT_D / 256; o.prologue = BK_PRO_PLAIN; o.epilogue = BK_EPI_STORE;
        o.vsrc = att; o.out = planesO + (size_t)rank * H; o.exchange = world > 1;
        o.peer_out[rank] = o.out;
        S->phases[pi++] = o;
        bk_phase gu = {};
        gu.kind = BK_MATVEC; gu.map = 4 * l + 2; gu.nrows = F; gu.nsb = H / 256; gu.prologue = BK_PRO_NORM; gu.epilogue = BK_EPI_GATE2;
        gu.up_row0 = F; gu.planes = planesO; gu.nplanes = world; gu.norm_w = b.ffn_norm; gu.out = abuf;
        S->phases[pi++] = gu;
        bk_phase dn = {};
        dn.kind = BK_MATVEC; dn.map = 4 * l + 3; dn.nrows = H; dn.nsb = F / 256; dn.prologue = BK_PRO_PLAIN; dn.epilogue = BK_EPI_STORE;
        dn.vsrc = abuf; dn.out = planesD + (size_t)rank * H; dn.exchange = world > 1;
        dn.peer_out[rank] = dn.out;
        S->phases[pi++] = dn;
    }
    if (d->head) {
        maps[4 * L] = map16(d->head);
        bk_phase h = {};
        h.kind = BK_MATVEC; h.map = 4 * L; h.nrows = V; h.nsb = H / 256; h.prologue = BK_PRO_NORM; h.epilogue = BK_EPI_ARGMAX;
        h.planes = planesD; h.nplanes = world; h.norm_w = d->final_norm; h.out_f32 = S->logits;
        S->phases[pi++] = h;
        bk_phase f = {};
        f.kind = BK_FINAL;
        S->phases[pi++] = f;
    }
    e = cudaSuccess;
    if (maps_ok) e = cudaMemcpy(B + o_maps, maps.data(), (size_t)nmaps * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (maps_ok && e == cudaSuccess) e = cudaMemcpy(S->phases_dev, S->phases.data(), (size_t)nph * sizeof(bk_phase), cudaMemcpyHostToDevice);
    if (!maps_ok || e != cudaSuccess) {
        cudaGetLastError();
        cudaFree(S->buf); cudaFree(S->slot);
        delete S;
        return maps_ok ? jl_set_err(ctx, JL_ECUDA, "block kernel set-up: %s", cudaGetErrorString(e))
                       : jl_set_err(ctx, JL_DECLINED, "the driver refused a tensor map for a gate|up matrix");
    }
    bk_params &P = S->P;
    memset(&P, 0, sizeof P);
    P.phases = S->phases_dev; P.nphases = nph; P.maps = (const CUtensorMap *)(B + o_maps);
    P.hidden = H; P.hq = hq; P.hkv = hkv; P.max_len = d->max_len; P.eps = d->eps; P.cos_t = d->cos_t; P.sin_t = d->sin_t;
    P.emb = (const __nv_bfloat16 *)d->emb_bf16;
    P.part = (float *)(B + o_part); P.cand_val = (float *)(B + o_cv); P.cand_idx = (int *)(B + o_ci);
    P.bar = (unsigned *)(B + o_bar); P.abort_word = (int *)(B + o_bar) + 1; P.status = ctx->dev_status;
    P.rank = rank; P.world = world; P.seq = (unsigned *)(B + o_seq);
    *out = S;
    return JL_OK;
}

JL_EXPORT void jl_layers_free(jl_ctx *ctx, jl_layers *S) {
    if (!ctx || !S) return;
    std::lock_guard<std::mutex> lk(ctx->mu);
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (S->buf) cudaFree(S->buf);
    if (S->slot) cudaFree(S->slot);
    delete S;
}

// Where the other ranks store their partial sums and flags for this rank (device memory of this GPU).
JL_EXPORT int jl_tp_slot(jl_ctx *ctx, jl_layers *S, void **slot_dev, size_t *bytes) {
    if (!ctx || !S || !slot_dev || !bytes) return JL_EINVAL;
    *slot_dev = S->slot; *bytes = S->slot_bytes;
    return JL_OK;
}
// Handles for handing a slot to the other ranks' processes (CUDA IPC; 64 bytes each).
JL_EXPORT int jl_tp_ipc_export(const void *dev_ptr, void *handle64) {
    if (!dev_ptr || !handle64) return JL_EINVAL;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr)) != cudaSuccess) { cudaGetLastError(); return JL_ECOMM; }
    static_assert(sizeof h == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    return JL_OK;
}
JL_EXPORT int jl_tp_ipc_open(const void *handle64, void **dev_ptr) {
    if (!handle64 || !dev_ptr) return JL_EINVAL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    if (cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return JL_ECOMM; }
    return JL_OK;
}
JL_EXPORT int jl_tp_ipc_close(void *dev_ptr) {
    if (!dev_ptr) return JL_EINVAL;
    if (cudaIpcCloseMemHandle(dev_ptr) != cudaSuccess) { cudaGetLastError(); return JL_ECOMM; }
    return JL_OK;
}
// peer_slots[r] = rank r's slot as THIS process can address it (own slot at [rank]). After every rank has attached,
// the ranks meet once on the host (a barrier) before the first jl_layers_run.
JL_EXPORT int jl_tp_attach(jl_ctx *ctx, jl_layers *S, void *const *peer_slots, int n) {
    if (!ctx || !S || !peer_slots || n != S->world) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    if (peer_slots[S->rank] != S->slot) return jl_set_err(ctx, JL_EINVAL, "peer_slots[rank] must be this rank's own slot");
    const size_t plane = bk_al((size_t)S->world * S->hidden * sizeof(bk_ll));
    for (int r = 0; r < S->world; r++)
        if (!peer_slots[r]) return JL_EINVAL;
    for (int l = 0; l < S->n_layer; l++) {
        bk_phase &o = S->phases[5 * l + 2], &dn = S->phases[5 * l + 4];   // a block's phases: q|k|v, attention, o, gate|up, down
        for (int r = 0; r < S->world; r++) {
            o.peer_out[r] = (bk_ll *)peer_slots[r] + (size_t)S->rank * S->hidden;
            dn.peer_out[r] = (bk_ll *)((uint8_t *)peer_slots[r] + plane) + (size_t)S->rank * S->hidden;
        }
    }
    JL_CUDA(ctx, cudaMemcpy(S->phases_dev, S->phases.data(), S->phases.size() * sizeof(bk_phase), cudaMemcpyHostToDevice));
    S->attached = true;
    return JL_OK;
}

// Layers(0, n_layer, pos, 1, x, head) (engine/nn/device.go:1104-1118) with the residual row filled from the token
// id on the device (EmbedDevice, :1178-1191): one launch runs every block and, when a head was given, the output
// norm, the vocabulary projection and the greedy argmax. *tok_dev, *pos_dev are read on the device, so a captured
// graph can be replayed; with `advance` the kernel itself stores the next token into *tok_dev and increments
// *pos_dev. logits_out_dev / next_tok_dev may be NULL. Asynchronous on `stream`; poll jl_status_poll afterwards.
static int layers_run_locked(jl_ctx *ctx, jl_layers *S, long long *tok_dev, long long *pos_dev, float *logits_out_dev,
                             long long *next_tok_dev, int advance, void *stream, bool trace) {
    if (ctx->unhealthy) return jl_set_err(ctx, JL_ECUDA, "context is unhealthy after an earlier CUDA error");
    if (!S->attached) return jl_set_err(ctx, JL_ECOMM, "tensor-parallel blocks: jl_tp_attach has not been called");
    if (!S->P.emb) return jl_set_err(ctx, JL_EINVAL, "jl_layers_run needs the embedding table given at jl_layers_prep");
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t s = (cudaStream_t)stream;
    bk_params P = S->P;
    P.tok = tok_dev; P.pos = pos_dev; P.advance = advance; P.next_tok = next_tok_dev;
    P.trace = trace ? S->trace : nullptr;
    JL_CUDA(ctx, cudaMemsetAsync(P.bar, 0, S->zero_bytes, s));   // barrier counter, abort word, attention tickets
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;                               // all CTAs co-resident: the grid barriers rely on it
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S->grid); cfg.blockDim = dim3(BK_THREADS); cfg.dynamicSmemBytes = BK_SMEM_BYTES; cfg.stream = s;
    cfg.attrs = at; cfg.numAttrs = 1;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, jl_block_kernel, P));
    ctx->st.launches++;
    if (logits_out_dev && S->vocab > 0)
        JL_CUDA(ctx, cudaMemcpyAsync(logits_out_dev, S->logits, (size_t)S->vocab * 4, cudaMemcpyDeviceToDevice, s));
    ctx->st.served++;
    return JL_OK;
}

JL_EXPORT int jl_layers_run(jl_ctx *ctx, jl_layers *S, long long *tok_dev, long long *pos_dev, float *logits_out_dev,
                            long long *next_tok_dev, int advance, void *stream) {
    if (!ctx || !S || !tok_dev || !pos_dev) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return layers_run_locked(ctx, S, tok_dev, pos_dev, logits_out_dev, next_tok_dev, advance, stream, false);
}

// Per-phase nanoseconds of one step (the reference keeps per-op ns counters, model.OpProfile,
// engine/model/forward.go:22-75): runs ONE step like jl_layers_run (no advance), waits for it, and returns for every
// phase four global-timer stamps of the grid's first CTA and of its last: phase start, prologue done, work done,
// barrier passed -- stamps_out[2][n_phases][4]. Phases: per block qkv, attention, o, gate|up, down; then head, argmax.
JL_EXPORT int jl_layers_profile(jl_ctx *ctx, jl_layers *S, long long *tok_dev, long long *pos_dev, void *stream,
                                unsigned long long *stamps_out, int n_phases) {
    if (!ctx || !S || !tok_dev || !pos_dev || !stamps_out) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (n_phases != S->P.nphases) return jl_set_err(ctx, JL_EINVAL, "this stack has %d phases", S->P.nphases);
    size_t bytes = (size_t)2 * n_phases * 4 * 8;
#ifdef BK_FINE_TRACE
    // experimental builds: clock counts of the consume loop and the prologue, per-CTA attention stamps, every CTA's phase stamps
    bytes += (size_t)n_phases * 12 * 8 + (size_t)S->grid * 8 * 8 + (size_t)S->grid * n_phases * 4 * 8;
#endif
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    JL_CUDA(ctx, cudaMemsetAsync(S->trace, 0, bytes, (cudaStream_t)stream));
    int rc = layers_run_locked(ctx, S, tok_dev, pos_dev, nullptr, nullptr, 0, stream, true);
    if (rc) return rc;
    JL_CUDA(ctx, cudaMemcpyAsync(stamps_out, S->trace, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    JL_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return JL_OK;
}
JL_EXPORT int jl_layers_phases(jl_layers *S) { return S ? S->P.nphases : 0; }
