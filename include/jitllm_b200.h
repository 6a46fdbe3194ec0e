/*
 * jitllm_b200.h -- C ABI of libjitllm_b200.so
 *
 * A B200 (sm_100a) implementation of jitllm's quantized-matmul hot path, sitting
 * behind the seam the reference already has for accelerators: engine/nn's
 * Device.MatVec (engine/nn/device.go:23-31), the JIT.MatMul call site
 * (engine/nn/matmul.go:27) and the mixture-of-experts call sites
 * (engine/model/moe.go:502-760). Plain pointers and sizes only; a Go caller
 * reaches it through cgo or a dlopen FFI.
 *
 * Conventions
 *   - Every function returns a jl_status: 0 = served, 1 = DECLINED (a supported
 *     answer: the caller runs its own path, engine/nn/jit.go:935-940), < 0 = error.
 *   - The library never aborts, traps or reads the environment. Why the last
 *     call declined or failed is jl_last_error() (ErrReporter.Err,
 *     engine/nn/device.go:1592-1593).
 *   - Calls on one jl_ctx are serialised internally (the reference holds a
 *     per-device mutex across a matvec, jit/gpu/tier/tier.go:2842); different
 *     contexts are independent.
 *   - The caller owns every host buffer. The library owns device copies of
 *     weights and frees them on jl_forget / jl_weight_free / jl_close.
 *   - Quantized weights are RAW ggml blocks, row-major: nrows x (k / block_elems
 *     * block_bytes) bytes (format/quant/types.go:61-85).
 */
#ifndef JITLLM_B200_H
#define JITLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JL_ABI_VERSION 2

/* ggml type ids, format/quant/types.go:12-55. */
#define JL_TYPE_F32 0u
#define JL_TYPE_F16 1u
#define JL_TYPE_Q4_0 2u   /* 32 elements in 18 bytes  {f16 d; u8 qs[16]}               */
#define JL_TYPE_Q5_0 6u   /* 32 elements in 22 bytes  {f16 d; u32 qh; u8 qs[16]}       */
#define JL_TYPE_Q5_1 7u   /* 32 elements in 24 bytes  {f16 d, m; u32 qh; u8 qs[16]}    */
#define JL_TYPE_Q8_0 8u   /* 32 elements in 34 bytes  {f16 d; i8 qs[32]}              */
#define JL_TYPE_Q4_K 12u  /* 256 elements in 144 bytes {f16 d,dmin; u8 sc[12]; u8 qs[128]} */
#define JL_TYPE_Q5_K 13u  /* 256 elements in 176 bytes {f16 d,dmin; u8 sc[12]; u8 qh[32]; u8 qs[128]} */
#define JL_TYPE_Q6_K 14u  /* 256 elements in 210 bytes {u8 ql[128]; u8 qh[64]; i8 sc[16]; f16 d} */
#define JL_TYPE_BF16 30u
#define JL_TYPE_MXFP4 39u /* 32 elements in 17 bytes  {u8 e; u8 qs[16]}               */

typedef enum jl_status {
    JL_OK = 0,          /* served */
    JL_DECLINED = 1,    /* not an error: unsupported type/shape, too small to pay */
    JL_EINVAL = -1,
    JL_ECUDA = -2,      /* a CUDA call failed; the context reports unhealthy */
    JL_ENOMEM = -3,
    JL_EDEVICE = -4,    /* injected device failure (jl_test_fail_at) */
    JL_ETIMEDOUT = -5,  /* a bounded device-side wait ran out */
    JL_ENOTSUP = -6,
    JL_ECOMM = -7
} jl_status;

/* Element types of activations / outputs on the batched entry points. */
typedef enum jl_dtype { JL_DT_F32 = 0, JL_DT_F16 = 1, JL_DT_BF16 = 2 } jl_dtype;

/* Kernel families, reported by jl_select and pinnable through jl_opts: the
 * reference's per-shape selection (jit/gpu/tier/layer.go:10953-11016 batchMV,
 * jit/gpu/tier/tier.go:124-137 chooseSplit) maps onto these. */
typedef enum jl_kernel {
    JL_K_AUTO = 0,
    JL_K_SIMT = 1,   /* one warp per row, f32 FMA: every shape, the check kernel     */
    JL_K_MMA = 2,    /* decode on mma.sync: Q4_K/Q8_0 codes as u8/s8 against two int8 digits
                        of each activation (m16n8k32, s32), MXFP4 codes placed bit-wise into
                        f16 fragments (m16n8k16); scales folded in f32                    */
    JL_K_TC5 = 3     /* TMA -> smem dequant -> tcgen05.mma, TMEM accumulators: prefill */
} jl_kernel;

/* Gated activations of the mixture layer, jit/gpu/kernels/actkind.go:13-39. */
typedef enum jl_act { JL_ACT_SILU = 0, JL_ACT_SWIGLU_OAI = 1 } jl_act;

/* Options: the reference's libraries read no environment, every knob is a
 * With...() option (engine/nn/options.go:7-13). Zero-initialise, set
 * struct_size = sizeof(jl_opts), then override. */
/* Forms of the Q4_K tensor-core decode (JL_K_MMA). All share one arithmetic; they differ in who
 * converts the activation row into the kernel's operand (two int8 digits per value, in MMA
 * fragment order) and in how many rows a CTA covers. jl_select reports the form that runs. */
typedef enum jl_decode_form {
    JL_FORM_AUTO = 0,
    JL_FORM_SPLIT = 1, /* a prep launch converts x once; 16-row CTAs stage the operand in shared memory */
    JL_FORM_FUSED = 2, /* one launch; every 16-row CTA converts the super-blocks it consumes          */
    JL_FORM_WIDE = 3,  /* one launch; a CTA of 16 x row_groups rows converts the whole row once      */
    JL_FORM_L1 = 4     /* a prep launch; small CTAs hold weight tiles only and read the operand
                          through L1 (most weight bytes in flight: for overlapped matvecs)           */
} jl_decode_form;

typedef struct jl_opts {
    uint32_t struct_size;
    int32_t pin_kernel;        /* jl_kernel; JL_K_AUTO = per-shape selection          */
    int32_t pin_warps;         /* warps per CTA of the decode kernel; 0 = selected    */
    uint64_t min_weight_bytes; /* jl_matvec declines smaller weights (the reference's
                                  mvPays break-even, jit/gpu/tier/tier.go:2404-2424);
                                  0 = serve everything                                */
    uint64_t max_resident_bytes; /* cap on device copies kept for host-pointer calls;
                                  0 = no cap                                          */
    uint32_t flags;            /* JL_FLAG_* */
    int32_t decode_form;       /* jl_decode_form; pins the Q4_K decode form (the reference pins
                                  its choices with WithSplit etc., jit/gpu/tier/split.go:18-31) */
    int32_t pin_stages;        /* TMA ring depth per warp; 0 = the form's default     */
    int32_t pin_row_groups;    /* JL_FORM_WIDE: 16-row groups per CTA; 0 = default    */
    uint32_t wait_limit_us;    /* bound of every device-side wait, microseconds of the GPU's
                                  global timer; 0 = 2,000,000 (2 s)                   */
} jl_opts;

/* Launch decode kernels without programmatic dependent launch (by default a decode kernel
 * starts fetching its weights while its predecessor in the stream is still draining). */
#define JL_FLAG_NO_PDL 1u
/* Stream decode weights with per-lane 128-bit loads instead of TMA tile copies. */
#define JL_FLAG_NO_TMA 2u
/* The caller keeps several independent matvecs in flight on this GPU (streams, graph branches, experts): the
 * Q4_K decode then takes the variant with the most weight bytes in flight per SM (small CTAs, weight tiles
 * only in shared memory, the prepared activations read through L1) instead of the one with the shortest
 * single-launch latency. The arithmetic is the same; only the order in which the warps' f32 partial sums
 * meet can differ (each variant is run-to-run bit-stable). */
#define JL_FLAG_DECODE_CONCURRENT 16u

typedef struct jl_ctx jl_ctx;
typedef struct jl_weight jl_weight;

/* What would run for a shape (jl_select). */
typedef struct jl_choice {
    int32_t kernel;   /* jl_kernel */
    int32_t warps;    /* warps per CTA */
    int32_t rows_per_cta;
    int32_t split_k;  /* how many partial sums meet per output row */
    int32_t tile_m, tile_n, tile_k; /* tensor-core tile (rows, tokens, k) or 0 */
    int32_t grid;     /* CTAs of the main kernel */
    int32_t form;     /* jl_decode_form of a Q4_K JL_K_MMA choice, else 0 */
    int32_t stages;   /* TMA ring depth per warp, or 0 */
    int32_t launches; /* kernels one call launches (jl_stats.launches grows by this) */
} jl_choice;

/* Counters, the tier's Stats (jit/gpu/tier/tier.go:1246,2330). */
typedef struct jl_stats {
    uint64_t served, declined, errors;
    uint64_t uploads, upload_bytes, resident_bytes, forgets;
    uint64_t launches;       /* kernels this context launched */
    uint64_t injected;       /* failures injected by jl_test_fail_at */
} jl_stats;

const char *jl_version(void);
int jl_abi_version(void);

/* ---- context: tier.OpenWith (jit/gpu/tier/open.go:94) ------------------- */
int jl_open(int device, const jl_opts *opts, jl_ctx **out);
void jl_close(jl_ctx *ctx);
/* Device.Reserve (engine/nn/device.go:1169-1175): pre-size staging so nothing
 * grows on the serving path. */
int jl_reserve(jl_ctx *ctx, int max_rows, int max_k, int max_tok);
/* ErrReporter.Err (engine/nn/device.go:1592-1593). Valid until the next call on ctx. */
const char *jl_last_error(jl_ctx *ctx);
int jl_stats_get(jl_ctx *ctx, jl_stats *out);

/* ---- the decode operator: nn.Device.MatVec (engine/nn/device.go:23-31) --- */
/* out[0:nrows] = W x. w: raw ggml blocks on the HOST; x, out: host f32. The
 * device copy of w is keyed on (w, w_bytes): the first call uploads (and may
 * repack, bit-exactly), later calls reuse it. The caller guarantees the bytes
 * at w stay unchanged until jl_forget covers them. Types: Q4_K, Q8_0, MXFP4 on the tensor-core
 * decode kernels; Q4_0, Q5_0, Q5_1, Q5_K, Q6_K (what real Q4_K_M files mix in,
 * format/quant/dequant.go:85-146,399-470) on the one-warp-per-row kernel, which decodes each weight
 * exactly as quant.Dequant32 does. Any other type is DECLINED. */
int jl_matvec(jl_ctx *ctx, float *out, uint32_t type, const void *w, size_t w_bytes,
              const float *x, int nrows, int k);
/* CopyForgetter.Forget (engine/nn/device.go:1570-1581): drop every device copy
 * whose host range lies in [p, p+n). Any thread; never waits on device work
 * the caller did not start. */
int jl_forget(jl_ctx *ctx, const void *p, size_t n);

/* ---- the batched operator: JIT.MatMul (engine/nn/matmul.go:27) ----------- */
/* x is [ntok][k], out is [ntok][nrows], both token-major, host memory.
 * x_dtype / out_dtype: f32, f16 or bf16. Accumulation is f32. */
int jl_matmul(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const void *w, size_t w_bytes,
              const void *x, int x_dtype, int nrows, int k, int ntok);

/* ---- container-packed weights: nn.Packed{QS, D, SC, Row, Stride} (engine/nn/device.go:62-80) ----
 * What the reference's .jlm containers store and JIT.MatVecPacked / MatMulPacked read
 * (engine/nn/packed.go:24, engine/nn/packedmm.go:23): the blocks' fields as three planes laid out
 * [sub-block][word][row] by kernels.PackWeights (jit/gpu/kernels/pack.go:27-239). stride is the row
 * count of the whole buffer, row where this weight starts in it (both 0: the whole buffer). Served for
 * Q4_K, Q8_0 and MXFP4: the planes are re-interleaved once, at upload, into the raw blocks the kernels
 * stream (the exact inverse of PackWeights: jl_packed_to_blocks), so results are those of the raw
 * entry points bit for bit. Residency of the host calls is keyed on the payload plane (plus row);
 * jl_forget over the payload plane's bytes drops it. sc is NULL / 0 for formats without a
 * sub-block scale table (Q8_0, MXFP4). */
typedef struct jl_packed {
    const void *qs, *d, *sc;
    size_t qs_bytes, d_bytes, sc_bytes;
    int32_t row, stride;
} jl_packed;
int jl_packed_to_blocks(uint32_t type, const jl_packed *p, int nrows, int k, void *raw_out, size_t raw_bytes);
int jl_weight_upload_packed(jl_ctx *ctx, uint32_t type, const jl_packed *p, int nrows, int k, jl_weight **out);
int jl_matvec_packed(jl_ctx *ctx, float *out, uint32_t type, const jl_packed *p, const float *x, int nrows, int k);
int jl_matmul_packed(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const jl_packed *p, const void *x, int x_dtype,
                     int nrows, int k, int ntok);

/* ---- the mixture layer: State.moeBatch (engine/model/moe.go:502-760) ----- */
/* Banks are [n_expert][rows][k/32*17] raw MXFP4 blocks (banks of any other type are DECLINED):
 * gate, up: rows = ffn, k = hidden; down: rows = hidden, k = ffn.
 * Gate: softmax over all experts (internal/oracle/moe.go:204-262). Served: logit_bias (added to
 * the logits BEFORE the softmax, so it changes the weights too: gpt-oss), sel_bias (added to the
 * gated scores for the SELECTION only, the weights come from the unbiased scores: the
 * reference's MoEGate.Bias), norm, scale. Not served (no field; such a layer keeps its host
 * path): the sigmoid gate, per-expert ExpScale, grouped top-k. */
typedef struct jl_moe_desc {
    uint32_t struct_size;
    uint32_t type;                 /* bank block type */
    int32_t n_expert, top_k, hidden, ffn;
    int32_t act;                   /* jl_act */
    int32_t norm;                  /* renormalise by the selected sum (+1e-20), moetopk.go:137 */
    float scale;                   /* routed_scaling_factor; 0 or 1 = none */
    const void *gate, *up, *down;  /* host banks (jl_moe) or jl_weight handles (jl_moe_dev) */
    size_t gate_bytes, up_bytes, down_bytes;
    const float *gate_bias, *up_bias, *down_bias; /* [n_expert][rows] f32 or NULL */
    const float *router_bias;      /* logit bias [n_expert]: added to the logits before the softmax, or NULL */
    const float *sel_bias;         /* selection-only bias [n_expert] on the gated scores, or NULL */
    int32_t arm;                   /* jl_moe_arm; 0 = the exact-weights arm (the parity arm) */
} jl_moe_desc;
/* Numerics arms of the expert GEMMs (jl_moe, jl_moe_dev and jl_moe_experts_dev).
 * EXACT: MXFP4 weights dequantised exactly to f16, activations as f16 hi + lo, tcgen05 kind::f16: meets the
 * 2e-3 parity bar against the reference's f32-activation arithmetic. BLOCK_SCALED: tcgen05
 * kind::mxf8f6f4.block_scale on the e2m1 codes and e8m0 scales as they are, activations quantised per 32
 * elements to e4m3 with a ue8m0 scale -- faster (no warp converts a weight), but the activation
 * quantisation (3 mantissa bits) puts its error near 1e-2: it does NOT meet the parity bar and is never
 * selected implicitly. BLOCK_SCALED_X3: the same MMAs over THREE e4m3 digits per activation (digit d + 1 is
 * the e4m3 rounding of what digits 0..d leave; the digits share the block's scale and are three columns of
 * the tile, added when the accumulators are drained; bf16 input rows take two digits, which hold their 8
 * significant bits): 12 significant bits, weights and weight scales exact
 * as in the other arms, so it meets the 2e-3 parity bar at close to the one-digit arm's speed. No
 * counterpart in the reference (its grouped expert GEMM is mma.sync, jit/gpu/kernels/gemm70.go:123-129). */
typedef enum jl_moe_arm { JL_MOE_ARM_EXACT = 0, JL_MOE_ARM_BLOCK_SCALED = 1, JL_MOE_ARM_BLOCK_SCALED_X3 = 2 } jl_moe_arm;
/* 1 when the last block-scaled launch of this context took its weight tiles by TMA (packed 4-bit tensor maps),
 * 0 when the driver refused those maps and the codes went through registers. */
int jl_moe_bs_weights_by_tma(jl_ctx *ctx);
/* out[ntok][hidden] f32 += sum over each row's top_k experts, ascending expert
 * id, of w_e * down_e(act(gate_e h, up_e h)). logits [ntok][n_expert] f32 are
 * the router's raw outputs: softmax, lexicographic top-k (ties to the lowest
 * id), divisor summed in selection order (engine/nn/moetopk.go:316-385).
 * h is [ntok][hidden] in h_dtype. sel_out/wt_out ([ntok][top_k], selection
 * order) may be NULL. */
int jl_moe(jl_ctx *ctx, float *out, const void *h, int h_dtype, const float *logits, int ntok,
           const jl_moe_desc *desc, int32_t *sel_out, float *wt_out);

/* The router alone (softmax, lexicographic top-k, renormalised weights), device pointers:
 * engine/nn/moetopk.go:316-385. sel/wt are [ntok][top_k] in selection order. */
int jl_moe_route_dev(jl_ctx *ctx, const float *logits_dev, int ntok, const jl_moe_desc *desc,
                     int32_t *sel_out_dev, float *wt_out_dev, void *stream);
/* The experts alone over rows that are ALREADY routed: y[i] = down_e(act(gate_e h_i, up_e h_i)) with
 * e = expert_ids[i] (local index into the banks), written in the caller's row order. This is what an
 * expert-parallel rank runs on the rows it received (cf. LayerWeights.HostExpertsRows,
 * engine/nn/device.go:275-279). Scratch as jl_moe_reserve(nrows, n_expert, 1, hidden, ffn). */
int jl_moe_experts_dev(jl_ctx *ctx, float *y_dev, const void *h_dev, int h_dtype, const int32_t *expert_ids_dev,
                       int nrows, const jl_moe_desc *desc, void *stream);

/* Pre-size the mixture layer's scratch (token lists, gathered rows, intermediates) so that
 * jl_moe_dev never needs more than it finds. */
int jl_moe_reserve(jl_ctx *ctx, int ntok, int n_expert, int top_k, int hidden, int ffn);

/* ---- per-shape selection: batchMV / chooseSplit --------------------------
 * What a call with f32 activations of this shape launches (jl_matvec, jl_matvec_dev, jl_matmul* with
 * JL_DT_F32): selection and launch read the same table, and jl_stats.launches grows by
 * jl_choice.launches per served call. 16-bit activations take one MMA column per token instead
 * of two in the tcgen05 GEMM (tile_n / split_k may then differ). */
int jl_select(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out);

/* ---- measured selection: tuneSplit (jit/gpu/tier/split.go:18-75), the tune cache
 * (jit/gpu/tier/choose.go:196-216), WithTune / WithTuneCache ----------------------------------
 * With tuning on, the first upload of a (type, rows, k) shape times the admissible variants of its
 * decode kernel against the resident copy (one launch each, L2 flushed in front, 2 warm-up + 9 timed
 * rounds, CUDA events): a candidate whose sample is dispersed (IQR / median > 0.10) is refused, a
 * later candidate must beat the best so far by more than 1 %, and the table's pick is tried first,
 * so it wins every tie. The verdict overrides the table for jl_select and for the launch alike. It
 * persists in <cache_dir>/jl_select1 keyed by GPU UUID + driver version + build of this library;
 * an entry that does not parse or names a variant the shape cannot take is measured again and
 * overwritten. Contexts that pin a kernel or form, or set JL_FLAG_DECODE_CONCURRENT, do not tune.
 * Served today: the Q4_K decode kernel (1..8 tokens). */
typedef enum jl_tune_mode { JL_TUNE_OFF = 0, JL_TUNE_ON = 1, JL_TUNE_FORCE = 2 /* ignore persisted verdicts */ } jl_tune_mode;
int jl_tune_configure(jl_ctx *ctx, int mode, const char *cache_dir /* NULL: do not persist */);
/* Measure (or load) the verdict for w's shape at ntok tokens now; *out (may be NULL) = the choice. */
int jl_tune(jl_ctx *ctx, const jl_weight *w, int ntok, jl_choice *out);
/* out[0] timed launches, [1] shapes measured, [2] shapes answered from the file, [3] candidates refused. */
int jl_tune_stats(jl_ctx *ctx, int64_t out[4]);
/* The duel itself, host code: timer(user, candidate, round) returns a rate (higher is better; <= 0 =
 * the run failed). refused[c] / medians[c] may be NULL. Returns the winner or -1 when no candidate
 * gave a usable sample. */
int jl_tune_duel(int ncand, int nrounds, double (*timer)(void *user, int cand, int round), void *user,
                 double iqr_gate, double margin, int *refused, double *medians);
/* The verdict file: 1 = found / saved, 0 = not. */
int jl_tune_cache_lookup(const char *dir, const char *key, char *value, size_t cap);
int jl_tune_cache_save(const char *dir, const char *key, const char *value);
/* 16 hex digits identifying (GPU UUID, driver version, library build). */
void jl_tune_device_key(const void *uuid16, int driver_version, const char *build_id, char out[17]);
const char *jl_build_id(void);

/* ---- integer view of the blocks: kernels.extract (jit/gpu/kernels/pack.go:252-386)
 * One record per 32-element sub-block: q[32] codes (Q4_K 0..15, Q8_0 -128..127,
 * MXFP4 raw e2m1 code 0..15, Q4_0 0..15, Q5_0 / Q5_1 / Q5_K 0..31), raw f16 bits of d
 * (MXFP4: the stored byte e-1, pack.go:388-395) and dmin (Q5_1: its m with the sign bit
 * flipped, pack.go:275-290), the 6-bit sc and m. Q6_K: one record per SIXTEEN elements,
 * q[16] in 0..63 and sc = the int8 scale biased by 128 (pack.go:367-384). n_blocks counts
 * format blocks; q holds one code per element in every case.
 * jl_unpack runs on the host; jl_unpack_resident reads the DEVICE-RESIDENT
 * (possibly repacked) copy back through a kernel, which is how a repack is
 * shown to be bit-exact. Host output buffers in both. */
int jl_unpack(uint32_t type, const void *blocks, size_t n_blocks, int8_t *q, uint16_t *d_bits,
              uint16_t *dmin_bits, uint8_t *sc, uint8_t *m);
int jl_unpack_resident(jl_ctx *ctx, const jl_weight *w, int8_t *q, uint16_t *d_bits,
                       uint16_t *dmin_bits, uint8_t *sc, uint8_t *m);

/* ---- device-pointer twins: no host round trip ----------------------------
 * What tier.resident() does inside the reference (jit/gpu/tier/tier.go:2831-2903):
 * the weight lives on the device, activations and outputs are device pointers,
 * the launch goes on `stream` (a cudaStream_t; NULL is CUDA's default stream, as everywhere in
 * CUDA). Launches are asynchronous: the caller orders them with its own stream operations. */
int jl_weight_upload(jl_ctx *ctx, uint32_t type, const void *w_host, size_t w_bytes, int nrows,
                     int k, jl_weight **out);
/* As jl_weight_upload for a bank of n_expert equal matrices. */
int jl_weight_upload_bank(jl_ctx *ctx, uint32_t type, const void *w_host, size_t w_bytes,
                          int n_expert, int nrows, int k, jl_weight **out);
void jl_weight_free(jl_ctx *ctx, jl_weight *w);
/* x_dev [ntok][k] f32, out_dev [ntok][nrows] f32. ntok = 1 is the decode matvec. */
int jl_matvec_dev(jl_ctx *ctx, float *out_dev, const jl_weight *w, const float *x_dev, int ntok,
                  void *stream);
int jl_matmul_dev(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, const void *x_dev,
                  int x_dtype, int ntok, void *stream);
/* desc->gate/up/down are jl_weight* banks; biases and all other pointers are device pointers. */
int jl_moe_dev(jl_ctx *ctx, float *out_dev, const void *h_dev, int h_dtype, const float *logits_dev,
               int ntok, const jl_moe_desc *desc, int32_t *sel_out_dev, float *wt_out_dev, void *stream);

/* ---- allocation-free decode (no counterpart in the reference) -------------
 * out_dev[0:nrows] = W x for Q4_K, for callers that must not allocate device memory (inside a
 * stream capture, under a memory planner that forbids late cudaMalloc, in a latency-critical
 * loop). No context: w_dev is the raw ggml Q4_K tensor ALREADY on the device (16-byte
 * aligned), x_dev and out_dev are device f32, `stream` a cudaStream_t on the current device.
 * The kernel's scratch is a fixed array inside the library, so k is limited to
 * jl_noalloc_max_k() (16384); a larger k returns JL_ENOMEM. The call performs no cudaMalloc,
 * cudaFree or other allocating call. The first call on each device looks up the array's
 * address: make that call before starting a stream capture. All calls on a device share the
 * array, so calls that can overlap on the GPU (different streams) race; use one stream. */
int jl_noalloc_max_k(void);
int jl_matvec_q4k_noalloc(float *out_dev, const void *w_dev, const float *x_dev, int nrows, int k, void *stream);

/* ---- decode-step neighbours (no seam in the reference: its CPU engine runs these as Go loops,
 * engine/model/forward.go:2785 rmsnorm, engine/nn/ropetable.go:71 RopeTable) ----------------
 * Short device-pointer kernels that sit between two matvecs of a decode step, so that a caller
 * which keeps activations on the GPU chains the path with one launch in between: residual add +
 * RMSNorm, RoPE + KV-cache append, single-query attention over the cache, SiLU(gate)*up. They
 * join the same dependent-launch chain as the matvec kernels and allocate nothing.
 *   caches: bf16 [n][hkv][max_len][d]; *pos_dev: the position of the new token, read on the device
 *   (so a captured graph can be replayed while the caller increments it); cos/sin: f32 [max_len][d/2],
 *   adjacent-pair rotation; jl_aux_attn_decode needs d == 128 and a scratch of
 *   jl_aux_attn_scratch_bytes() bytes that was zero-filled once. */
int jl_aux_add_rmsnorm(float *x_io, const float *delta /* or NULL */, const float *w /* or NULL */, float eps,
                       float *out /* or NULL when operand_out is given */, void *operand_out, int n, int h, void *stream);
/* The batched counterpart: the normalised rows go out as the tcgen05 GEMM's activation operand (where jl_gemm_operand
 * said), and jl_matmul_dev_prepared consumes it: no conversion launch between the norm and the GEMM. h % 256 == 0. */
int jl_aux_add_rmsnorm_gemm(float *x_io, const float *delta /* or NULL */, const float *w /* or NULL */, float eps,
                            void *rows_f16, float *inv_scale, int n, int h, void *stream);
int jl_aux_silu_mul(float *out /* or NULL when operand_out is given */, void *operand_out,
                    const float *gate_up /* [n][2*ffn] */, int n, int ffn, void *stream);
int jl_aux_argmax(long long *out /* [n] */, const float *x /* [n][v] */, int n, int v, void *stream);
int jl_aux_rope_kv(void *q_out_bf16, const float *qkv, void *k_cache_bf16, void *v_cache_bf16,
                   const long long *pos_dev, const float *cos_t, const float *sin_t, int n, int hq, int hkv, int d,
                   int max_len, void *stream);
size_t jl_aux_attn_scratch_bytes(int n, int hq, int hkv, int max_len);
int jl_aux_attn_decode(float *out /* or NULL when operand_out is given */, void *operand_out, const void *q_bf16,
                       const void *k_cache_bf16, const void *v_cache_bf16, const long long *pos_dev,
                       void *scratch_zeroed_once, int n, int hq, int hkv, int d, int max_len, void *stream);

/* A producer can hand its result to the next Q4_K matvec without a conversion launch in between:
 * jl_decode_operand(ctx, w, ntok) names the place (inside ctx's scratch) where the decode kernel for weight
 * `w` expects its prepared activation operand, or NULL when that weight / token count has no such form;
 * the jl_aux_* kernels write it when given as `operand_out` (n must equal ntok, the row length w's k, a
 * multiple of 256; attention needs an even number of query heads per kv head); jl_matvec_dev_prepared then
 * runs the matvec on it. One operand per context at a time: produce, consume, then produce the next. The
 * pointer is valid until the context's scratch next grows (a weight upload, jl_reserve, jl_moe_reserve or a
 * host-pointer call): size the context first, then ask. */
void *jl_decode_operand(jl_ctx *ctx, const jl_weight *w, int ntok);
int jl_matvec_dev_prepared(jl_ctx *ctx, float *out_dev, const jl_weight *w, int ntok, void *stream);
/* The same for token counts that go to the tcgen05 GEMM: jl_gemm_operand names where a producer
 * (jl_aux_add_rmsnorm_gemm) writes the f16 hi / lo rows ([2 tok], [2 tok + 1], w->k halves each) and the per-token
 * 1/scale; JL_DECLINED when (w, ntok) is not served by the GEMM or the scratch is too small (jl_reserve).
 * jl_matmul_dev_prepared then runs the GEMM on what was written there. */
int jl_gemm_operand(jl_ctx *ctx, const jl_weight *w, int ntok, void **rows_f16, float **inv_scale);
int jl_matmul_dev_prepared(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, int ntok, void *stream);

/* ---- whole blocks in one submission: nn.LayerDevice (engine/nn/device.go:1096-1176) ------------
 * PrepLayer hands a block's weights to the device, Layers runs blocks [lo, hi) for the positions of one
 * step without the residual stream leaving the device, an optional Head continues the same submission
 * with the output norm and the vocabulary projection (device.go:1104-1118), and EmbedDevice fills the
 * residual row from the token id on the card (device.go:1178-1191). Here: ONE persistent kernel per decode
 * step of ONE sequence runs every block (fused: residual add + RMSNorm, q|k|v, RoPE + KV append,
 * attention over the cache, o, gate|up with SiLU(gate)*up, down), the head and the greedy argmax. The
 * weights are Q4_K jl_weight handles of this context (q|k|v and gate|up row-concatenated, as the
 * reference's MatVecSegments / Gate2 fuse them, jit/gpu/kernels/matvec.go:283-290); everything else is a
 * device pointer. Shapes the block kernel does not serve are DECLINED at prep and the caller keeps its
 * per-matvec path: head_dim must be 128, 1, 2 or 4 query heads per kv head, rows of at most 16384.
 * Tensor parallel (world > 1): q|k|v, gate|up and the head hold this rank's rows, o and down this rank's
 * k-range; the ranks exchange the row-parallel partial sums inside the kernel through peer-mapped slot
 * buffers (jl_tp_*), one process per GPU. */
typedef struct jl_layers jl_layers;
typedef struct jl_layers_block {
    const jl_weight *qkv, *o, *gate_up, *down;
    const float *attn_norm, *ffn_norm;   /* [hidden] f32, or NULL for all ones */
    void *k_cache, *v_cache;             /* bf16 [n_kv][max_len][128] of the one sequence */
} jl_layers_block;
typedef struct jl_layers_desc {
    uint32_t struct_size;
    int32_t n_layer, hidden, n_head, n_kv, head_dim, ffn, vocab, max_len; /* n_head, n_kv, ffn, vocab: THIS rank's share */
    float eps;
    const jl_layers_block *blocks;       /* host array [n_layer] */
    const jl_weight *head;               /* [vocab][hidden] or NULL: no head, no argmax */
    const float *final_norm;             /* [hidden] f32 or NULL */
    const void *emb_bf16;                /* [all token ids][hidden] bf16: the residual row of *tok */
    const float *cos_t, *sin_t;          /* f32 [max_len][64], adjacent-pair rotation */
    int32_t rank, world;                 /* tensor parallel; world <= 1: none */
} jl_layers_desc;
int jl_layers_prep(jl_ctx *ctx, const jl_layers_desc *desc, jl_layers **out);
void jl_layers_free(jl_ctx *ctx, jl_layers *layers);
/* One decode step. *tok_dev (token id) and *pos_dev (its position) are read ON THE DEVICE, so a captured
 * graph can be replayed; with advance != 0 the kernel stores the next token into *tok_dev and increments
 * *pos_dev itself. logits_out_dev ([vocab] f32) and next_tok_dev may be NULL. Asynchronous on `stream`;
 * a wait that ran out inside the kernel is reported by jl_status_poll. */
int jl_layers_run(jl_ctx *ctx, jl_layers *layers, long long *tok_dev, long long *pos_dev, float *logits_out_dev,
                  long long *next_tok_dev, int advance, void *stream);

/* Per-phase timing of one step, the reference's per-op nanosecond counters (model.OpProfile,
 * engine/model/forward.go:22-75): runs one step (no advance), waits for it and returns, for every phase,
 * four GPU global-timer stamps (ns) of the grid's first and last CTA -- phase start, prologue done, work
 * done, barrier passed: stamps_out[2][jl_layers_phases()][4] in host memory. Phases per block: q|k|v,
 * attention, o, gate|up, down; then the head and the argmax. */
int jl_layers_phases(jl_layers *layers);
int jl_layers_profile(jl_ctx *ctx, jl_layers *layers, long long *tok_dev, long long *pos_dev, void *stream,
                      unsigned long long *stamps_out, int n_phases);

/* ---- tensor-parallel exchange without a collective library (no counterpart in the reference, which has
 * no tensor parallelism: docs/perf/current.md:582) ------------------------------------------------
 * Each rank owns a slot buffer (jl_tp_slot) that the other ranks' kernels store their partial sums and a
 * sequence flag into with plain peer stores over NVLink. One process per GPU: export the slot as a 64-byte
 * CUDA IPC handle, exchange the handles by any host channel, open the peers' handles, hand all world
 * pointers (own slot at [rank]) to jl_tp_attach, then meet once on the host before the first step. In
 * one process with peer access enabled the raw pointers can be attached directly. */
int jl_tp_slot(jl_ctx *ctx, jl_layers *layers, void **slot_dev, size_t *bytes);
int jl_tp_ipc_export(const void *dev_ptr, void *handle64);
int jl_tp_ipc_open(const void *handle64, void **dev_ptr);
int jl_tp_ipc_close(void *dev_ptr);
int jl_tp_attach(jl_ctx *ctx, jl_layers *layers, void *const *peer_slots, int n);

/* ---- bounded device waits ---------------------------------------------------
 * Every wait inside a kernel of this library (an mbarrier a copy completes, a ring slot, a grid
 * barrier, a peer's flag) gives up after jl_opts.wait_limit_us of the GPU's global timer, records a
 * code in a status word of the context and lets the kernel return; the output of that launch is
 * then incomplete. The host-pointer calls read the word themselves and return JL_ETIMEDOUT. After
 * device-pointer calls the caller polls it: jl_status_poll enqueues a copy of the word on
 * `stream`, waits for that stream, clears the word when it was set and returns JL_OK or
 * JL_ETIMEDOUT (jl_last_error names the code). Not to be called during a stream capture. This
 * mirrors the reference's rule that a failed device call is a decline the caller sees
 * (engine/nn/device.go:1592-1593), never a wedged stream. */
int jl_status_poll(jl_ctx *ctx, void *stream);
/* The same for jl_matvec_q4k_noalloc's status word on the current device (allocates nothing). */
int jl_noalloc_status(void *stream);
/* Test-only: a one-thread kernel waits on an mbarrier that nothing ever completes, with
 * `limit_us` as its bound, and records the timeout; jl_status_poll then reports it. The GPU is
 * not faulted and the context stays usable. */
int jl_test_wait_timeout(jl_ctx *ctx, uint32_t limit_us, void *stream);
/* Measurement helper: `iters` passes over `nw` weights, one jl_matvec per weight (host pointers in and out,
 * exactly the public call), issued from a loop inside the library so that the caller's language adds nothing
 * to the time. *seconds = wall clock of the loop. Stops at the first call that is not served and returns its
 * status. */
int jl_test_matvec_loop(jl_ctx *ctx, float *out, uint32_t type, const void *const *ws, size_t w_bytes, const float *x,
                        int nrows, int k, int nw, int iters, double *seconds);

/* ---- host-side fault injection: JITLLM_DEVICE_FAIL_AT (jit/gpu/tier/fault.go:12-58)
 * The n-th, ... serving calls on ctx (1-based ordinals, counted from this call)
 * fail with JL_EDEVICE before anything is launched. n = 0 disarms. Test-only. */
int jl_test_fail_at(jl_ctx *ctx, const int *ordinals, int n);

#ifdef __cplusplus
}
#endif
#endif /* JITLLM_B200_H */
