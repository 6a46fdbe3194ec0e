// Internal declarations shared by the translation units of libjitllm_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/jitllm_b200.h"

#define JL_EXPORT extern "C" __attribute__((visibility("default")))

// Block geometry, format/quant/types.go:61-85.
__host__ __device__ static inline int jl_block_elems(uint32_t t) {
    switch (t) {
    case JL_TYPE_Q8_0: case JL_TYPE_Q4_0: case JL_TYPE_Q5_0: case JL_TYPE_Q5_1: return 32;
    case JL_TYPE_Q4_K: case JL_TYPE_Q5_K: case JL_TYPE_Q6_K: return 256;
    case JL_TYPE_MXFP4: return 32;
    case JL_TYPE_F32: case JL_TYPE_F16: case JL_TYPE_BF16: return 1;
    }
    return 0;
}
__host__ __device__ static inline int jl_block_bytes(uint32_t t) {
    switch (t) {
    case JL_TYPE_Q8_0: return 34;
    case JL_TYPE_Q4_0: return 18;
    case JL_TYPE_Q5_0: return 22;
    case JL_TYPE_Q5_1: return 24;
    case JL_TYPE_Q4_K: return 144;
    case JL_TYPE_Q5_K: return 176;
    case JL_TYPE_Q6_K: return 210;
    case JL_TYPE_MXFP4: return 17;
    case JL_TYPE_F32: return 4;
    case JL_TYPE_F16: case JL_TYPE_BF16: return 2;
    }
    return 0;
}
// Formats that stay as raw ggml blocks on the device and run on the one-warp-per-row kernel only.
__host__ __device__ static inline bool jl_type_raw_simt(uint32_t t) {
    return t == JL_TYPE_Q4_0 || t == JL_TYPE_Q5_0 || t == JL_TYPE_Q5_1 || t == JL_TYPE_Q5_K || t == JL_TYPE_Q6_K;
}
static inline bool jl_type_served(uint32_t t) {
    return t == JL_TYPE_Q4_K || t == JL_TYPE_Q8_0 || t == JL_TYPE_MXFP4 || jl_type_raw_simt(t);
}
static inline size_t jl_row_bytes(uint32_t t, int k) {
    return (size_t)(k / jl_block_elems(t)) * (size_t)jl_block_bytes(t);
}

// A weight (or a bank of n_expert equal weights) resident on the device.
//
// Resident layouts (every repack is a byte permutation, shown bit-exact by
// jl_unpack_resident):
//   Q4_K   data = the raw 144-byte super-blocks, untouched. Rows are 16-byte
//          multiples, so every super-block is nine aligned 16-byte chunks.
//   Q8_0   data = int8 codes, [row][k/64 spans][4 lanes][16 B]; lane t's 16
//          bytes are four words: block 2s codes [4t,4t+4), block 2s codes
//          [16+4t,16+4t+4), then the same two of block 2s+1 -- the order in
//          which one mma.sync lane consumes them. scales = f16 d, [row][k/32].
//   MXFP4  data = the 16 code bytes of each block, [row][k/32][16];
//          scales = the e8m0 byte of each block, [row][scale_stride].
//   Q4_0, Q5_0, Q5_1, Q5_K, Q6_K   data = the raw blocks, untouched.
struct jl_weight {
    uint32_t type;
    int n_expert, nrows, k;
    size_t raw_bytes;       // bytes of the raw ggml tensor this came from
    uint8_t *data;
    uint8_t *scales;
    size_t data_bytes, scales_bytes;
    int scale_stride;       // elements per row of the scales plane
    const void *host_key;   // host address it was uploaded from (cache identity) or NULL
    // Q4_K: 2-D tensor map over the raw bytes, [n_expert * nrows][row_bytes] u8, box 144 B x 16
    // rows = one super-block of 16 rows per TMA copy (decode kernel).
    alignas(64) CUtensorMap map_sb16;
    bool has_map_sb16;
    int emin, emax;         // MXFP4: smallest / largest e8m0 byte of a block that is not all zeros
    // the host-pointer decode call's launches for this weight as an instantiated graph, with what it baked in
    void *zc_exec;          // cudaGraphExec_t or NULL
    void *zc_scratch, *zc_x, *zc_o;
    int zc_ntok, zc_form, zc_launches;
    uint32_t zc_flags;
};

struct jl_ctx {
    int device;
    jl_opts opts;
    cudaStream_t stream;
    std::mutex mu;          // serving calls: held across launches and, on the host-pointer calls, a stream sync
    std::mutex cache_mu;    // the residency map, the LRU list and the graveyard only: never held across device work
    std::string err;
    bool unhealthy;
    jl_stats st;
    int sm_count;
    // host-pointer residency: keyed on the host address (Device.MatVec's contract).
    std::map<uintptr_t, jl_weight *> cache;
    std::vector<uintptr_t> lru;
    std::vector<uintptr_t> pins;        // keys the running call is using: never evicted
    std::vector<jl_weight *> graveyard; // copies jl_forget dropped; freed by the next serving call
    void *moe_stage; size_t moe_stage_cap;   // jl_moe's device staging (h, logits, out, sel, wt, biases)
    int *stat_pin;          // pinned word the status rides home in
    // the decode call's zero-copy staging: pinned host memory the kernels read x from and write y to directly
    void *x_map; size_t x_map_cap;
    void *o_map; size_t o_map_cap;
    volatile int *done_map; // pinned {sequence number, status}: written by the call's last kernel, polled by the host
    int done_seq;
    // staging for the host entry points (grown by jl_reserve or on demand).
    void *x_dev; size_t x_cap;
    void *o_dev; size_t o_cap;
    void *scratch; size_t scratch_cap;
    void *x_pin; size_t x_pin_cap;
    void *o_pin; size_t o_pin_cap;
    int *dev_status;        // device words: [0] code a kernel sets when a bounded wait ran out, [1] the limit (us)
    // fault injection
    std::vector<int> fail_at;
    int call_ordinal;
    // measured selection (tune.cu)
    int tune_mode;                      // jl_tune_mode
    std::string tune_dir;               // where verdicts persist ("" = nowhere)
    char tune_devkey[17];               // GPU UUID + driver + build of this library, hashed
    std::map<uint64_t, int> tuned;      // (type, rows, k, tokens) -> decode variant
    int force_variant;                  // >= 0 while a trial times that variant
    int64_t tune_trials, tune_measured, tune_cached, tune_refused;
    int moe_bs_tma;                     // the last block-scaled mixture launch took its weights by TMA (1) or through registers (0)
};

static inline uint64_t jl_tune_shape_key(uint32_t type, int nrows, int k, int ntok) {
    return ((uint64_t)type << 56) ^ ((uint64_t)ntok << 48) ^ ((uint64_t)(uint32_t)nrows << 24) ^ (uint64_t)(uint32_t)k;
}
// tune.cu / gemv.cu
int jl_tune_shape_locked(jl_ctx *ctx, const jl_weight *w, int ntok);
int jl_gemv_tune_candidates(jl_ctx *ctx, int nrows, int k, int ntok, int *out, int cap);
int jl_gemv_variant_index(int form, int warps, int stages, int minb, int rg, int nsb);
void jl_gemv_variant_describe(int idx, int *form, int *warps, int *stages, int *minb, int *rg);

#define JL_CUDA(ctx, call)                                                           \
    do {                                                                             \
        cudaError_t e__ = (call);                                                    \
        if (e__ != cudaSuccess) {                                                    \
            jl_set_err((ctx), JL_ECUDA, "%s:%d %s: %s", __FILE__, __LINE__, #call,   \
                       cudaGetErrorString(e__));                                     \
            return JL_ECUDA;                                                         \
        }                                                                            \
    } while (0)

int jl_set_err(jl_ctx *ctx, int code, const char *fmt, ...);

// formats.cu
int jl_repack_upload(jl_ctx *ctx, uint32_t type, const void *w_host, size_t w_bytes, int n_expert,
                     int nrows, int k, jl_weight **out);
void jl_weight_release(jl_weight *w);

// gemv.cu -- decode kernels. x_dev [ntok][k] f32, out_dev [ntok][nrows] f32.
size_t jl_gemv_q8_scratch_bytes(int k, int ntok);
size_t jl_gemv_mxfp4_scratch_bytes(int k, int ntok);
int jl_launch_gemv_mxfp4(jl_ctx *ctx, float *out_dev, const uint8_t *codes, const uint8_t *eplane, int e_stride,
                         const float *x_dev, int nrows, int k, int ntok, cudaStream_t s);
void jl_gemv_q8_batch_plan(int nrows, int k, int *warps, int *slices);
int jl_launch_gemv_q8(jl_ctx *ctx, float *out_dev, const uint8_t *codes, const uint8_t *scales, int d_stride,
                      const float *x_dev, int nrows, int k, int ntok, cudaStream_t s);
int jl_launch_gemv(jl_ctx *ctx, float *out_dev, const jl_weight *w, int expert, const float *x_dev,
                   int ntok, int kernel, cudaStream_t s);
int jl_gemv_choice(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out);
size_t jl_gemv_scratch_bytes(uint32_t type, int k, int ntok);
int jl_grow_scratch(jl_ctx *ctx, size_t need);
// ctx.cu: device copy of a host bank keyed on its address (as jl_matvec does for one matrix)
int jl_resident_bank(jl_ctx *ctx, uint32_t type, const void *w, size_t w_bytes, int n_expert, int nrows, int k,
                     jl_weight **out);
void jl_resident_unpin(jl_ctx *ctx);
bool jl_resident_known(jl_ctx *ctx, const void *key, uint32_t type, int nrows, int k);
int jl_matmul_keyed(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const void *key, const void *raw, size_t raw_bytes,
                    const void *x, int x_dtype, int nrows, int k, int ntok);
void jl_drain_graveyard(jl_ctx *ctx);
int jl_read_status(jl_ctx *ctx, cudaStream_t s);

// gemm_tc5.cu -- prefill kernels (tcgen05).
int jl_gemm_tc5_operand(jl_ctx *ctx, const jl_weight *w, int ntok, void **rows, float **inv_scale);
int jl_launch_gemm_tc5(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, int expert,
                       const void *x_dev, int x_dtype, int ntok, cudaStream_t s);
int jl_gemm_tc5_supported(uint32_t type, int nrows, int k, int ntok);
int jl_gemm_tc5_choice(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out);
size_t jl_gemm_tc5_scratch_bytes(int nrows, int k, int ntok, int x_dtype, int sms);
