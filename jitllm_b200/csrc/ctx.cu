// The C ABI: contexts, residency keyed on host addresses, the host-pointer and
// device-pointer entry points, selection, statistics, host-side fault injection.
#include "jl_internal.cuh"

#include <chrono>
#include "tma.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>

int jl_set_err(jl_ctx *ctx, int code, const char *fmt, ...) {
    if (ctx) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        ctx->err = buf;
        if (code == JL_DECLINED) ctx->st.declined++;
        else if (code < 0) ctx->st.errors++;
    }
    return code;
}

JL_EXPORT const char *jl_version(void) { return "jitllm_b200 0.1 (sm_100a)"; }
JL_EXPORT int jl_abi_version(void) { return JL_ABI_VERSION; }

JL_EXPORT int jl_open(int device, const jl_opts *opts, jl_ctx **out) {
    if (!out) return JL_EINVAL;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) {
        cudaGetLastError();
        return JL_ECUDA;  // no usable device: there is deliberately no CPU fallback
    }
    if (cudaSetDevice(device) != cudaSuccess) return JL_ECUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return JL_ECUDA;
    if (prop.major != 10) return JL_ENOTSUP;  // built for sm_100a only
    jl_ctx *c = new jl_ctx();
    c->device = device;
    memset(&c->opts, 0, sizeof c->opts);
    if (opts) memcpy(&c->opts, opts, std::min<size_t>(opts->struct_size, sizeof(jl_opts)));
    c->unhealthy = false;
    memset(&c->st, 0, sizeof c->st);
    c->sm_count = prop.multiProcessorCount;
    c->x_dev = c->o_dev = c->scratch = c->x_pin = c->o_pin = nullptr;
    c->x_cap = c->o_cap = c->scratch_cap = c->x_pin_cap = c->o_pin_cap = 0;
    c->call_ordinal = 0;
    c->tune_mode = JL_TUNE_OFF; c->tune_devkey[0] = 0; c->force_variant = -1;
    c->tune_trials = c->tune_measured = c->tune_cached = c->tune_refused = 0;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete c;
        return JL_ECUDA;
    }
    c->dev_status = nullptr;
    c->stat_pin = nullptr;
    c->moe_stage = nullptr; c->moe_stage_cap = 0;
    c->x_map = c->o_map = nullptr; c->x_map_cap = c->o_map_cap = 0; c->done_map = nullptr; c->done_seq = 0;
    const int words[4] = {0, (int)c->opts.wait_limit_us, 0, 0};   // code, wait limit, the done kernel's sequence counter, spare
    if (cudaMalloc(&c->dev_status, sizeof words) != cudaSuccess ||
        cudaMemcpy(c->dev_status, words, sizeof words, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMallocHost(&c->stat_pin, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        if (c->dev_status) cudaFree(c->dev_status);
        cudaStreamDestroy(c->stream);
        delete c;
        return JL_ECUDA;
    }
    *out = c;
    return JL_OK;
}

JL_EXPORT void jl_close(jl_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->cache) jl_weight_release(kv.second);
    ctx->cache.clear();
    for (jl_weight *w : ctx->graveyard) jl_weight_release(w);
    ctx->graveyard.clear();
    if (ctx->moe_stage) cudaFree(ctx->moe_stage);
    if (ctx->stat_pin) cudaFreeHost(ctx->stat_pin);
    if (ctx->x_map) cudaFreeHost(ctx->x_map);
    if (ctx->o_map) cudaFreeHost(ctx->o_map);
    if (ctx->done_map) cudaFreeHost((void *)ctx->done_map);
    if (ctx->x_dev) cudaFree(ctx->x_dev);
    if (ctx->o_dev) cudaFree(ctx->o_dev);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->x_pin) cudaFreeHost(ctx->x_pin);
    if (ctx->o_pin) cudaFreeHost(ctx->o_pin);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

JL_EXPORT const char *jl_last_error(jl_ctx *ctx) { return ctx ? ctx->err.c_str() : "no context"; }

JL_EXPORT int jl_stats_get(jl_ctx *ctx, jl_stats *out) {
    if (!ctx || !out) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    std::lock_guard<std::mutex> lk2(ctx->cache_mu);
    *out = ctx->st;
    return JL_OK;
}

static int grow_dev(jl_ctx *ctx, void **p, size_t *cap, size_t need) {
    if (*cap >= need) return JL_OK;
    if (*p) { cudaFree(*p); *p = nullptr; *cap = 0; }
    cudaError_t e = cudaMalloc(p, need);
    if (e != cudaSuccess) { cudaGetLastError(); return jl_set_err(ctx, JL_ENOMEM, "cudaMalloc(%zu): %s", need, cudaGetErrorString(e)); }
    *cap = need;
    return JL_OK;
}
static int grow_pin(jl_ctx *ctx, void **p, size_t *cap, size_t need) {
    if (*cap >= need) return JL_OK;
    if (*p) { cudaFreeHost(*p); *p = nullptr; *cap = 0; }
    cudaError_t e = cudaMallocHost(p, need);
    if (e != cudaSuccess) { cudaGetLastError(); return jl_set_err(ctx, JL_ENOMEM, "cudaMallocHost(%zu): %s", need, cudaGetErrorString(e)); }
    *cap = need;
    return JL_OK;
}

// Device scratch of the decode kernels (the prepared activation operand). It only ever
// grows, and only here: at weight upload, in jl_reserve and before a host-pointer call,
// never inside a device-pointer call (which may be under stream capture).
int jl_grow_scratch(jl_ctx *ctx, size_t need) {
    if (ctx->scratch_cap >= need) return JL_OK;
    cudaError_t e = cudaDeviceSynchronize();  // an earlier launch may still read the old buffer
    if (e != cudaSuccess) return jl_set_err(ctx, JL_ECUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    return grow_dev(ctx, &ctx->scratch, &ctx->scratch_cap, need);
}

static int grow_map(jl_ctx *ctx, void **p, size_t *cap, size_t need) {
    if (*cap >= need) return JL_OK;
    if (*p) { cudaStreamSynchronize(ctx->stream); cudaFreeHost(*p); *p = nullptr; *cap = 0; }
    cudaError_t e = cudaHostAlloc(p, need, cudaHostAllocMapped);
    if (e != cudaSuccess) { cudaGetLastError(); return jl_set_err(ctx, JL_ENOMEM, "cudaHostAlloc(%zu): %s", need, cudaGetErrorString(e)); }
    *cap = need;
    return JL_OK;
}

static int reserve_locked(jl_ctx *ctx, size_t x_bytes, size_t o_bytes) {
    int rc;
    // the decode call's zero-copy staging (a few tokens at most)
    if ((rc = grow_map(ctx, &ctx->x_map, &ctx->x_map_cap, x_bytes < (1u << 20) ? x_bytes : (1u << 20)))) return rc;
    if ((rc = grow_map(ctx, &ctx->o_map, &ctx->o_map_cap, o_bytes < (1u << 22) ? o_bytes : (1u << 22)))) return rc;
    if (!ctx->done_map) {
        void *p = nullptr;
        if (cudaHostAlloc(&p, 64, cudaHostAllocMapped) != cudaSuccess) { cudaGetLastError(); return jl_set_err(ctx, JL_ENOMEM, "cudaHostAlloc(64)"); }
        memset(p, 0, 64);
        ctx->done_map = (volatile int *)p;
    }
    if ((rc = grow_dev(ctx, &ctx->x_dev, &ctx->x_cap, x_bytes))) return rc;
    if ((rc = grow_dev(ctx, &ctx->o_dev, &ctx->o_cap, o_bytes))) return rc;
    if ((rc = grow_pin(ctx, &ctx->x_pin, &ctx->x_pin_cap, x_bytes))) return rc;
    if ((rc = grow_pin(ctx, &ctx->o_pin, &ctx->o_pin_cap, o_bytes))) return rc;
    return JL_OK;
}

JL_EXPORT int jl_reserve(jl_ctx *ctx, int max_rows, int max_k, int max_tok) {
    if (!ctx || max_rows < 1 || max_k < 1 || max_tok < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    const int k256 = (max_k + 255) / 256 * 256;
    const int dtok = max_tok < 8 ? max_tok : 8;
    size_t need = jl_gemv_scratch_bytes(JL_TYPE_Q4_K, k256, dtok);      // the decode kernels' operand, any format
    for (uint32_t t : {JL_TYPE_Q8_0, JL_TYPE_MXFP4}) {
        const size_t n = jl_gemv_scratch_bytes(t, k256, t == JL_TYPE_Q8_0 ? (max_tok < 32 ? max_tok : 32) : dtok);
        if (n > need) need = n;
    }
    // The GEMM's split-K partial planes are largest for SMALL row counts (few tiles -> many K splits), so the
    // worst case over every row count up to max_rows is taken, for both activation widths.
    size_t need_gemm = 0;
    for (int r = 256;; r += 256) {
        const int rows = r < max_rows ? r : max_rows;
        for (int dt : {JL_DT_F32, JL_DT_BF16}) {
            const size_t n = jl_gemm_tc5_scratch_bytes(rows, k256, max_tok, dt, ctx->sm_count);
            if (n > need_gemm) need_gemm = n;
        }
        if (rows == max_rows) break;
    }
    if (max_tok > 8 && need_gemm > need) need = need_gemm;
    int rc = jl_grow_scratch(ctx, need);
    if (rc) return rc;
    return reserve_locked(ctx, (size_t)max_tok * max_k * 4, (size_t)max_tok * max_rows * 4);
}

// Serving calls share this prologue: health, fault injection.
static int serving_prologue(jl_ctx *ctx) {
    if (ctx->unhealthy) return jl_set_err(ctx, JL_ECUDA, "context is unhealthy after an earlier CUDA error");
    jl_drain_graveyard(ctx);
    ctx->call_ordinal++;
    for (int o : ctx->fail_at)
        if (o == ctx->call_ordinal) {
            ctx->st.injected++;
            return jl_set_err(ctx, JL_EDEVICE, "injected device failure at call %d", o);
        }
    return JL_OK;
}

JL_EXPORT int jl_test_fail_at(jl_ctx *ctx, const int *ordinals, int n) {
    if (!ctx || n < 0 || (n > 0 && !ordinals)) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->fail_at.assign(ordinals, ordinals + n);
    ctx->call_ordinal = 0;
    return JL_OK;
}

// ---------------------------------------------------------------- residency
// The map, the LRU list, the pins and the graveyard are guarded by cache_mu, which is never held
// across device work; serving calls additionally hold ctx->mu.

// Frees what jl_forget dropped. Runs at the start of a serving call (which holds ctx->mu, so no
// launch of this context is being issued); the copies were unlinked from the map when they were
// forgotten, so nothing can pick them up any more. cudaFree waits for the device by itself.
void jl_drain_graveyard(jl_ctx *ctx) {
    std::vector<jl_weight *> dead;
    {
        std::lock_guard<std::mutex> lk(ctx->cache_mu);
        dead.swap(ctx->graveyard);
    }
    for (jl_weight *w : dead) jl_weight_release(w);
}

// Makes room for `incoming` bytes under the cap by releasing least-recently-used copies that the
// running call does not use. False when the pinned copies alone leave no room. cache_mu held.
static bool evict_for(jl_ctx *ctx, size_t incoming, std::vector<jl_weight *> &dead) {
    const uint64_t cap = ctx->opts.max_resident_bytes;
    if (!cap) return true;
    size_t i = 0;
    while (ctx->st.resident_bytes + incoming > cap && i < ctx->lru.size()) {
        const uintptr_t key = ctx->lru[i];
        if (std::find(ctx->pins.begin(), ctx->pins.end(), key) != ctx->pins.end()) { i++; continue; }
        ctx->lru.erase(ctx->lru.begin() + i);
        auto it = ctx->cache.find(key);
        if (it == ctx->cache.end()) continue;
        ctx->st.resident_bytes -= it->second->raw_bytes;
        dead.push_back(it->second);      // freed by the caller once cache_mu is released
        ctx->cache.erase(it);
    }
    return ctx->st.resident_bytes + incoming <= cap;
}

static void touch(jl_ctx *ctx, uintptr_t key) {
    auto it = std::find(ctx->lru.begin(), ctx->lru.end(), key);
    if (it != ctx->lru.end()) ctx->lru.erase(it);
    ctx->lru.push_back(key);
}

// The device copy of a host tensor, keyed on its address (Device.MatVec's
// contract, engine/nn/device.go:25-30). A different shape or type at a known
// address means the caller reused the memory without telling us: re-upload.
// The copy stays pinned (safe from eviction) until jl_resident_unpin.
static int resident(jl_ctx *ctx, uint32_t type, const void *w, size_t w_bytes, int n_expert, int nrows,
                    int k, jl_weight **out, const void *key_ptr = nullptr) {
    // key_ptr: the address residency is keyed on when it is not the source bytes' own (a packed weight is keyed on
    // its payload plane while the bytes uploaded are the re-interleaved blocks); w may then be NULL for a lookup.
    const uintptr_t key = (uintptr_t)(key_ptr ? key_ptr : w);
    const size_t need = (size_t)n_expert * nrows * jl_row_bytes(type, k);
    std::vector<jl_weight *> dead;
    bool fits = true;
    {
        std::lock_guard<std::mutex> lk(ctx->cache_mu);
        auto it = ctx->cache.find(key);
        if (it != ctx->cache.end()) {
            jl_weight *c = it->second;
            if (c->type == type && c->nrows == nrows && c->k == k && c->n_expert == n_expert) {
                touch(ctx, key);
                ctx->pins.push_back(key);
                *out = c;
                return JL_OK;
            }
            ctx->st.resident_bytes -= c->raw_bytes;
            auto l = std::find(ctx->lru.begin(), ctx->lru.end(), key);
            if (l != ctx->lru.end()) ctx->lru.erase(l);
            dead.push_back(c);
            ctx->cache.erase(it);
        }
        fits = evict_for(ctx, need, dead);
    }
    for (jl_weight *d : dead) jl_weight_release(d);   // the caller holds ctx->mu: no launch of this context is in flight
    if (!fits)
        return jl_set_err(ctx, JL_ENOMEM, "%zu weight bytes do not fit under max_resident_bytes = %llu beside the "
                          "copies this call already uses", need, (unsigned long long)ctx->opts.max_resident_bytes);
    if (!w) return jl_set_err(ctx, JL_EINVAL, "no resident copy under this key and no bytes to upload");
    jl_weight *nw = nullptr;
    int rc = jl_repack_upload(ctx, type, w, w_bytes, n_expert, nrows, k, &nw);   // device work: cache_mu released
    if (rc) return rc;
    nw->host_key = (const void *)key;
    std::lock_guard<std::mutex> lk(ctx->cache_mu);
    ctx->cache[key] = nw;
    touch(ctx, key);
    ctx->pins.push_back(key);
    ctx->st.resident_bytes += nw->raw_bytes;
    *out = nw;
    return JL_OK;
}

int jl_resident_bank(jl_ctx *ctx, uint32_t type, const void *w, size_t w_bytes, int n_expert, int nrows, int k,
                     jl_weight **out) {
    return resident(ctx, type, w, w_bytes, n_expert, nrows, k, out);
}
void jl_resident_unpin(jl_ctx *ctx) {
    std::lock_guard<std::mutex> lk(ctx->cache_mu);
    ctx->pins.clear();
}

// Forget never waits for the device (engine/nn/device.go:1575-1578): it takes only the small cache
// mutex, unlinks the copies so that no later call can find them, and leaves the cudaFree to the next
// serving call on this context (or jl_close). A call that is using one of them right now holds a pin:
// its copy is unlinked too, and freed after that call has finished.
JL_EXPORT int jl_forget(jl_ctx *ctx, const void *p, size_t n) {
    if (!ctx) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->cache_mu);
    uintptr_t lo = (uintptr_t)p, hi = lo + n;
    // Every copy whose host range intersects [p, p+n).
    for (auto it = ctx->cache.begin(); it != ctx->cache.end();) {
        uintptr_t a = it->first, b = a + it->second->raw_bytes;
        if (a < hi && b > lo) {
            ctx->st.resident_bytes -= it->second->raw_bytes;
            auto l = std::find(ctx->lru.begin(), ctx->lru.end(), a);
            if (l != ctx->lru.end()) ctx->lru.erase(l);
            ctx->graveyard.push_back(it->second);
            it = ctx->cache.erase(it);
            ctx->st.forgets++;
        } else {
            ++it;
        }
    }
    return JL_OK;
}

JL_EXPORT int jl_weight_upload_bank(jl_ctx *ctx, uint32_t type, const void *w_host, size_t w_bytes,
                                    int n_expert, int nrows, int k, jl_weight **out) {
    if (!ctx || !w_host || !out) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    int rc = jl_grow_scratch(ctx, jl_gemv_scratch_bytes(type, k, type == JL_TYPE_Q8_0 ? 32 : 8));
    if (rc) return rc;
    rc = jl_repack_upload(ctx, type, w_host, w_bytes, n_expert, nrows, k, out);
    if (rc == JL_OK) {
        std::lock_guard<std::mutex> lk2(ctx->cache_mu);
        ctx->st.resident_bytes += (*out)->raw_bytes;
    }
    // measured selection: the decode variant of a new shape is timed here, against the copy that will be read
    if (rc == JL_OK && ctx->tune_mode != JL_TUNE_OFF) jl_tune_shape_locked(ctx, *out, 1);
    return rc;
}

JL_EXPORT int jl_weight_upload(jl_ctx *ctx, uint32_t type, const void *w_host, size_t w_bytes, int nrows,
                               int k, jl_weight **out) {
    return jl_weight_upload_bank(ctx, type, w_host, w_bytes, 1, nrows, k, out);
}

JL_EXPORT void jl_weight_free(jl_ctx *ctx, jl_weight *w) {
    if (!ctx || !w) return;
    std::lock_guard<std::mutex> lk(ctx->mu);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    {
        std::lock_guard<std::mutex> lk2(ctx->cache_mu);
        ctx->st.resident_bytes -= w->raw_bytes;
    }
    jl_weight_release(w);
}

// ---------------------------------------------------------------- selection

static int choose(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out) {
    int pin = ctx->opts.pin_kernel;
    // the decode kernels serve up to 8 tokens; Q8_0 has a batch kernel for up to 32 (one pass over the weights,
    // no conversion of the codes: at 32 tokens the GEMM's fixed cost is several times that kernel's whole run)
    const int decode_max = (type == JL_TYPE_Q8_0 && k % 256 == 0) ? 32 : 8;
    if ((pin == JL_K_TC5 || (pin == JL_K_AUTO && ntok > decode_max)) && jl_gemm_tc5_supported(type, nrows, k, ntok))
        return jl_gemm_tc5_choice(ctx, type, nrows, k, ntok, out);
    if (pin == JL_K_TC5) return JL_DECLINED;
    return jl_gemv_choice(ctx, type, nrows, k, ntok, out);
}

JL_EXPORT int jl_select(jl_ctx *ctx, uint32_t type, int nrows, int k, int ntok, jl_choice *out) {
    if (!ctx || !out) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    int be = jl_block_elems(type);
    if (!jl_type_served(type) || nrows < 1 || k < be || k % be || ntok < 1)
        return jl_set_err(ctx, JL_DECLINED, "no kernel for type %u, %d x %d, %d token(s)", type, nrows, k, ntok);
    return choose(ctx, type, nrows, k, ntok, out);
}

// ------------------------------------------------------------ device twins

static int matmul_dev_locked(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, int expert,
                             const void *x_dev, int x_dtype, int ntok, cudaStream_t s) {
    jl_choice ch;
    int rc = choose(ctx, w->type, w->nrows, w->k, ntok, &ch);
    if (rc) return rc == JL_DECLINED ? jl_set_err(ctx, JL_DECLINED, "pinned kernel cannot serve this shape") : rc;
    if (ch.kernel == JL_K_TC5)
        return jl_launch_gemm_tc5(ctx, out_dev, out_dtype, w, expert, x_dev, x_dtype, ntok, s);
    if (x_dtype != JL_DT_F32 || out_dtype != JL_DT_F32) {
        // 16-bit activations or outputs: the GEMM converts them, the decode kernels do not
        if (ctx->opts.pin_kernel == JL_K_AUTO && jl_gemm_tc5_supported(w->type, w->nrows, w->k, ntok))
            return jl_launch_gemm_tc5(ctx, out_dev, out_dtype, w, expert, x_dev, x_dtype, ntok, s);
        return jl_set_err(ctx, JL_DECLINED, "the decode kernels take f32 activations and outputs");
    }
    return jl_launch_gemv(ctx, (float *)out_dev, w, expert, (const float *)x_dev, ntok, ch.kernel, s);
}

JL_EXPORT int jl_matvec_dev(jl_ctx *ctx, float *out_dev, const jl_weight *w, const float *x_dev, int ntok,
                            void *stream) {
    if (!ctx || !out_dev || !w || !x_dev || ntok < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    int rc = serving_prologue(ctx);
    if (rc) return rc;
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = matmul_dev_locked(ctx, out_dev, JL_DT_F32, w, 0, x_dev, JL_DT_F32, ntok,
                           (cudaStream_t)stream);
    if (rc == JL_OK) ctx->st.served++;
    return rc;
}

// Where a producer kernel writes the decode kernel's prepared activation operand for weight `w`, or NULL
// when this weight / token count is not served by the Q4_K tensor-core decode kernel's split form.
JL_EXPORT void *jl_decode_operand(jl_ctx *ctx, const jl_weight *w, int ntok) {
    if (!ctx || !w || ntok < 1 || ntok > 8) return nullptr;
    std::lock_guard<std::mutex> lk(ctx->mu);
    jl_choice ch;
    if (w->type != JL_TYPE_Q4_K || !w->has_map_sb16 || (ctx->opts.flags & JL_FLAG_NO_TMA)) return nullptr;
    if (choose(ctx, w->type, w->nrows, w->k, ntok, &ch) != JL_OK || ch.kernel != JL_K_MMA) return nullptr;
    if (ctx->scratch_cap < jl_gemv_scratch_bytes(w->type, w->k, ntok)) return nullptr;
    return ctx->scratch;
}

JL_EXPORT int jl_matvec_dev_prepared(jl_ctx *ctx, float *out_dev, const jl_weight *w, int ntok, void *stream) {
    if (!ctx || !out_dev || !w || ntok < 1 || ntok > 8) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    int rc = serving_prologue(ctx);
    if (rc) return rc;
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    jl_choice ch;
    if (w->type != JL_TYPE_Q4_K || !w->has_map_sb16 || (ctx->opts.flags & JL_FLAG_NO_TMA) ||
        choose(ctx, w->type, w->nrows, w->k, ntok, &ch) != JL_OK || ch.kernel != JL_K_MMA)
        return jl_set_err(ctx, JL_DECLINED, "no prepared-operand form for this weight (jl_decode_operand returned NULL)");
    rc = jl_launch_gemv(ctx, out_dev, w, 0, nullptr, ntok, JL_K_MMA, (cudaStream_t)stream);
    if (rc == JL_OK) ctx->st.served++;
    return rc;
}

JL_EXPORT int jl_matmul_dev(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, const void *x_dev,
                            int x_dtype, int ntok, void *stream) {
    if (!ctx || !out_dev || !w || !x_dev || ntok < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    int rc = serving_prologue(ctx);
    if (rc) return rc;
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = matmul_dev_locked(ctx, out_dev, out_dtype, w, 0, x_dev, x_dtype, ntok,
                           (cudaStream_t)stream);
    if (rc == JL_OK) ctx->st.served++;
    return rc;
}

// The batched counterpart of jl_decode_operand: where a producer kernel (jl_aux_add_rmsnorm_gemm) writes the tcgen05
// GEMM's activation operand for `ntok` rows of weight `w`, so that no conversion launch sits between the two.
// JL_DECLINED when this (weight, token count) does not go to the GEMM or the scratch is too small (jl_reserve).
JL_EXPORT int jl_gemm_operand(jl_ctx *ctx, const jl_weight *w, int ntok, void **rows_f16, float **inv_scale) {
    if (!ctx || !w || !rows_f16 || !inv_scale || ntok < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    jl_choice ch;
    if (choose(ctx, w->type, w->nrows, w->k, ntok, &ch) != JL_OK || ch.kernel != JL_K_TC5) return JL_DECLINED;
    return jl_gemm_tc5_operand(ctx, w, ntok, rows_f16, inv_scale);
}

JL_EXPORT int jl_matmul_dev_prepared(jl_ctx *ctx, void *out_dev, int out_dtype, const jl_weight *w, int ntok, void *stream) {
    if (!ctx || !out_dev || !w || ntok < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    int rc = serving_prologue(ctx);
    if (rc) return rc;
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    jl_choice ch;
    if (choose(ctx, w->type, w->nrows, w->k, ntok, &ch) != JL_OK || ch.kernel != JL_K_TC5)
        return jl_set_err(ctx, JL_DECLINED, "no prepared-operand GEMM for this weight and token count (jl_gemm_operand declined)");
    rc = jl_launch_gemm_tc5(ctx, out_dev, out_dtype, w, 0, nullptr, JL_DT_F32, ntok, (cudaStream_t)stream);
    if (rc == JL_OK) ctx->st.served++;
    return rc;
}

// ------------------------------------------------------- host entry points

static size_t dtype_bytes(int dt) { return dt == JL_DT_F32 ? 4 : 2; }

// Last kernel of a zero-copy decode call: the status word and then the call's sequence number, into pinned host memory.
__global__ void jl_done_kernel(int *status, volatile int *done) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // launched early; runs once the matvec has completed
    const int code = *status;
    if (code) *status = 0;
    const int seq = ++status[2];     // the call's number: the host counts the same launches (one thread, one stream)
    done[1] = code;
    __threadfence_system();
    done[0] = seq;
}

// Waits for the call's sequence number to arrive in pinned memory: polls the word; now and then asks the stream
// whether it failed, so that a kernel fault ends the wait with the error instead of an endless poll.
static int jl_launch_done(jl_ctx *ctx) {
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(1); cfg.stream = ctx->stream; cfg.attrs = at;
    cfg.numAttrs = (ctx->opts.flags & JL_FLAG_NO_PDL) ? 0 : 1;
    JL_CUDA(ctx, cudaLaunchKernelEx(&cfg, jl_done_kernel, ctx->dev_status, ctx->done_map));
    ctx->st.launches++;
    return JL_OK;
}
static int jl_wait_done(jl_ctx *ctx) {
    const int seq = ++ctx->done_seq;
    for (unsigned spins = 0;; spins++) {
        if (ctx->done_map[0] == seq) break;
        if ((spins & 0xFFFu) == 0xFFFu) {
            const cudaError_t q = cudaStreamQuery(ctx->stream);
            if (q != cudaSuccess && q != cudaErrorNotReady) {
                ctx->unhealthy = true;
                return jl_set_err(ctx, JL_ECUDA, "kernel failed: %s", cudaGetErrorString(q));
            }
            if (q == cudaSuccess && ctx->done_map[0] != seq) {
                // the stream is idle and the record is not ours: a launch of this call never ran. Fall back in step.
                ctx->done_seq = ctx->done_map[0];
                return jl_set_err(ctx, JL_ECUDA, "the call's completion record never arrived");
            }
        }
    }
    const int code = ctx->done_map[1];
    if (code) return jl_set_err(ctx, JL_ETIMEDOUT, "a bounded device-side wait ran out (code %d)", code);
    return JL_OK;
}

static int matmul_host(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const void *w, size_t w_bytes,
                       const void *x, int x_dtype, int nrows, int k, int ntok, const void *key = nullptr) {
    int be = jl_block_elems(type);
    if (!jl_type_served(type))
        return jl_set_err(ctx, JL_DECLINED, "type %u is not served", type);
    if (nrows < 1 || k < be || k % be || ntok < 1)
        return jl_set_err(ctx, JL_DECLINED, "shape %d x %d x %d tokens does not tile %d-element blocks", nrows, k, ntok, be);
    size_t need = (size_t)nrows * jl_row_bytes(type, k);
    if (w && w_bytes < need) return jl_set_err(ctx, JL_EINVAL, "weight has %zu bytes, shape needs %zu", w_bytes, need);
    if (ctx->opts.min_weight_bytes && need < ctx->opts.min_weight_bytes)
        return jl_set_err(ctx, JL_DECLINED, "%zu weight bytes is below the %llu-byte break-even", need,
                          (unsigned long long)ctx->opts.min_weight_bytes);
    int rc = serving_prologue(ctx);
    if (rc) return rc;
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    jl_weight *dw = nullptr;
    rc = resident(ctx, type, w, w_bytes, 1, nrows, k, &dw, key);
    jl_resident_unpin(ctx);   // ctx->mu is held to the end of this call: nothing else can evict dw meanwhile
    if (rc) return rc;
    size_t xb = (size_t)ntok * k * dtype_bytes(x_dtype), ob = (size_t)ntok * nrows * dtype_bytes(out_dtype);
    if ((rc = reserve_locked(ctx, xb, ob))) return rc;
    {
        size_t need = jl_gemv_scratch_bytes(type, k, ntok);
        const size_t need_gemm = jl_gemm_tc5_scratch_bytes(nrows, k, ntok, x_dtype, ctx->sm_count);
        if (need_gemm > need) need = need_gemm;
        if ((rc = jl_grow_scratch(ctx, need))) return rc;
    }
    {
        // Decode calls (a few tokens, f32 in and out): no copy engine and no stream synchronisation on the path. The
        // kernels read x from and write y to pinned host memory directly (16 KB each way at 4096 x 4096), a last
        // one-warp kernel posts the status word and a sequence number there, and the host polls that word. The
        // activation row is converted by the prep launch (read across the bus ONCE), so the forms in which every
        // CTA converts the row itself are not used here.
        jl_choice ch;
        if (x_dtype == JL_DT_F32 && out_dtype == JL_DT_F32 && xb <= ctx->x_map_cap && ob <= ctx->o_map_cap && ctx->done_map &&
            choose(ctx, type, nrows, k, ntok, &ch) == JL_OK && ch.kernel == JL_K_MMA) {
            const int saved_form = ctx->opts.decode_form;
            if (ch.kernel == JL_K_MMA && type == JL_TYPE_Q4_K && (ch.form == JL_FORM_WIDE || ch.form == JL_FORM_FUSED))
                ctx->opts.decode_form = JL_FORM_SPLIT;
            memcpy(ctx->x_map, x, xb);
            // The call's launches (activation prep, matvec, done) are the same every time for a resident weight:
            // they are captured once into a graph kept with the weight and replayed with ONE launch call. The graph
            // is rebuilt when anything it baked in moves (scratch, staging buffers, token count, options).
            jl_weight *mw = const_cast<jl_weight *>(dw);
            const bool fresh = mw->zc_exec && mw->zc_ntok == ntok && mw->zc_scratch == ctx->scratch && mw->zc_x == ctx->x_map &&
                               mw->zc_o == ctx->o_map && mw->zc_flags == ctx->opts.flags && mw->zc_form == ctx->opts.decode_form;
            if (!fresh) {
                if (mw->zc_exec) { cudaGraphExecDestroy((cudaGraphExec_t)mw->zc_exec); mw->zc_exec = nullptr; }
                const int64_t launches0 = ctx->st.launches;
                cudaGraph_t graph = nullptr;
                cudaGraphExec_t exec = nullptr;
                if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                    rc = matmul_dev_locked(ctx, ctx->o_map, out_dtype, dw, 0, ctx->x_map, x_dtype, ntok, ctx->stream);
                    if (rc == JL_OK) rc = jl_launch_done(ctx);
                    const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
                    if (rc == JL_OK && ce == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
                        mw->zc_exec = exec; mw->zc_ntok = ntok; mw->zc_scratch = ctx->scratch; mw->zc_x = ctx->x_map;
                        mw->zc_o = ctx->o_map; mw->zc_flags = ctx->opts.flags; mw->zc_form = ctx->opts.decode_form;
                        mw->zc_launches = (int)(ctx->st.launches - launches0);
                    }
                    if (graph) cudaGraphDestroy(graph);
                    cudaGetLastError();
                }
                ctx->st.launches = launches0;             // nothing has run yet
                if (rc != JL_OK && rc != JL_DECLINED) { ctx->opts.decode_form = saved_form; return rc; }
            }
            if (mw->zc_exec) {
                ctx->opts.decode_form = saved_form;
                JL_CUDA(ctx, cudaGraphLaunch((cudaGraphExec_t)mw->zc_exec, ctx->stream));
                ctx->st.launches += mw->zc_launches;
            } else {                                      // capture refused: the plain launches
                rc = matmul_dev_locked(ctx, ctx->o_map, out_dtype, dw, 0, ctx->x_map, x_dtype, ntok, ctx->stream);
                ctx->opts.decode_form = saved_form;
                if (rc) return rc;
                if ((rc = jl_launch_done(ctx))) return rc;
            }
            if ((rc = jl_wait_done(ctx))) return rc;
            memcpy(out, ctx->o_map, ob);
            ctx->st.served++;
            return JL_OK;
        }
    }
    memcpy(ctx->x_pin, x, xb);
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->x_dev, ctx->x_pin, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = matmul_dev_locked(ctx, ctx->o_dev, out_dtype, dw, 0, ctx->x_dev, x_dtype, ntok, ctx->stream);
    if (rc) return rc;
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->o_pin, ctx->o_dev, ob, cudaMemcpyDeviceToHost, ctx->stream));
    if ((rc = jl_read_status(ctx, ctx->stream))) return rc;   // the status word rides along; synchronises
    memcpy(out, ctx->o_pin, ob);
    ctx->st.served++;
    return JL_OK;
}

// packed.cu: is there a resident copy of this shape under `key`?
bool jl_resident_known(jl_ctx *ctx, const void *key, uint32_t type, int nrows, int k) {
    std::lock_guard<std::mutex> lk(ctx->cache_mu);
    auto it = ctx->cache.find((uintptr_t)key);
    return it != ctx->cache.end() && it->second->type == type && it->second->nrows == nrows && it->second->k == k &&
           it->second->n_expert == 1;
}
// packed.cu: the host-pointer matmul with residency keyed on `key`; raw (may be NULL when the copy is resident) are the
// re-interleaved blocks to upload.
int jl_matmul_keyed(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const void *key, const void *raw, size_t raw_bytes,
                    const void *x, int x_dtype, int nrows, int k, int ntok) {
    std::lock_guard<std::mutex> lk(ctx->mu);
    return matmul_host(ctx, out, out_dtype, type, raw, raw_bytes, x, x_dtype, nrows, k, ntok, key);
}

JL_EXPORT int jl_matvec(jl_ctx *ctx, float *out, uint32_t type, const void *w, size_t w_bytes, const float *x,
                        int nrows, int k) {
    if (!ctx || !out || !w || !x) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return matmul_host(ctx, out, JL_DT_F32, type, w, w_bytes, x, JL_DT_F32, nrows, k, 1);
}

JL_EXPORT int jl_matmul(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const void *w, size_t w_bytes,
                        const void *x, int x_dtype, int nrows, int k, int ntok) {
    if (!ctx || !out || !w || !x) return JL_EINVAL;
    if (out_dtype < 0 || out_dtype > 2 || x_dtype < 0 || x_dtype > 2) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    return matmul_host(ctx, out, out_dtype, type, w, w_bytes, x, x_dtype, nrows, k, ntok);
}

// ------------------------------------------------------------ device status

// Copies the status word home on `s`, waits for `s`, clears the word when it was set.
int jl_read_status(jl_ctx *ctx, cudaStream_t s) {
    *ctx->stat_pin = 0;
    cudaError_t e = cudaMemcpyAsync(ctx->stat_pin, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        ctx->unhealthy = true;
        return jl_set_err(ctx, JL_ECUDA, "kernel or copy failed: %s", cudaGetErrorString(e));
    }
    const int code = *ctx->stat_pin;
    if (!code) return JL_OK;
    e = cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return jl_set_err(ctx, JL_ECUDA, "clearing the status word: %s", cudaGetErrorString(e));
    static const char *const what[] = {"", "a weight tile of the decode kernel never landed", "a ring slot of the prefill GEMM",
                                       "a ring slot of the grouped expert GEMM", "a phase's input or the grid barrier inside the block kernel",
                                       "a peer's partial sums (tensor-parallel exchange)", "the test wait"};
    return jl_set_err(ctx, JL_ETIMEDOUT, "a bounded device-side wait ran out (code %d: %s)", code,
                      code > 0 && code < 7 ? what[code] : "unknown");
}

JL_EXPORT int jl_status_poll(jl_ctx *ctx, void *stream) {
    if (!ctx) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    return jl_read_status(ctx, (cudaStream_t)stream);
}

// One thread waits on an mbarrier that expects bytes nobody sends; the wait is bounded like every
// other wait in the library, runs out after `limit_ns`, and the kernel reports it and returns.
__global__ void jl_test_wait_kernel(int *status, uint64_t limit_ns) {
    __shared__ uint64_t bar;
    mbar_init(smem_u32(&bar), 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(smem_u32(&bar), 16);          // 16 bytes that never arrive
    if (!mbar_wait_ns(smem_u32(&bar), 0, limit_ns)) atomicExch(status, 6);
}

JL_EXPORT int jl_test_wait_timeout(jl_ctx *ctx, uint32_t limit_us, void *stream) {
    if (!ctx || limit_us < 1 || limit_us > 1000000u) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    jl_test_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(ctx->dev_status, (uint64_t)limit_us * 1000ull);
    ctx->st.launches++;
    JL_CUDA(ctx, cudaGetLastError());
    return JL_OK;
}

// The public host-pointer call in a loop of the library's own (see the header).
JL_EXPORT int jl_test_matvec_loop(jl_ctx *ctx, float *out, uint32_t type, const void *const *ws, size_t w_bytes, const float *x,
                                  int nrows, int k, int nw, int iters, double *seconds) {
    if (!ctx || !out || !ws || !x || nw < 1 || iters < 1 || !seconds) return JL_EINVAL;
    const auto t0 = std::chrono::steady_clock::now();
    for (int it = 0; it < iters; it++)
        for (int i = 0; i < nw; i++) {
            const int rc = jl_matvec(ctx, out, type, ws[i], w_bytes, x, nrows, k);
            if (rc != JL_OK) return rc;
        }
    *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return JL_OK;
}
