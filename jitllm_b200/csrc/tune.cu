// Measured selection: which variant of the decode kernel serves a shape is timed on the device that will run it,
// against the resident weight, once per (type, rows, k, tokens); the table's pick stands unless a challenger wins
// clearly. The reference does the same for its split width (jit/gpu/tier/split.go:18-75): a paired duel at load, a
// dispersed sample (IQR / median above 0.10) is refused rather than rounded, a later candidate has to beat the best
// so far by more than 1 %, and the verdict is persisted keyed by device UUID + driver + executable so the next
// process skips the measurement (jit/gpu/tier/choose.go:196-216).
//
// The protocol (jl_tune_duel) and the verdict file (jl_tune_cache_*) are host code with an injectable timer, so
// they are tested without a GPU; the device part only supplies the timer: CUDA events around one launch of the
// candidate, L2 flushed in front of it.
#include "jl_internal.cuh"

#include <errno.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>

#include <algorithm>
#include <string>
#include <vector>

#ifndef JL_BUILD_ID
#define JL_BUILD_ID "unversioned"
#endif

#define JL_TUNE_ROUNDS 9
#define JL_TUNE_WARMUP 2
#define JL_TUNE_IQR_GATE 0.10
#define JL_TUNE_MARGIN 0.01

// ---------------------------------------------------------------------------------------------- the protocol

// timer(user, cand, round) returns the RATE (work per second, higher is better) of one timed run of candidate
// `cand`, or a value <= 0 when the run failed. Candidates are tried in order; candidate 0 is the table's pick.
// refused[c] (may be NULL) is set to 1 for a candidate whose sample was dispersed or failed. Returns the winner, or
// -1 when no candidate gave a usable sample (the table's answer stands and nothing is persisted).
JL_EXPORT int jl_tune_duel(int ncand, int nrounds, double (*timer)(void *user, int cand, int round), void *user,
                           double iqr_gate, double margin, int *refused, double *medians) {
    if (ncand < 1 || nrounds < 1 || !timer) return -1;
    int best = -1;
    double best_rate = 0.0;
    std::vector<double> rs(nrounds);
    for (int c = 0; c < ncand; c++) {
        bool ok = true;
        for (int r = 0; r < nrounds && ok; r++) {
            rs[r] = timer(user, c, r);
            if (!(rs[r] > 0.0)) ok = false;
        }
        double med = 0.0;
        if (ok) {
            std::sort(rs.begin(), rs.end());
            med = rs[nrounds / 2];
            const double iqr = rs[(3 * nrounds) / 4] - rs[nrounds / 4];
            if (!(med > 0.0) || iqr / med > iqr_gate) ok = false;      // dispersed: refused, not rounded
        }
        if (refused) refused[c] = ok ? 0 : 1;
        if (medians) medians[c] = ok ? med : 0.0;
        // a later candidate must beat the best so far by the margin: inside it the trial cannot tell them apart
        if (ok && med > best_rate * (1.0 + margin)) { best = c; best_rate = med; }
    }
    return best;
}

// ------------------------------------------------------------------------------------------- the verdict file

// One file per directory, "jl_select1": lines "<key> <value>\n". A file that cannot be read or a line that does not
// parse is no entry: the caller measures again and rewrites it.
static std::string cache_file(const char *dir) { return std::string(dir) + "/jl_select1"; }

JL_EXPORT int jl_tune_cache_lookup(const char *dir, const char *key, char *value, size_t cap) {
    if (!dir || !*dir || !key || !*key || !value || cap < 2) return 0;
    FILE *f = fopen(cache_file(dir).c_str(), "r");
    if (!f) return 0;
    char line[512];
    int found = 0;
    const size_t kl = strlen(key);
    while (fgets(line, sizeof line, f)) {
        size_t n = strlen(line);
        if (n == 0 || line[n - 1] != '\n') continue;              // a torn last line is no entry
        line[--n] = 0;
        if (n > kl + 1 && !strncmp(line, key, kl) && line[kl] == ' ') {
            snprintf(value, cap, "%s", line + kl + 1);            // the LAST entry for a key wins
            found = 1;
        }
    }
    fclose(f);
    return found;
}

// Rewrites the file with the key's entry replaced (or appended), through a temporary file and a rename so that a
// reader never sees half a file. Returns 1 when saved.
JL_EXPORT int jl_tune_cache_save(const char *dir, const char *key, const char *value) {
    if (!dir || !*dir || !key || !*key || !value || strchr(key, ' ') || strchr(key, '\n') || strchr(value, '\n')) return 0;
    if (mkdir(dir, 0777) != 0 && errno != EEXIST) return 0;
    const std::string path = cache_file(dir), tmp = path + ".tmp";
    std::vector<std::string> keep;
    if (FILE *f = fopen(path.c_str(), "r")) {
        char line[512];
        const size_t kl = strlen(key);
        while (fgets(line, sizeof line, f)) {
            size_t n = strlen(line);
            if (n == 0 || line[n - 1] != '\n') continue;
            if (n > kl + 1 && !strncmp(line, key, kl) && line[kl] == ' ') continue;
            keep.push_back(line);
        }
        fclose(f);
    }
    FILE *o = fopen(tmp.c_str(), "w");
    if (!o) return 0;
    for (const std::string &l : keep) fputs(l.c_str(), o);
    fprintf(o, "%s %s\n", key, value);
    if (fclose(o) != 0) return 0;
    return rename(tmp.c_str(), path.c_str()) == 0 ? 1 : 0;
}

// Identity of what a verdict was measured on: GPU UUID, driver version and this build of the library. FNV-1a.
static uint64_t fnv1a(const void *p, size_t n, uint64_t h = 1469598103934665603ull) {
    const uint8_t *b = (const uint8_t *)p;
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
}
JL_EXPORT void jl_tune_device_key(const void *uuid16, int driver_version, const char *build_id, char out[17]) {
    uint64_t h = fnv1a("cuda/", 5);
    h = fnv1a(uuid16, 16, h);
    h = fnv1a(&driver_version, sizeof driver_version, h);
    if (build_id) h = fnv1a(build_id, strlen(build_id), h);
    snprintf(out, 17, "%016llx", (unsigned long long)h);
}
JL_EXPORT const char *jl_build_id(void) { return JL_BUILD_ID; }

// ------------------------------------------------------------------------------------------------ on the device

JL_EXPORT int jl_tune_configure(jl_ctx *ctx, int mode, const char *cache_dir) {
    if (!ctx || mode < JL_TUNE_OFF || mode > JL_TUNE_FORCE) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->tune_mode = mode;
    ctx->tune_dir = cache_dir ? cache_dir : "";
    if (!ctx->tune_devkey[0]) {
        cudaDeviceProp prop;
        int drv = 0;
        if (cudaGetDeviceProperties(&prop, ctx->device) == cudaSuccess && cudaDriverGetVersion(&drv) == cudaSuccess)
            jl_tune_device_key(prop.uuid.bytes, drv, JL_BUILD_ID, ctx->tune_devkey);
    }
    return JL_OK;
}

JL_EXPORT int jl_tune_stats(jl_ctx *ctx, int64_t out[4]) {
    if (!ctx || !out) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    out[0] = ctx->tune_trials; out[1] = ctx->tune_measured; out[2] = ctx->tune_cached; out[3] = ctx->tune_refused;
    return JL_OK;
}

struct tune_run {
    jl_ctx *ctx;
    const jl_weight *w;
    int ntok;
    const int *cands;
    float *x, *y;
    void *flush;
    size_t flush_bytes;
    cudaEvent_t e0, e1;
};

static double tune_timer(void *user, int cand, int round) {
    tune_run *t = (tune_run *)user;
    jl_ctx *ctx = t->ctx;
    ctx->force_variant = t->cands[cand];
    double rate = 0.0;
    const int reps = round == 0 ? 1 + JL_TUNE_WARMUP : 1;        // the first round of a candidate warms it up
    for (int i = 0; i < reps; i++) {
        if (t->flush && cudaMemsetAsync(t->flush, i, t->flush_bytes, ctx->stream) != cudaSuccess) break;
        if (cudaEventRecord(t->e0, ctx->stream) != cudaSuccess) break;
        if (jl_launch_gemv(ctx, t->y, t->w, 0, t->x, t->ntok, JL_K_MMA, ctx->stream) != JL_OK) break;
        if (cudaEventRecord(t->e1, ctx->stream) != cudaSuccess) break;
        if (cudaEventSynchronize(t->e1) != cudaSuccess) break;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, t->e0, t->e1) != cudaSuccess || !(ms > 0.f)) break;
        if (i == reps - 1) rate = 1e3 / ms;
    }
    ctx->force_variant = -1;
    ctx->tune_trials += reps;
    return rate;
}

// Measures (or loads) the verdict of w's shape at ntok tokens. Called with ctx->mu held.
int jl_tune_shape_locked(jl_ctx *ctx, const jl_weight *w, int ntok) {
    if (ctx->tune_mode == JL_TUNE_OFF || w->type != JL_TYPE_Q4_K || !w->has_map_sb16 || w->n_expert != 1) return JL_OK;
    if (ctx->opts.pin_kernel != JL_K_AUTO || ctx->opts.decode_form != JL_FORM_AUTO || ctx->opts.pin_warps ||
        (ctx->opts.flags & (JL_FLAG_DECODE_CONCURRENT | JL_FLAG_NO_TMA)))
        return JL_OK;                                             // the caller chose already
    const uint64_t key = jl_tune_shape_key(w->type, w->nrows, w->k, ntok);
    if (ctx->tuned.count(key)) return JL_OK;
    int cands[32];
    const int nc = jl_gemv_tune_candidates(ctx, w->nrows, w->k, ntok, cands, 32);
    if (nc < 2) return JL_OK;
    ctx->tuned[key] = cands[0];                                   // so a failure below is not retried per layer
    char ck[96] = "";
    if (ctx->tune_devkey[0]) snprintf(ck, sizeof ck, "%s/%u-%dx%dx%d", ctx->tune_devkey, w->type, w->nrows, w->k, ntok);
    char val[64];
    if (ck[0] && ctx->tune_mode != JL_TUNE_FORCE && jl_tune_cache_lookup(ctx->tune_dir.c_str(), ck, val, sizeof val)) {
        // an entry that does not parse, or names a variant this shape cannot take, is measured again and overwritten
        int f, wp, st, mb, rg;
        if (sscanf(val, "%d %d %d %d %d", &f, &wp, &st, &mb, &rg) == 5) {
            const int idx = jl_gemv_variant_index(f, wp, st, mb, rg, w->k / 256);
            if (idx >= 0 && std::find(cands, cands + nc, idx) != cands + nc) {
                ctx->tuned[key] = idx;
                ctx->tune_cached++;
                return JL_OK;
            }
        }
    }
    if (cudaSetDevice(ctx->device) != cudaSuccess) return JL_OK;
    if (jl_grow_scratch(ctx, jl_gemv_scratch_bytes(w->type, w->k, ntok)) != JL_OK) return JL_OK;
    tune_run t = {};
    t.ctx = ctx; t.w = w; t.ntok = ntok; t.cands = cands;
    t.flush_bytes = (size_t)160 << 20;                            // larger than L2: every timed launch reads HBM
    bool ok = cudaMalloc(&t.x, (size_t)ntok * w->k * 4) == cudaSuccess;
    ok = ok && cudaMalloc(&t.y, (size_t)ntok * w->nrows * 4) == cudaSuccess;
    ok = ok && cudaMemsetAsync(t.x, 0, (size_t)ntok * w->k * 4, ctx->stream) == cudaSuccess;
    if (ok && cudaMalloc(&t.flush, t.flush_bytes) != cudaSuccess) { t.flush = nullptr; cudaGetLastError(); }
    ok = ok && cudaEventCreate(&t.e0) == cudaSuccess && cudaEventCreate(&t.e1) == cudaSuccess;
    int winner = -1, refused[32] = {0};
    const int64_t launches0 = ctx->st.launches;
    if (ok) winner = jl_tune_duel(nc, JL_TUNE_ROUNDS, tune_timer, &t, JL_TUNE_IQR_GATE, JL_TUNE_MARGIN, refused, nullptr);
    ctx->st.launches = launches0;                                 // trials are not served work
    cudaStreamSynchronize(ctx->stream);
    if (t.e0) cudaEventDestroy(t.e0);
    if (t.e1) cudaEventDestroy(t.e1);
    cudaFree(t.flush); cudaFree(t.y); cudaFree(t.x);
    cudaGetLastError();
    for (int c = 0; c < nc; c++) ctx->tune_refused += refused[c];
    if (winner < 0) return JL_OK;                                 // nothing usable: the table's answer stands
    ctx->tuned[key] = cands[winner];
    ctx->tune_measured++;
    if (ck[0] && !ctx->tune_dir.empty()) {
        int f, wp, st, mb, rg;
        jl_gemv_variant_describe(cands[winner], &f, &wp, &st, &mb, &rg);
        snprintf(val, sizeof val, "%d %d %d %d %d", f, wp, st, mb, rg);
        jl_tune_cache_save(ctx->tune_dir.c_str(), ck, val);
    }
    return JL_OK;
}

JL_EXPORT int jl_tune(jl_ctx *ctx, const jl_weight *w, int ntok, jl_choice *out) {
    if (!ctx || !w || ntok < 1) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->unhealthy) return jl_set_err(ctx, JL_ECUDA, "context is unhealthy after an earlier CUDA error");
    const int saved = ctx->tune_mode;
    if (saved == JL_TUNE_OFF) ctx->tune_mode = JL_TUNE_ON;        // an explicit call measures even when uploads do not
    int rc = jl_tune_shape_locked(ctx, w, ntok);
    ctx->tune_mode = saved;
    if (rc == JL_OK && out) rc = jl_gemv_choice(ctx, w->type, w->nrows, w->k, ntok, out);
    return rc;
}
