// Block formats: the integer view (jl_unpack), the device-resident layouts and
// the repack kernels that produce them.
//
// Layout knowledge restated from format/quant/dequant.go:148-174,360-397 and
// jit/gpu/kernels/pack.go:252-386 (extract).
#include "jl_internal.cuh"
#include "tma.cuh"

#include <stdlib.h>
#include <string.h>

// ---------------------------------------------------------------- host unpack

static inline uint16_t le16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// The j-th 6-bit (scale, min) pair of a Q4_K block's 12 packed bytes.
__host__ __device__ static inline void q4k_scale_min(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

#include "raw_formats.cuh"

JL_EXPORT int jl_unpack(uint32_t type, const void *blocks, size_t n_blocks, int8_t *q, uint16_t *d_bits,
                        uint16_t *dmin_bits, uint8_t *sc, uint8_t *m) {
    if (!blocks || !q || !d_bits || !dmin_bits || !sc || !m) return JL_EINVAL;
    const uint8_t *src = (const uint8_t *)blocks;
    size_t r = 0;
    switch (type) {
    case JL_TYPE_Q8_0:
        for (size_t b = 0; b < n_blocks; b++, r++) {
            const uint8_t *blk = src + b * 34;
            memcpy(q + r * 32, blk + 2, 32);
            d_bits[r] = le16(blk); dmin_bits[r] = 0; sc[r] = 0; m[r] = 0;
        }
        return JL_OK;
    case JL_TYPE_MXFP4:
        for (size_t b = 0; b < n_blocks; b++, r++) {
            const uint8_t *blk = src + b * 17;
            for (int l = 0; l < 16; l++) {
                q[r * 32 + l] = (int8_t)(blk[1 + l] & 0xF);
                q[r * 32 + 16 + l] = (int8_t)(blk[1 + l] >> 4);
            }
            d_bits[r] = (uint16_t)(uint8_t)(blk[0] - 1); dmin_bits[r] = 0; sc[r] = 0; m[r] = 0;
        }
        return JL_OK;
    case JL_TYPE_Q4_K:
        for (size_t b = 0; b < n_blocks; b++) {
            const uint8_t *blk = src + b * 144;
            for (int s = 0; s < 8; s++, r++) {
                q4k_scale_min(s, blk + 4, &sc[r], &m[r]);
                const uint8_t *grp = blk + 16 + (s / 2) * 32;
                for (int l = 0; l < 32; l++)
                    q[r * 32 + l] = (int8_t)((s & 1) ? (grp[l] >> 4) : (grp[l] & 0xF));
                d_bits[r] = le16(blk); dmin_bits[r] = le16(blk + 2);
            }
        }
        return JL_OK;
    case JL_TYPE_Q4_0: case JL_TYPE_Q5_0: case JL_TYPE_Q5_1: case JL_TYPE_Q5_K: case JL_TYPE_Q6_K: {
        // element by element through the same accessors the kernels use (raw_formats.cuh)
        const int be = jl_block_elems(type), bb = jl_block_bytes(type), sub = type == JL_TYPE_Q6_K ? 16 : 32;
        for (size_t b = 0; b < n_blocks; b++) {
            const uint8_t *blk = src + b * bb;
            for (int s = 0; s < be / sub; s++, r++) {
                for (int l = 0; l < sub; l++) q[r * sub + l] = (int8_t)jl_raw_code(type, blk, s * sub + l);
                jl_raw_record(type, blk, s, &d_bits[r], &dmin_bits[r], &sc[r], &m[r]);
            }
        }
        return JL_OK;
    }
    }
    return JL_ENOTSUP;
}

// ------------------------------------------------------------ repack kernels

// Where code `kk` (0..63) of a 64-element span sits in the resident Q8_0 order.
__host__ __device__ static inline int q8_span_pos(int kk) {
    int blk = kk >> 5, within = kk & 31;
    int half = within >> 4, r16 = within & 15;
    int t = r16 >> 2, byte = r16 & 3;
    int wi = blk * 2 + half;
    return t * 16 + wi * 4 + byte;
}

// raw [rows][k/32] x 34 B  ->  codes [rows][k] (span order), d [rows][k/32].
__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ codes,
                                   uint16_t *__restrict__ d, size_t total_rows, int k) {
    size_t nb_row = (size_t)k / 32;
    size_t nblk = total_rows * nb_row;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblk;
         b += (size_t)gridDim.x * blockDim.x) {
        size_t row = b / nb_row;
        int bi = (int)(b % nb_row);
        const uint8_t *blk = raw + b * 34;
        d[b] = (uint16_t)(blk[0] | (blk[1] << 8));
        uint8_t *dst = codes + row * (size_t)k + (size_t)(bi >> 1) * 64;
        for (int l = 0; l < 32; l++) dst[q8_span_pos((bi & 1) * 32 + l)] = blk[2 + l];
    }
}

// raw [rows][k/32] x 17 B  ->  codes [rows][k/32][16], e [rows][stride].
__global__ void repack_mxfp4_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ codes,
                                    uint8_t *__restrict__ e, size_t total_rows, int k, int stride) {
    size_t nb_row = (size_t)k / 32;
    size_t nblk = total_rows * nb_row;
    for (size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x; b < nblk;
         b += (size_t)gridDim.x * blockDim.x) {
        size_t row = b / nb_row;
        int bi = (int)(b % nb_row);
        const uint8_t *blk = raw + b * 17;
        e[row * (size_t)stride + bi] = blk[0];
        uint8_t *dst = codes + b * 16;
        for (int l = 0; l < 16; l++) dst[l] = blk[1 + l];
    }
}

void jl_weight_release(jl_weight *w) {
    if (!w) return;
    if (w->zc_exec) cudaGraphExecDestroy((cudaGraphExec_t)w->zc_exec);
    if (w->data) cudaFree(w->data);
    if (w->scales) cudaFree(w->scales);
    delete w;
}

int jl_repack_upload(jl_ctx *ctx, uint32_t type, const void *w_host, size_t w_bytes, int n_expert,
                     int nrows, int k, jl_weight **out) {
    int be = jl_block_elems(type);
    if (!jl_type_served(type))
        return jl_set_err(ctx, JL_DECLINED, "type %u has no resident layout", type);
    if (nrows < 1 || k < be || k % be || n_expert < 1)
        return jl_set_err(ctx, JL_DECLINED, "shape %d x %d does not tile %d-element blocks", nrows, k, be);
    if (type == JL_TYPE_Q8_0 && k % 64)
        return jl_set_err(ctx, JL_DECLINED, "Q8_0 needs k %% 64 == 0, k = %d", k);
    size_t rows = (size_t)n_expert * (size_t)nrows;
    size_t need = rows * jl_row_bytes(type, k);
    if (w_bytes < need)
        return jl_set_err(ctx, JL_EINVAL, "weight has %zu bytes, %zu rows x %d need %zu", w_bytes, rows, k, need);

    jl_weight *w = new jl_weight();
    memset(w, 0, sizeof(*w));
    w->type = type; w->n_expert = n_expert; w->nrows = nrows; w->k = k; w->raw_bytes = need;
    w->emin = 255; w->emax = 0;
    if (type == JL_TYPE_MXFP4) {   // the scale range decides whether f16 can hold the weights exactly
        const uint8_t *b = (const uint8_t *)w_host;
        for (size_t i = 0; i < need; i += 17) {
            bool zero = true;
            for (int j = 1; j < 17 && zero; j++) zero = (b[i + j] & 0x77) == 0;
            if (zero) continue;
            if (b[i] < w->emin) w->emin = b[i];
            if (b[i] > w->emax) w->emax = b[i];
        }
        if (w->emin > w->emax) { w->emin = 127; w->emax = 127; }
    }
    cudaError_t e;
    if (type == JL_TYPE_Q4_K || jl_type_raw_simt(type)) {
        // +16 so a kernel may over-read one aligned chunk past the end.
        w->data_bytes = need;
        if ((e = cudaMalloc(&w->data, need + 16)) != cudaSuccess) goto oom;
        if ((e = cudaMemcpyAsync(w->data, w_host, need, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) goto fail;
        if (type == JL_TYPE_Q4_K) w->has_map_sb16 = jl_make_tmap_2d(&w->map_sb16, w->data, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1,
                                          jl_row_bytes(type, k), rows, jl_row_bytes(type, k), 144, 16,
                                          CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        uint8_t *raw = nullptr;
        if ((e = cudaMalloc(&raw, need)) != cudaSuccess) goto oom;
        if ((e = cudaMemcpyAsync(raw, w_host, need, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) {
            cudaFree(raw); goto fail;
        }
        size_t nblk = rows * (size_t)(k / 32);
        int grid = (int)((nblk + 255) / 256 < 148 * 8 ? (nblk + 255) / 256 : 148 * 8);
        if (type == JL_TYPE_Q8_0) {
            w->data_bytes = rows * (size_t)k;
            w->scale_stride = k / 32;
            w->scales_bytes = rows * (size_t)w->scale_stride * 2;
            if ((e = cudaMalloc(&w->data, w->data_bytes + 16)) != cudaSuccess) { cudaFree(raw); goto oom; }
            if ((e = cudaMalloc(&w->scales, w->scales_bytes + 16)) != cudaSuccess) { cudaFree(raw); goto oom; }
            repack_q8_0_kernel<<<grid, 256, 0, ctx->stream>>>(raw, w->data, (uint16_t *)w->scales, rows, k);
        } else {
            w->data_bytes = nblk * 16;
            w->scale_stride = ((k / 32) + 15) / 16 * 16;
            w->scales_bytes = rows * (size_t)w->scale_stride;
            // slack behind the code plane: the block-scaled mixture arm's last TMA box of the last row reads up to 64
            // bytes past the end (zero codes)
            if ((e = cudaMalloc(&w->data, w->data_bytes + 128)) != cudaSuccess) { cudaFree(raw); goto oom; }
            if ((e = cudaMemsetAsync(w->data + w->data_bytes, 0, 128, ctx->stream)) != cudaSuccess) { cudaFree(raw); goto fail; }
            if ((e = cudaMalloc(&w->scales, w->scales_bytes + 16)) != cudaSuccess) { cudaFree(raw); goto oom; }
            if ((e = cudaMemsetAsync(w->scales, 0, w->scales_bytes, ctx->stream)) != cudaSuccess) { cudaFree(raw); goto fail; }
            repack_mxfp4_kernel<<<grid, 256, 0, ctx->stream>>>(raw, w->data, w->scales, rows, k, w->scale_stride);
        }
        ctx->st.launches++;
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        cudaFree(raw);
        if (e != cudaSuccess) goto fail;
    }
    if ((e = cudaStreamSynchronize(ctx->stream)) != cudaSuccess) goto fail;
    ctx->st.uploads++;
    ctx->st.upload_bytes += need;
    *out = w;
    return JL_OK;
oom:
    jl_weight_release(w);
    cudaGetLastError();
    return jl_set_err(ctx, JL_ENOMEM, "cudaMalloc of %zu weight bytes: %s", need, cudaGetErrorString(e));
fail:
    jl_weight_release(w);
    ctx->unhealthy = true;
    return jl_set_err(ctx, JL_ECUDA, "weight upload: %s", cudaGetErrorString(e));
}

// --------------------------------------------------- unpack the resident copy

// One thread per 32-element sub-block record, reading the RESIDENT layout.
__global__ void unpack_resident_kernel(uint32_t type, const uint8_t *__restrict__ data,
                                       const uint8_t *__restrict__ scales, int scale_stride, size_t rows,
                                       int k, int8_t *q, uint16_t *d_bits, uint16_t *dmin_bits, uint8_t *sc,
                                       uint8_t *m) {
    size_t nsub_row = (size_t)k / 32;
    size_t nsub = rows * nsub_row;
    for (size_t r = blockIdx.x * (size_t)blockDim.x + threadIdx.x; r < nsub;
         r += (size_t)gridDim.x * blockDim.x) {
        size_t row = r / nsub_row;
        int si = (int)(r % nsub_row);
        if (type == JL_TYPE_Q4_K) {
            const uint8_t *blk = data + row * (nsub_row / 8) * 144 + (size_t)(si / 8) * 144;
            int s = si & 7;
            uint8_t a, b;
            q4k_scale_min(s, blk + 4, &a, &b);
            sc[r] = a; m[r] = b;
            d_bits[r] = (uint16_t)(blk[0] | (blk[1] << 8));
            dmin_bits[r] = (uint16_t)(blk[2] | (blk[3] << 8));
            const uint8_t *grp = blk + 16 + (s / 2) * 32;
            for (int l = 0; l < 32; l++) q[r * 32 + l] = (int8_t)((s & 1) ? (grp[l] >> 4) : (grp[l] & 0xF));
        } else if (jl_type_raw_simt(type)) {
            // raw blocks: sub-block si of the row (Q6_K: two 16-element records)
            const int be = jl_block_elems(type), bb = jl_block_bytes(type);
            const uint8_t *blk = data + (row * (size_t)(k / be) + (size_t)(si * 32 / be)) * bb;
            const int e0 = (si * 32) % be;
            for (int l = 0; l < 32; l++) q[r * 32 + l] = (int8_t)jl_raw_code(type, blk, e0 + l);
            if (type == JL_TYPE_Q6_K) {
                jl_raw_record(type, blk, e0 / 16, &d_bits[2 * r], &dmin_bits[2 * r], &sc[2 * r], &m[2 * r]);
                jl_raw_record(type, blk, e0 / 16 + 1, &d_bits[2 * r + 1], &dmin_bits[2 * r + 1], &sc[2 * r + 1], &m[2 * r + 1]);
            } else {
                jl_raw_record(type, blk, e0 / 32, &d_bits[r], &dmin_bits[r], &sc[r], &m[r]);
            }
        } else if (type == JL_TYPE_Q8_0) {
            const uint8_t *span = data + row * (size_t)k + (size_t)(si >> 1) * 64;
            for (int l = 0; l < 32; l++) q[r * 32 + l] = (int8_t)span[q8_span_pos((si & 1) * 32 + l)];
            d_bits[r] = ((const uint16_t *)scales)[row * (size_t)scale_stride + si];
            dmin_bits[r] = 0; sc[r] = 0; m[r] = 0;
        } else {
            const uint8_t *c = data + r * 16;
            for (int l = 0; l < 16; l++) {
                q[r * 32 + l] = (int8_t)(c[l] & 0xF);
                q[r * 32 + 16 + l] = (int8_t)(c[l] >> 4);
            }
            d_bits[r] = (uint16_t)(uint8_t)(scales[row * (size_t)scale_stride + si] - 1);
            dmin_bits[r] = 0; sc[r] = 0; m[r] = 0;
        }
    }
}

JL_EXPORT int jl_unpack_resident(jl_ctx *ctx, const jl_weight *w, int8_t *q, uint16_t *d_bits,
                                 uint16_t *dmin_bits, uint8_t *sc, uint8_t *m) {
    if (!ctx || !w || !q || !d_bits || !dmin_bits || !sc || !m) return JL_EINVAL;
    std::lock_guard<std::mutex> lk(ctx->mu);
    JL_CUDA(ctx, cudaSetDevice(ctx->device));
    size_t rows = (size_t)w->n_expert * (size_t)w->nrows;
    size_t nsub = rows * (size_t)(w->k / 32);
    const size_t nrec = w->type == JL_TYPE_Q6_K ? 2 * nsub : nsub;   // Q6_K: a record per 16 elements
    int8_t *dq = nullptr; uint16_t *dd = nullptr, *ddm = nullptr; uint8_t *dsc = nullptr, *dm = nullptr;
    cudaError_t e = cudaMalloc(&dq, nsub * 32);
    if (e == cudaSuccess) e = cudaMalloc(&dd, nrec * 2);
    if (e == cudaSuccess) e = cudaMalloc(&ddm, nrec * 2);
    if (e == cudaSuccess) e = cudaMalloc(&dsc, nrec);
    if (e == cudaSuccess) e = cudaMalloc(&dm, nrec);
    if (e == cudaSuccess) {
        int grid = (int)((nsub + 127) / 128 < 148 * 8 ? (nsub + 127) / 128 : 148 * 8);
        unpack_resident_kernel<<<grid, 128, 0, ctx->stream>>>(w->type, w->data, w->scales, w->scale_stride,
                                                             rows, w->k, dq, dd, ddm, dsc, dm);
        ctx->st.launches++;
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(q, dq, nsub * 32, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_bits, dd, nrec * 2, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dmin_bits, ddm, nrec * 2, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(sc, dsc, nrec, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m, dm, nrec, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(dq); cudaFree(dd); cudaFree(ddm); cudaFree(dsc); cudaFree(dm);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return jl_set_err(ctx, JL_ECUDA, "jl_unpack_resident: %s", cudaGetErrorString(e));
    }
    return JL_OK;
}
