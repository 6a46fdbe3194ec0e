// Container-packed weights: the reference's nn.Packed{QS, D, SC, Row, Stride} planes (engine/nn/device.go:62-80),
// which its .jlm containers store and JIT.MatVecPacked / MatMulPacked read (engine/nn/packed.go:24,
// engine/nn/packedmm.go:23). The planes are a permutation of the ggml blocks' fields made by kernels.PackWeights
// (jit/gpu/kernels/pack.go:27-239): [sub-block][word][row]. The kernels here stream raw blocks (whole 144-byte
// super-blocks per TMA copy), so a packed weight is re-interleaved ONCE, at upload, back into raw blocks -- the
// exact inverse of PackWeights, bit for bit -- and then served by the same kernels; jl_unpack_resident shows the
// device copy equal to the integer view of the blocks the planes were packed from.
//
//   payload  words (si * pw + w) * stride + row: sub-block si of a row, pw = 4 words for the 4-bit formats (byte j =
//            element j in the low, element j + 16 in the high nibble) or 8 words of signed bytes for Q8_0
//   d plane  Q4_K: word super * stride + row = d | dmin << 16; Q8_0: two rows a word, f16 each; MXFP4: four rows a
//            word, one stored exponent byte (e - 1) each (DIndex / DSlots, pack.go:545-575)
//   sc plane Q4_K: three words per (super-block, row), sixteen 6-bit fields -- sub-block 0's scale, its minimum,
//            sub-block 1's scale, ... -- at bit 6 f of the 96 (jit/gpu/kernels/scstream.go:26-62)
#include "jl_internal.cuh"

#include <string.h>

#include <vector>

static int packed_dslots(uint32_t t) { return t == JL_TYPE_MXFP4 ? 4 : (t == JL_TYPE_Q8_0 ? 2 : 1); }

// The 6-bit field (sub-block, scale or minimum) of a row's three stream words.
static uint8_t sc_field(const uint32_t w[3], int sub, bool min) {
    const int f = 2 * sub + (min ? 1 : 0), wi = f * 6 / 32, b = f * 6 % 32;
    uint64_t two = w[wi];
    if (wi + 1 < 3) two |= (uint64_t)w[wi + 1] << 32;
    return (uint8_t)((two >> b) & 63);
}

// The twelve scale bytes of a Q4_K block from its eight (scale, minimum) pairs: the inverse of scaleMinK4
// (format/quant/dequant.go:360-365).
static void q4k_pack_scales(const uint8_t sc[8], const uint8_t m[8], uint8_t out[12]) {
    for (int j = 0; j < 4; j++) {
        out[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        out[j + 4] = (uint8_t)((m[j] & 63) | ((m[j + 4] >> 4) << 6));
        out[j + 8] = (uint8_t)((sc[j + 4] & 0xF) | ((m[j + 4] & 0xF) << 4));
    }
}

static int packed_check(uint32_t type, const jl_packed *p, int nrows, int k, int *stride_out) {
    if (!p || !p->qs || !p->d) return JL_EINVAL;
    if (type != JL_TYPE_Q4_K && type != JL_TYPE_Q8_0 && type != JL_TYPE_MXFP4) return JL_DECLINED;
    if (nrows < 1 || k < jl_block_elems(type) || k % jl_block_elems(type)) return JL_DECLINED;
    const int stride = p->stride > 0 ? p->stride : nrows;
    if (p->row < 0 || p->row + nrows > stride) return JL_EINVAL;
    const int nsub = k / 32, pw = type == JL_TYPE_Q8_0 ? 8 : 4, ds = packed_dslots(type);
    const int nsuper = type == JL_TYPE_Q4_K ? k / 256 : nsub;
    if (p->qs_bytes < (size_t)stride * nsub * pw * 4) return JL_EINVAL;
    if (p->d_bytes < (size_t)nsuper * ((stride + ds - 1) / ds) * 4) return JL_EINVAL;
    if (type == JL_TYPE_Q4_K && (!p->sc || p->sc_bytes < (size_t)nsuper * 3 * stride * 4)) return JL_EINVAL;
    *stride_out = stride;
    return JL_OK;
}

// Planes -> raw ggml blocks, row-major: nrows x (k / block_elems * block_bytes) bytes into `raw`.
JL_EXPORT int jl_packed_to_blocks(uint32_t type, const jl_packed *p, int nrows, int k, void *raw, size_t raw_bytes) {
    int stride = 0;
    int rc = packed_check(type, p, nrows, k, &stride);
    if (rc) return rc;
    if (!raw || raw_bytes < (size_t)nrows * jl_row_bytes(type, k)) return JL_EINVAL;
    const uint32_t *qs = (const uint32_t *)p->qs, *d = (const uint32_t *)p->d, *sc = (const uint32_t *)p->sc;
    uint8_t *out = (uint8_t *)raw;
    const size_t rb = jl_row_bytes(type, k);
    for (int r = 0; r < nrows; r++) {
        const size_t R = (size_t)p->row + r;
        uint8_t *row = out + (size_t)r * rb;
        if (type == JL_TYPE_Q4_K) {
            for (int sup = 0; sup < k / 256; sup++) {
                uint8_t *blk = row + (size_t)sup * 144;
                const uint32_t dw = d[(size_t)sup * stride + R];
                blk[0] = (uint8_t)dw; blk[1] = (uint8_t)(dw >> 8); blk[2] = (uint8_t)(dw >> 16); blk[3] = (uint8_t)(dw >> 24);
                uint32_t w3[3];
                for (int w = 0; w < 3; w++) w3[w] = sc[((size_t)sup * 3 + w) * stride + R];
                uint8_t scv[8], mv[8];
                for (int s = 0; s < 8; s++) { scv[s] = sc_field(w3, s, false); mv[s] = sc_field(w3, s, true); }
                q4k_pack_scales(scv, mv, blk + 4);
                // a packed sub-block is 16 bytes: byte j = element j | element j + 16 << 4. A raw 64-element group is
                // 32 bytes: byte l = sub-block 2g's element l | sub-block 2g + 1's element l << 4.
                for (int g = 0; g < 4; g++) {
                    uint8_t pe[16], po[16];
                    for (int w = 0; w < 4; w++) {
                        const uint32_t we = qs[((size_t)(sup * 8 + 2 * g) * 4 + w) * stride + R];
                        const uint32_t wo = qs[((size_t)(sup * 8 + 2 * g + 1) * 4 + w) * stride + R];
                        memcpy(pe + 4 * w, &we, 4);
                        memcpy(po + 4 * w, &wo, 4);
                    }
                    uint8_t *grp = blk + 16 + g * 32;
                    for (int l = 0; l < 32; l++) {
                        const uint8_t qe = l < 16 ? (pe[l] & 0xF) : (pe[l - 16] >> 4);
                        const uint8_t qo = l < 16 ? (po[l] & 0xF) : (po[l - 16] >> 4);
                        grp[l] = (uint8_t)(qe | (qo << 4));
                    }
                }
            }
        } else if (type == JL_TYPE_Q8_0) {
            for (int si = 0; si < k / 32; si++) {
                uint8_t *blk = row + (size_t)si * 34;
                const uint32_t dw = d[(size_t)si * ((stride + 1) / 2) + R / 2] >> (16 * (R % 2));
                blk[0] = (uint8_t)dw; blk[1] = (uint8_t)(dw >> 8);
                for (int w = 0; w < 8; w++) {
                    const uint32_t v = qs[((size_t)si * 8 + w) * stride + R];
                    memcpy(blk + 2 + 4 * w, &v, 4);
                }
            }
        } else {   // MXFP4: the packed byte order is the block's own; the d plane holds e - 1
            for (int si = 0; si < k / 32; si++) {
                uint8_t *blk = row + (size_t)si * 17;
                blk[0] = (uint8_t)((d[(size_t)si * ((stride + 3) / 4) + R / 4] >> (8 * (R % 4))) + 1);
                for (int w = 0; w < 4; w++) {
                    const uint32_t v = qs[((size_t)si * 4 + w) * stride + R];
                    memcpy(blk + 1 + 4 * w, &v, 4);
                }
            }
        }
    }
    return JL_OK;
}

// The device copy of a packed weight (a raw-block jl_weight the ordinary kernels serve).
JL_EXPORT int jl_weight_upload_packed(jl_ctx *ctx, uint32_t type, const jl_packed *p, int nrows, int k, jl_weight **out) {
    if (!ctx || !out) return JL_EINVAL;
    int stride = 0;
    int rc = packed_check(type, p, nrows, k, &stride);
    if (rc) return jl_set_err(ctx, rc, "packed weight: %s", rc == JL_DECLINED ? "type or shape not served" : "planes do not match the shape");
    std::vector<uint8_t> raw((size_t)nrows * jl_row_bytes(type, k));
    if ((rc = jl_packed_to_blocks(type, p, nrows, k, raw.data(), raw.size()))) return jl_set_err(ctx, rc, "packed weight: re-interleave failed");
    return jl_weight_upload(ctx, type, raw.data(), raw.size(), nrows, k, out);
}

// JIT.MatVecPacked / MatMulPacked (engine/nn/packed.go:24, packedmm.go:23) on host buffers: residency is keyed on the
// payload plane's address plus the row offset (an expert of a bank shares the planes and differs in Row); the first
// call re-interleaves and uploads, later calls reuse the copy until jl_forget covers the payload plane's bytes.
JL_EXPORT int jl_matmul_packed(jl_ctx *ctx, void *out, int out_dtype, uint32_t type, const jl_packed *p, const void *x,
                               int x_dtype, int nrows, int k, int ntok) {
    if (!ctx || !out || !x || ntok < 1) return JL_EINVAL;
    if (out_dtype < 0 || out_dtype > 2 || x_dtype < 0 || x_dtype > 2) return JL_EINVAL;
    int stride = 0;
    int rc = packed_check(type, p, nrows, k, &stride);
    if (rc) return jl_set_err(ctx, rc, "packed weight: %s", rc == JL_DECLINED ? "type or shape not served" : "planes do not match the shape");
    const void *key = (const uint8_t *)p->qs + (size_t)p->row * 4;   // the row's first payload word: unique per (planes, Row)
    if (!jl_resident_known(ctx, key, type, nrows, k)) {
        std::vector<uint8_t> raw((size_t)nrows * jl_row_bytes(type, k));
        if ((rc = jl_packed_to_blocks(type, p, nrows, k, raw.data(), raw.size()))) return jl_set_err(ctx, rc, "packed weight: re-interleave failed");
        return jl_matmul_keyed(ctx, out, out_dtype, type, key, raw.data(), raw.size(), x, x_dtype, nrows, k, ntok);
    }
    return jl_matmul_keyed(ctx, out, out_dtype, type, key, nullptr, 0, x, x_dtype, nrows, k, ntok);
}

JL_EXPORT int jl_matvec_packed(jl_ctx *ctx, float *out, uint32_t type, const jl_packed *p, const float *x, int nrows, int k) {
    return jl_matmul_packed(ctx, out, JL_DT_F32, type, p, x, JL_DT_F32, nrows, k, 1);
}
