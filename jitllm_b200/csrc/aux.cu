// Neighbours of the matmul path that a decode step runs between two matmuls: residual-add + RMSNorm,
// RoPE + KV-cache append, single-query attention over the cache, SiLU(gate)*up. They exist so that a
// decoder harness can chain the quantized matvecs with ONE short launch between them (each joins the
// programmatic-dependent-launch chain the matvec kernels use); they are not part of the drop-in seam.
#include "jl_internal.cuh"
#include "q4k_prep.cuh"
#include <cuda_bf16.h>

#define AUX_PDL()                                                   \
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); \
    asm volatile("griddepcontrol.wait;" ::: "memory")

template <typename... Args>
static int aux_launch(void (*kern)(Args...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.stream = s; cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, args...) != cudaSuccess) { cudaGetLastError(); return JL_ECUDA; }
    return JL_OK;
}

__device__ __forceinline__ float aux_block_sum(float v, float *red) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += red[i];      // fixed order: bit-stable
    return t;
}

// x_io[row] += delta[row] (when delta != NULL); out[row] = x_io[row] * rsqrt(mean(x^2) + eps) * w.
__global__ void __launch_bounds__(256) aux_add_rmsnorm_kernel(float *x_io, const float *delta, const float *w, float eps,
                                                               float *out, int h) {
    __shared__ float red[8];
    AUX_PDL();
    float4 *x4 = (float4 *)(x_io + (size_t)blockIdx.x * h);
    const float4 *d4 = delta ? (const float4 *)(delta + (size_t)blockIdx.x * h) : nullptr;
    float4 *o4 = (float4 *)(out + (size_t)blockIdx.x * h);
    float ss = 0.f;
    for (int i = threadIdx.x; i < h / 4; i += 256) {
        float4 v = x4[i];
        if (d4) {
            float4 d = d4[i];
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            x4[i] = v;
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float r = rsqrtf(aux_block_sum(ss, red) / (float)h + eps);
    for (int i = threadIdx.x; i < h / 4; i += 256) {
        float4 v = x4[i];                                        // this thread's own writes
        float4 g = w ? ((const float4 *)w)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
        o4[i] = make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w);
    }
}

// The same for rows that are whole 256-element super-blocks: a warp owns a super-block in both passes, so it
// can also write the next Q4_K matvec's prepared activation operand (operand != NULL) with no launch between.
__global__ void __launch_bounds__(256) aux_add_rmsnorm_sb_kernel(float *x_io, const float *delta, const float *w, float eps,
                                                                  float *out, uint8_t *operand, int h) {
    __shared__ float red[8];
    AUX_PDL();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nsb = h / 256, row = blockIdx.x;
    float4 *x4 = (float4 *)(x_io + (size_t)row * h);
    const float4 *d4 = delta ? (const float4 *)(delta + (size_t)row * h) : nullptr;
    float ss = 0.f;
    for (int sb = warp; sb < nsb; sb += 8)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int i = sb * 64 + hf * 32 + lane;
            float4 v = x4[i];
            if (d4) {
                const float4 d = d4[i];
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                x4[i] = v;
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    const float r = rsqrtf(aux_block_sum(ss, red) / (float)h + eps);
    for (int sb = warp; sb < nsb; sb += 8) {
        float4 v[2];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int i = sb * 64 + hf * 32 + lane;
            const float4 a = x4[i];                              // this thread's own writes
            const float4 g = w ? ((const float4 *)w)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
            v[hf] = make_float4(a.x * r * g.x, a.y * r * g.y, a.z * r * g.z, a.w * r * g.w);
            if (out) ((float4 *)(out + (size_t)row * h))[i] = v[hf];
        }
        if (operand) q4k_prep_sb_vals(v[0], v[1], operand + ((size_t)row * nsb + sb) * Q4K_XP_SB_BYTES, lane);
    }
}

// The same producer for the batched path: the normalised row goes out as the tcgen05 GEMM's activation operand (the
// f16 hi / lo rows and the power-of-two scale act_to_f16_kernel would make of the f32 row, bit for bit), so that no
// conversion launch sits between the norm and the GEMM. Same ownership of super-blocks by warps as above, hence the
// same sums.
__global__ void __launch_bounds__(256) aux_add_rmsnorm_gemm_kernel(float *x_io, const float *delta, const float *w, float eps,
                                                                    __half *rows, float *inv_scale, int h) {
    __shared__ float red[8];
    AUX_PDL();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nsb = h / 256, row = blockIdx.x;
    float4 *x4 = (float4 *)(x_io + (size_t)row * h);
    const float4 *d4 = delta ? (const float4 *)(delta + (size_t)row * h) : nullptr;
    float ss = 0.f;
    for (int sb = warp; sb < nsb; sb += 8)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int i = sb * 64 + hf * 32 + lane;
            float4 v = x4[i];
            if (d4) {
                const float4 d = d4[i];
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                x4[i] = v;
            }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    const float r = rsqrtf(aux_block_sum(ss, red) / (float)h + eps);
    auto normed = [&](int i) {
        const float4 a = x4[i];                                  // this thread's own writes
        const float4 g = w ? ((const float4 *)w)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
        return make_float4(a.x * r * g.x, a.y * r * g.y, a.z * r * g.z, a.w * r * g.w);
    };
    float amax = 0.f;
    for (int sb = warp; sb < nsb; sb += 8)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const float4 v = normed(sb * 64 + hf * 32 + lane);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __syncthreads();                                             // red[] was read by everyone above
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    // the scale act_to_f16_kernel picks: a power of two that puts the row's largest magnitude in [2^14, 2^15)
    const int e = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127;
    int s = 14 - e;
    if (amax == 0.f || !(amax < __int_as_float(0x7f800000))) s = 0;
    s = max(-100, min(100, s));
    const float scale = __uint_as_float((uint32_t)(127 + s) << 23);
    if (threadIdx.x == 0) inv_scale[row] = __uint_as_float((uint32_t)(127 - s) << 23);
    __half *hi = rows + (size_t)(2 * row) * h, *lo = hi + h;
    for (int sb = warp; sb < nsb; sb += 8)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int i = sb * 64 + hf * 32 + lane;
            const float4 v = normed(i);
            const float a[4] = {v.x * scale, v.y * scale, v.z * scale, v.w * scale};
            uint32_t hw[2], lw[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const __half2 hh = __floats2half2_rn(a[2 * j], a[2 * j + 1]);
                const float2 back = __half22float2(hh);
                const __half2 ll = __floats2half2_rn(a[2 * j] - back.x, a[2 * j + 1] - back.y);
                hw[j] = *reinterpret_cast<const uint32_t *>(&hh);
                lw[j] = *reinterpret_cast<const uint32_t *>(&ll);
            }
            *reinterpret_cast<uint2 *>(hi + (size_t)i * 4) = make_uint2(hw[0], hw[1]);
            *reinterpret_cast<uint2 *>(lo + (size_t)i * 4) = make_uint2(lw[0], lw[1]);
        }
}

// One warp per 256 outputs: out and/or the prepared operand of the matvec that consumes them.
__global__ void __launch_bounds__(128) aux_silu_mul_sb_kernel(float *out, uint8_t *operand, const float *gu, int ffn) {
    AUX_PDL();
    const int lane = threadIdx.x & 31, sb = blockIdx.x * 4 + (threadIdx.x >> 5), row = blockIdx.y, nsb = ffn / 256;
    if (sb >= nsb) return;
    const float4 *g4 = (const float4 *)(gu + (size_t)row * 2 * ffn);
    const float4 *u4 = g4 + ffn / 4;
    float4 v[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        const int i = sb * 64 + hf * 32 + lane;
        const float4 g = g4[i], u = u4[i];
        v[hf] = make_float4(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y,
                            g.z / (1.f + __expf(-g.z)) * u.z, g.w / (1.f + __expf(-g.w)) * u.w);
        if (out) ((float4 *)(out + (size_t)row * ffn))[i] = v[hf];
    }
    if (operand) q4k_prep_sb_vals(v[0], v[1], operand + ((size_t)row * nsb + sb) * Q4K_XP_SB_BYTES, lane);
}

__global__ void __launch_bounds__(256) aux_silu_mul_kernel(float *out, const float *gu, int ffn) {
    AUX_PDL();
    const float4 *g4 = (const float4 *)(gu + (size_t)blockIdx.y * 2 * ffn);
    const float4 *u4 = g4 + ffn / 4;
    float4 *o4 = (float4 *)(out + (size_t)blockIdx.y * ffn);
    for (int i = blockIdx.x * 256 + threadIdx.x; i < ffn / 4; i += gridDim.x * 256) {
        float4 g = g4[i], u = u4[i];
        o4[i] = make_float4(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y,
                            g.z / (1.f + __expf(-g.z)) * u.z, g.w / (1.f + __expf(-g.w)) * u.w);
    }
}

// qkv [n][(hq + 2 hkv) * d] f32 -> q_out [n][hq][d] bf16 (rotated), k (rotated) and v appended to the
// caches [n][hkv][max_len][d] bf16 at position *pos. Adjacent-pair rotation; cos/sin are [max_len][d/2].
__global__ void __launch_bounds__(64) aux_rope_kv_kernel(__nv_bfloat16 *q_out, const float *qkv, __nv_bfloat16 *k_cache,
                                                          __nv_bfloat16 *v_cache, const long long *pos_dev, const float *cos_t,
                                                          const float *sin_t, int hq, int hkv, int d, int max_len) {
    AUX_PDL();
    const int row = blockIdx.y, hd = blockIdx.x;
    const long long pos = *pos_dev;
    if (pos < 0 || pos >= max_len) return;
    const float *src = qkv + (size_t)row * (hq + 2 * hkv) * d + (size_t)hd * d;
    for (int j = threadIdx.x; j < d / 2; j += 64) {
        float a = src[2 * j], b = src[2 * j + 1];
        __nv_bfloat162 o;
        if (hd < hq + hkv) {
            const float c = cos_t[pos * (d / 2) + j], s = sin_t[pos * (d / 2) + j];
            o = __floats2bfloat162_rn(a * c - b * s, a * s + b * c);
        } else {
            o = __floats2bfloat162_rn(a, b);
        }
        __nv_bfloat16 *dst;
        if (hd < hq) dst = q_out + ((size_t)row * hq + hd) * d;
        else if (hd < hq + hkv) dst = k_cache + (((size_t)row * hkv + (hd - hq)) * max_len + pos) * d;
        else dst = v_cache + (((size_t)row * hkv + (hd - hq - hkv)) * max_len + pos) * d;
        ((__nv_bfloat162 *)dst)[j] = o;
    }
}

// ------------------------------------------------------------------ single-query attention over the cache
// One CTA = one (sequence, kv head, chunk of ATT_CHUNK cache positions), all G query heads of the kv head
// at once (K and V rows are read once for the group). Partial (max, sum, weighted V) triples go to scratch;
// the CTA that takes the last ticket of its (sequence, kv head) merges them -- no CTA waits for another.
#define ATT_CHUNK 64
#define ATT_D 128
#define ATT_ROW 272   // bytes of one staged row: 256 + 16 of padding, so that rows start in different banks

__device__ __forceinline__ void aux_bf16x8(const uint4 &v, float *f) {
    const __nv_bfloat162 *p = (const __nv_bfloat162 *)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

// D (16 x 8, f32) += A (16 x 16 bf16, row) * B (16 x 8 bf16, col).
__device__ __forceinline__ void aux_mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#ifndef ATT_MIN_CTAS
#define ATT_MIN_CTAS 5          // 96 registers: five CTAs per SM (shared memory would allow six, but at 80 registers the kernel spills)
#endif
template <int G>
__global__ void __launch_bounds__(128, ATT_MIN_CTAS) aux_attn_decode_kernel(float *out, uint8_t *operand, const __nv_bfloat16 *q,
                                                              const __nv_bfloat16 *k_cache, const __nv_bfloat16 *v_cache,
                                                              const long long *pos_dev, float *part, unsigned *tickets, int hkv,
                                                              int max_len, int nsplit) {
    constexpr int HDR = (2 * G + 3) & ~3;              // max[G], sum[G], padded so that the V part is 16-byte aligned
    constexpr int STRIDE = HDR + G * ATT_D;
    // K and V tiles of the chunk, staged with coalesced 16-byte loads (all in flight at once); the
    // cross-group reduction buffer red[8][G][128] reuses the tiles once they have been consumed.
    __shared__ __align__(16) uint8_t tiles[2 * ATT_CHUNK * ATT_ROW];
    static_assert(4 * G * ATT_D * 4 <= 2 * ATT_CHUNK * ATT_ROW, "reduction buffer must fit in the tiles");
    __shared__ float mred[4][G], lred[4][G];
    __shared__ unsigned last;
    const int split = blockIdx.x, kv = blockIdx.y, row = blockIdx.z, t = threadIdx.x, hq = hkv * G;
    AUX_PDL();
    long long len = *pos_dev + 1;
    if (len > max_len) len = max_len;
    const int s0 = split * ATT_CHUNK;
    const int cnt = len - s0 < 0 ? 0 : (len - s0 > ATT_CHUNK ? ATT_CHUNK : (int)(len - s0));
    float *my = part + (((size_t)row * hkv + kv) * nsplit + split) * STRIDE;
    if (cnt > 0) {
        const size_t base_row = ((size_t)row * hkv + kv) * max_len + s0;
        const uint4 *kg = (const uint4 *)(k_cache + base_row * ATT_D), *vg = (const uint4 *)(v_cache + base_row * ATT_D);
        uint4 kreg[8], vreg[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {                            // 1024 16-byte pieces per tile, 8 per thread
            const int piece = i * 128 + t;
            kreg[i] = (piece >> 4) < cnt ? kg[piece] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int piece = i * 128 + t;
            vreg[i] = (piece >> 4) < cnt ? vg[piece] : make_uint4(0, 0, 0, 0);
        }
        // Scores and the weighted sum of V run on the tensor cores (mma.sync m16n8k16, bf16 in, f32 accumulate): the M
        // rows are the group's G query heads (rows G..15 are zero), a warp takes 16 of the chunk's 64 positions. q and
        // the cached K, V are bf16 as stored, so the products are exact; the softmax weights go in as a bf16 pair
        // (value + what the first rounding left: 16 significant bits). Per byte of cache this is a quarter of the
        // instructions of a scalar loop, which is what bounded the kernel at batch 64.
        const int warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
        uint32_t qa[8][2];                                      // A fragments of q: k-step s covers dims 16 s .. 16 s + 15
        {
            const uint32_t *qrow = reinterpret_cast<const uint32_t *>(q + ((size_t)row * hq + kv * G + (g < G ? g : 0)) * ATT_D);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qa[ks][0] = g < G ? __ldg(qrow + ks * 8 + tq) : 0u;            // dims 16 ks + 2 tq, + 1
                qa[ks][1] = g < G ? __ldg(qrow + ks * 8 + 4 + tq) : 0u;        // dims 16 ks + 8 + 2 tq, + 1
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int piece = i * 128 + t;
            *(uint4 *)(tiles + (piece >> 4) * ATT_ROW + (piece & 15) * 16) = kreg[i];
            *(uint4 *)(tiles + (ATT_CHUNK + (piece >> 4)) * ATT_ROW + (piece & 15) * 16) = vreg[i];
        }
        __syncthreads();
        const uint32_t tiles_s = (uint32_t)__cvta_generic_to_shared(tiles);
        const int p0 = warp * 16;                               // the warp's positions p0 .. p0 + 15 of the chunk
        // S[h][pos]: two n-tiles of 8 positions; lane (g, tq) ends up with S[g][p0 + 8 nt + 2 tq, + 1]
        float sacc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[nt][e] = 0.f;
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {                    // two k-steps (32 dims) per ldmatrix.x4
                // matrices: K[p0 + 8 nt + 0..7][dims 32 kp + 0..7 | 8..15 | 16..23 | 24..31]
                const uint32_t addr = tiles_s + (p0 + 8 * nt + (lane & 7)) * ATT_ROW + (32 * kp + 8 * (lane >> 3)) * 2;
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
                aux_mma_bf16(sacc[nt], qa[2 * kp][0], 0u, qa[2 * kp][1], 0u, b0, b1);
                aux_mma_bf16(sacc[nt], qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u, b2, b3);
            }
        }
        float sv[4];                                            // this lane's four scores of head g
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int pos = p0 + 8 * nt + 2 * tq + e;
                sv[2 * nt + e] = pos < cnt ? sacc[nt][e] * 0.08838834764831845f : -INFINITY;
            }
        {
            float m = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            if (tq == 0 && g < G) mred[warp][g] = m;
        }
        __syncthreads();
        const int gh = g < G ? g : 0;
        const float M = fmaxf(fmaxf(mred[0][gh], mred[1][gh]), fmaxf(mred[2][gh], mred[3][gh]));
        float pv[4], l = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            pv[e] = (g < G && sv[e] > -INFINITY) ? __expf(sv[e] - M) : 0.f;
            l += pv[e];
        }
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (tq == 0 && g < G) lred[warp][g] = l;
        // A fragments of the weights: positions p0 + 2 tq, + 1 (a0) and p0 + 8 + 2 tq, + 1 (a2), as value + remainder
        uint32_t ph[2], pl[2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const __nv_bfloat162 hi = __floats2bfloat162_rn(pv[2 * nt], pv[2 * nt + 1]);
            const float2 hf = __bfloat1622float2(hi);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(pv[2 * nt] - hf.x, pv[2 * nt + 1] - hf.y);
            ph[nt] = *reinterpret_cast<const uint32_t *>(&hi);
            pl[nt] = *reinterpret_cast<const uint32_t *>(&lo);
        }
        // O[h][dim] += P[h][pos] V[pos][dim]: sixteen n-tiles of 8 dims, two per ldmatrix.x4.trans
        float oacc[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) oacc[j][e] = 0.f;
#pragma unroll
        for (int jp = 0; jp < 8; ++jp) {
            // matrices: V[p0 + 0..7][dims 16 jp + 0..7], V[p0 + 8..15][same], V[p0 + 0..7][dims 16 jp + 8..15], V[p0 + 8..15][same]
            const int mi = lane >> 3;
            const uint32_t addr = tiles_s + (ATT_CHUNK + p0 + 8 * (mi & 1) + (lane & 7)) * ATT_ROW + (16 * jp + 8 * (mi >> 1)) * 2;
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
            aux_mma_bf16(oacc[2 * jp], ph[0], 0u, ph[1], 0u, b0, b1);
            aux_mma_bf16(oacc[2 * jp], pl[0], 0u, pl[1], 0u, b0, b1);
            aux_mma_bf16(oacc[2 * jp + 1], ph[0], 0u, ph[1], 0u, b2, b3);
            aux_mma_bf16(oacc[2 * jp + 1], pl[0], 0u, pl[1], 0u, b2, b3);
        }
        __syncthreads();                                        // tiles consumed (and lred complete): reuse them
        if (t < G) {
            my[t] = fmaxf(fmaxf(mred[0][t], mred[1][t]), fmaxf(mred[2][t], mred[3][t]));
            my[G + t] = (lred[0][t] + lred[1][t]) + (lred[2][t] + lred[3][t]);
        }
        float(*red)[G][ATT_D] = (float(*)[G][ATT_D])tiles;      // red[warp][head][dim]
        if (g < G) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                *reinterpret_cast<float2 *>(&red[warp][g][8 * j + 2 * tq]) = make_float2(oacc[j][0], oacc[j][1]);
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < G; ++h)
            my[HDR + h * ATT_D + t] = (red[0][h][t] + red[1][h][t]) + (red[2][h][t] + red[3][h][t]);
    } else if (t < G) {
        my[t] = -INFINITY;
        my[G + t] = 0.f;
    }
    __threadfence();
    __syncthreads();
    if (t == 0) last = atomicAdd(&tickets[row * hkv + kv], 1u) == (unsigned)(nsplit - 1);
    __syncthreads();
    if (!last) return;
    __threadfence();
    const float *base = part + ((size_t)row * hkv + kv) * nsplit * STRIDE;
    const int nlive = (int)((len + ATT_CHUNK - 1) / ATT_CHUNK);   // chunks past the sequence hold nothing
    // Merge: warp w takes heads w, w+4, ...; its lanes first scan the chunks' (max, sum) pairs side by side,
    // then each lane owns four output dims and walks the chunks in ascending order (bit-stable) with the
    // loads of eight chunks in flight at a time.
    {
        const int warp = t >> 5, lane = t & 31;
        for (int h = warp; h < G; h += 4) {
            // every lane keeps the (max, sum) of chunks lane, lane+32, ... (up to MAXR of them) in registers:
            // one round trip to L2 for all of them, then the weights exp(m_s - M) are handed round by shuffle
            constexpr int MAXR = 4;                             // 128 chunks = 8192 cached positions per merge pass
            float mr[MAXR], lr[MAXR];
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int s = lane + 32 * r;
                mr[r] = s < nlive ? __ldcg(base + (size_t)s * STRIDE + h) : -INFINITY;
                lr[r] = s < nlive ? __ldcg(base + (size_t)s * STRIDE + G + h) : 0.f;
            }
            float M = fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3]));
            for (int s = lane + 32 * MAXR; s < nlive; s += 32) M = fmaxf(M, __ldcg(base + (size_t)s * STRIDE + h));
            for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            float L = 0.f;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                mr[r] = __expf(mr[r] - M);                      // now the chunk's weight (0 for chunks that do not exist)
                L = fmaf(lr[r], mr[r], L);
            }
            for (int s = lane + 32 * MAXR; s < nlive; s += 32)
                L += __ldcg(base + (size_t)s * STRIDE + G + h) * __expf(__ldcg(base + (size_t)s * STRIDE + h) - M);
            for (int o = 16; o; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const float *ob = base + HDR + h * ATT_D + 4 * lane;
            const int nreg = nlive < 32 * MAXR ? nlive : 32 * MAXR;
            int s = 0;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                for (int s0b = 32 * r; s0b < nreg && s0b < 32 * (r + 1); s0b += 16) {   // ascending chunk order: bit-stable
                    float4 v[16];
#pragma unroll
                    for (int u = 0; u < 16; ++u)
                        v[u] = s0b + u < nreg ? __ldcg(reinterpret_cast<const float4 *>(ob + (size_t)(s0b + u) * STRIDE))
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const float w = __shfl_sync(0xffffffffu, mr[r], (s0b + u) & 31);
                        acc.x = fmaf(v[u].x, w, acc.x); acc.y = fmaf(v[u].y, w, acc.y);
                        acc.z = fmaf(v[u].z, w, acc.z); acc.w = fmaf(v[u].w, w, acc.w);
                    }
                }
            }
            for (s = nreg; s < nlive; ++s) {                    // very long sequences: the plain walk
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(ob + (size_t)s * STRIDE));
                const float w = __expf(__ldcg(base + (size_t)s * STRIDE + h) - M);
                acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y);
                acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            const float4 res = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
            if (out) *reinterpret_cast<float4 *>(out + (size_t)row * hq * ATT_D + (size_t)(kv * G + h) * ATT_D + 4 * lane) = res;
            if (operand) reinterpret_cast<float4 *>(tiles)[h * (ATT_D / 4) + lane] = res;
        }
    }
    if (t == 0) tickets[row * hkv + kv] = 0;                    // ready for the next launch
    if constexpr (G % 2 == 0) {
        if (operand) {
            // two heads = one 256-element super-block of the output projection's input: write its prepared operand
            __syncthreads();
            const int warp = t >> 5, lane = t & 31;
            if (warp < G / 2) {
                const float4 *c4 = reinterpret_cast<const float4 *>(tiles) + warp * 64;
                q4k_prep_sb_vals(c4[lane], c4[32 + lane],
                                 operand + ((size_t)row * (hq / 2) + kv * (G / 2) + warp) * Q4K_XP_SB_BYTES, lane);
            }
        }
    }
}

// First index of the row maximum (ties: the lowest index, as a sequential scan gives).
__global__ void __launch_bounds__(1024) aux_argmax_kernel(long long *out, const float *x, int v) {
    __shared__ float bm[32];
    __shared__ int bi[32];
    AUX_PDL();
    const float *r = x + (size_t)blockIdx.x * v;
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = threadIdx.x; i < v; i += 1024) {
        const float f = r[i];
        if (f > m || (f == m && i < mi)) { m = f; mi = i; }
    }
    for (int o = 16; o; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bm[threadIdx.x >> 5] = m; bi[threadIdx.x >> 5] = mi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        m = bm[threadIdx.x]; mi = bi[threadIdx.x];
        for (int o = 16; o; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o);
            const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
            if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = mi == 0x7fffffff ? 0 : mi;
    }
}

static size_t aux_attn_ticket_bytes(int n, int hkv) { return (((size_t)n * hkv * 4) + 255) & ~(size_t)255; }

// ------------------------------------------------------------------ C ABI
// The kernels use 16-byte vector accesses: a pointer that is not 16-byte aligned is refused here, on the host.
static inline bool aux_misaligned(const void *p) { return p && ((uintptr_t)p & 15u); }
JL_EXPORT int jl_aux_add_rmsnorm(float *x_io, const float *delta, const float *w, float eps, float *out, void *operand_out,
                                 int n, int h, void *stream) {
    if (!x_io || (!out && !operand_out) || n < 1 || h < 4 || h % 4) return JL_EINVAL;
    if (aux_misaligned(x_io) || aux_misaligned(delta) || aux_misaligned(w) || aux_misaligned(out) || aux_misaligned(operand_out))
        return JL_EINVAL;
    if (h % 256 == 0)
        return aux_launch(aux_add_rmsnorm_sb_kernel, dim3(n), dim3(256), (cudaStream_t)stream, x_io, delta, w, eps, out,
                          (uint8_t *)operand_out, h);
    if (operand_out || !out) return JL_EINVAL;          // the prepared operand is made of whole super-blocks
    return aux_launch(aux_add_rmsnorm_kernel, dim3(n), dim3(256), (cudaStream_t)stream, x_io, delta, w, eps, out, h);
}

JL_EXPORT int jl_aux_add_rmsnorm_gemm(float *x_io, const float *delta, const float *w, float eps, void *rows_f16,
                                      float *inv_scale, int n, int h, void *stream) {
    if (!x_io || !rows_f16 || !inv_scale || n < 1 || h < 256 || h % 256) return JL_EINVAL;
    if (aux_misaligned(x_io) || aux_misaligned(delta) || aux_misaligned(w) || aux_misaligned(rows_f16)) return JL_EINVAL;
    return aux_launch(aux_add_rmsnorm_gemm_kernel, dim3(n), dim3(256), (cudaStream_t)stream, x_io, delta, w, eps,
                      (__half *)rows_f16, inv_scale, h);
}

JL_EXPORT int jl_aux_silu_mul(float *out, void *operand_out, const float *gu, int n, int ffn, void *stream) {
    if ((!out && !operand_out) || !gu || n < 1 || ffn < 4 || ffn % 4) return JL_EINVAL;
    if (aux_misaligned(out) || aux_misaligned(gu) || aux_misaligned(operand_out)) return JL_EINVAL;
    if (ffn % 256 == 0)
        return aux_launch(aux_silu_mul_sb_kernel, dim3((ffn / 256 + 3) / 4, n), dim3(128), (cudaStream_t)stream, out,
                          (uint8_t *)operand_out, gu, ffn);
    if (operand_out || !out) return JL_EINVAL;
    int gx = (ffn / 4 + 255) / 256;
    if (gx > 64) gx = 64;
    return aux_launch(aux_silu_mul_kernel, dim3(gx, n), dim3(256), (cudaStream_t)stream, out, gu, ffn);
}

JL_EXPORT int jl_aux_argmax(long long *out, const float *x, int n, int v, void *stream) {
    if (!out || !x || n < 1 || v < 1) return JL_EINVAL;
    return aux_launch(aux_argmax_kernel, dim3(n), dim3(1024), (cudaStream_t)stream, out, x, v);
}

JL_EXPORT int jl_aux_rope_kv(void *q_out_bf16, const float *qkv, void *k_cache_bf16, void *v_cache_bf16,
                             const long long *pos_dev, const float *cos_t, const float *sin_t, int n, int hq, int hkv, int d,
                             int max_len, void *stream) {
    if (!q_out_bf16 || !qkv || !k_cache_bf16 || !v_cache_bf16 || !pos_dev || !cos_t || !sin_t) return JL_EINVAL;
    if (n < 1 || hq < 1 || hkv < 1 || d < 2 || d % 2 || max_len < 1) return JL_EINVAL;
    return aux_launch(aux_rope_kv_kernel, dim3(hq + 2 * hkv, n), dim3(64), (cudaStream_t)stream,
                      (__nv_bfloat16 *)q_out_bf16, qkv, (__nv_bfloat16 *)k_cache_bf16, (__nv_bfloat16 *)v_cache_bf16, pos_dev,
                      cos_t, sin_t, hq, hkv, d, max_len);
}

JL_EXPORT size_t jl_aux_attn_scratch_bytes(int n, int hq, int hkv, int max_len) {
    if (n < 1 || hq < 1 || hkv < 1 || hq % hkv || max_len < 1) return 0;
    const int g = hq / hkv, nsplit = (max_len + ATT_CHUNK - 1) / ATT_CHUNK;
    return aux_attn_ticket_bytes(n, hkv) + (size_t)n * hkv * nsplit * (((2 * g + 3) & ~3) + g * ATT_D) * sizeof(float);
}

JL_EXPORT int jl_aux_attn_decode(float *out, void *operand_out, const void *q_bf16, const void *k_cache_bf16,
                                 const void *v_cache_bf16, const long long *pos_dev, void *scratch_zeroed_once, int n, int hq,
                                 int hkv, int d, int max_len, void *stream) {
    if ((!out && !operand_out) || !q_bf16 || !k_cache_bf16 || !v_cache_bf16 || !pos_dev || !scratch_zeroed_once) return JL_EINVAL;
    if (n < 1 || hkv < 1 || hq % hkv || d != ATT_D || max_len < 1) return JL_EINVAL;
    if (aux_misaligned(out) || aux_misaligned(operand_out) || aux_misaligned(q_bf16) || aux_misaligned(k_cache_bf16) ||
        aux_misaligned(v_cache_bf16) || aux_misaligned(scratch_zeroed_once))
        return JL_EINVAL;
    const int g = hq / hkv, nsplit = (max_len + ATT_CHUNK - 1) / ATT_CHUNK;
    if (operand_out && (g & 1)) return JL_EINVAL;      // a super-block of the operand is two heads
    unsigned *tickets = (unsigned *)scratch_zeroed_once;
    float *part = (float *)((uint8_t *)scratch_zeroed_once + aux_attn_ticket_bytes(n, hkv));
    const dim3 grid(nsplit, hkv, n), block(128);
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t *op = (uint8_t *)operand_out;
    const __nv_bfloat16 *q = (const __nv_bfloat16 *)q_bf16, *kc = (const __nv_bfloat16 *)k_cache_bf16,
                        *vc = (const __nv_bfloat16 *)v_cache_bf16;
    switch (g) {
    case 1: return aux_launch(aux_attn_decode_kernel<1>, grid, block, s, out, op, q, kc, vc, pos_dev, part, tickets, hkv, max_len, nsplit);
    case 2: return aux_launch(aux_attn_decode_kernel<2>, grid, block, s, out, op, q, kc, vc, pos_dev, part, tickets, hkv, max_len, nsplit);
    case 4: return aux_launch(aux_attn_decode_kernel<4>, grid, block, s, out, op, q, kc, vc, pos_dev, part, tickets, hkv, max_len, nsplit);
    case 8: return aux_launch(aux_attn_decode_kernel<8>, grid, block, s, out, op, q, kc, vc, pos_dev, part, tickets, hkv, max_len, nsplit);
    }
    return JL_ENOTSUP;
}
