// TMA (cp.async.bulk.tensor), mbarrier and tensor-map helpers for sm_100a.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ------------------------------------------------------------------- device

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Makes freshly initialised barriers visible to the async (TMA / tensor core) proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same test without any suspension: for probing a barrier ahead of the point where its result is needed.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded waits: every spin in this library gives up after a limit measured on the GPU's global
// timer and reports it, so a lost copy, a missing peer or a barrier that never fills can never
// wedge the GPU. The limit travels beside the status word the kernel reports into:
//   status[0]  code a kernel sets when a wait ran out (0 = none)
//   status[1]  the limit in microseconds (0 = JL_WAIT_DEFAULT_US)
#define JL_WAIT_DEFAULT_US 2000000u
__device__ __forceinline__ uint64_t jl_gtime_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint64_t jl_wait_limit_ns(const int *status) {
    const uint32_t us = status ? reinterpret_cast<const volatile uint32_t *>(status)[1] : 0u;
    return (uint64_t)(us ? us : JL_WAIT_DEFAULT_US) * 1000ull;
}
// Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait_ns(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    const uint64_t t0 = jl_gtime_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (jl_gtime_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const int *status) {
#pragma unroll 1
    for (int i = 0; i < 16; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_ns(bar, parity, jl_wait_limit_ns(status));
}

// One 2-D tile, global -> shared, completion counted in bytes on `bar`.
// x (innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// The same tile, only as far as L2: no shared memory, no barrier. Lets a producer keep more bytes on their way from HBM
// than its shared-memory ring holds.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma).
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// --------------------------------------------------------------------- host

// cuTensorMapEncodeTiled through the runtime's driver entry point (no -lcuda needed).
typedef CUresult (*jl_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                       const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                       CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                       CUtensorMapFloatOOBfill);

static inline jl_encode_tiled_fn jl_get_encode_tiled() {
    static jl_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (jl_encode_tiled_fn)p;
    }
    return fn;
}

// A 2-D map over `rows` x `row_elems` elements of `esize` bytes (row pitch `pitch_bytes`),
// copied in boxes of `box_rows` x `box_elems`. Returns false if the driver refuses it.
static inline bool jl_make_tmap_2d(CUtensorMap *map, const void *base, CUtensorMapDataType dt, size_t esize,
                                   uint64_t row_elems, uint64_t rows, uint64_t pitch_bytes, uint32_t box_elems,
                                   uint32_t box_rows, CUtensorMapSwizzle swz) {
    jl_encode_tiled_fn enc = jl_get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {row_elems, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_elems, box_rows};
    cuuint32_t estr[2] = {1, 1};
    (void)esize;
    return enc(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
