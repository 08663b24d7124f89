// tcgen05 / TMA building blocks shared by the W4A16 tensor-memory kernels
// (internal header): mbarrier helpers with bounded waits, bulk and tensor-map
// copies, the K-major 128-byte-swizzle shared-memory descriptor, the bf16 MMA
// issue and commit, and the host-side tensor map of a [rows][K] bf16 matrix.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace ab2 {
namespace tc {

__device__ __forceinline__ uint32_t sptr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }


__device__ __forceinline__ void bar_init(uint64_t *b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(sptr(b)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t *b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(sptr(b)) : "memory");
}
// Arrival that hands a shared-memory slot back to a producer of asynchronous copies.  The arrival
// must not leave while a load of the slot is still under way (the copy that follows it may land
// first): `held` is a value every such load has fed, `hidden_zero` a zero the compiler cannot see
// (derived from a kernel argument); the address of the arrival takes in held & hidden_zero, so the
// instruction waits for the loads.
__device__ __forceinline__ void bar_arrive_after(uint64_t *b, uint32_t held, uint32_t hidden_zero) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(sptr(b) + (held & hidden_zero)) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t *b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(sptr(b)), "r"(bytes) : "memory");
}
// Bounded wait (two seconds of wall clock, read from %globaltimer; a probe may itself
// sleep for a while, so counting probes bounds nothing); also gives up as soon as another
// warp of the CTA has failed.
__device__ __forceinline__ unsigned long long wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool bar_wait(uint64_t *b, uint32_t parity, volatile int *failed) {
    const uint32_t addr = sptr(b);
    unsigned long long t0 = 0;
    for (int spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((spin & 31) == 31) {  // the timer is a slow register: read only once a wait has lasted
            if (*failed) return false;
            const unsigned long long now = wall_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) break;
        }
    }
    *failed = 1;
    return false;
}

__device__ __forceinline__ void bulk_copy(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
                     "r"(sptr(dst)), "l"(src), "r"(bytes), "r"(sptr(bar)) : "memory");
}
// 2-D tile load: coordinates (k element, token row); completion counted on `bar`.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::
            "r"(sptr(dst)), "l"(map), "r"(sptr(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: 8-row groups are
// 1024 bytes apart, the start address advances by 32 bytes per K = 16 step.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major): 1
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;             // descriptor version
    d |= (uint64_t)2 << 61;             // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::
            "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(sptr(bar)) : "memory");
}

__device__ __forceinline__ uint32_t bf16x2_add_(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_mul_(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}


typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int make_x_map(CUtensorMap *map, const void *x, int M, int K, int ntok) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        AB2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        AB2_REQUIRE(fn != nullptr && qres == cudaDriverEntryPointSuccess, AB2_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is unavailable");
        encode = (EncodeTiledFn)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)ntok};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    AB2_REQUIRE(r == CUDA_SUCCESS, AB2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return AB2_OK;
}


}  // namespace tc
}  // namespace ab2
