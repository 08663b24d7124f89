// Building blocks shared by the W4A16 (group 128) decode GEMV kernels: the
// warp-level tensor-core MMA (m16n8k16, bf16 x bf16 -> f32), the nibble -> bf16
// extraction (0x4300 | q == 128 + q exactly, one shift and one LOP3 per pair of
// codes), and the mbarrier / bulk-copy primitives.  Every mbarrier wait is
// bounded; a wait that runs out records AB2_ERR_TIMEOUT in the status word.
#pragma once

#include "common.cuh"
#include "ops.cuh"
#include "w4a16_layout.cuh"

namespace ab2 {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same with a zero C operand (starts a fresh accumulator without register moves).
__device__ __forceinline__ void mma_bf16_16816_init(float (&d)[4], uint32_t a0, uint32_t a1,
                                                    uint32_t a2, uint32_t a3, uint32_t b0,
                                                    uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Pair j of a code word: elements (2j, 2j+1) as bf16x2 holding 128 + q:
// ((word >> 4j) & 0x000F000F) | 0x43004300 as one shift and one three-input
// logic op; mask and magic are passed in registers so the logic op stays single.
__device__ __forceinline__ uint32_t w4_pair_bf16(uint32_t word, int j, uint32_t mask,
                                                 uint32_t magic) {
    uint32_t d;
    const uint32_t sh = j ? (word >> (4 * j)) : word;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(sh), "r"(mask), "r"(magic));
    return d;
}

__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// ---- mbarrier / bulk-copy primitives ---------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: false when the phase did not complete within two seconds of wall
// clock (%globaltimer; a probe may itself sleep, so counting probes bounds nothing).
// The first probe is kept out of the loop so the common case costs one instruction.
__device__ __forceinline__ unsigned long long mbar_wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    if (mbar_try_wait(addr, parity)) return true;
    unsigned long long t0 = 0;  // read only once a wait has lasted: the timer is a slow register
    for (int spin = 0;; ++spin) {
        if (mbar_try_wait(addr, parity)) return true;
        if ((spin & 31) == 31) {
            const unsigned long long now = mbar_wall_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) return false;
        }
    }
}
// global -> shared bulk copy (16-byte aligned, size a multiple of 16), completion
// counted in bytes on `bar`.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
            "r"(smem_addr(dst)),
        "l"(src), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}

constexpr int W4_BLOCK_WORDS = 272;      // 16 rows x 16 code words + 16 parameter words

// What the warp that finishes a 16-row tile stores: the projection
// (W4_EPI_STORE), the residual plus the projection (W4_EPI_ADD; `resid` may
// alias `y`), silu(gate) * up for a weight whose 16-row tiles hold 8 gate rows
// followed by the 8 matching up rows (W4_EPI_SWIGLU; y is [M][N/2]), or the f32
// sums ([M][N] floats at `y`, W4_EPI_F32): the partial result of a row-parallel
// shard, summed across ranks before it is rounded.  W4_EPI_F32_PEER stores the
// same sums into every rank's inbox of the tensor-parallel peer exchange (`y`
// then points to the ab2_tp_peer_desc in device memory).
enum { W4_EPI_STORE = 0, W4_EPI_ADD = 1, W4_EPI_SWIGLU = 2, W4_EPI_F32 = 3, W4_EPI_F32_PEER = 4 };

}  // namespace ab2
