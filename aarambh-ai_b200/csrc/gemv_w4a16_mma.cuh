// W4A16 (group 128, bf16 activations) decode GEMV for 1..16 tokens.
//
// HBM-bound.  The weight lives in tile-major blocks (w4a16_layout.cuh): the 16
// rows x 128 columns a warp needs for one step, plus their 16 parameter words,
// are 1088 contiguous bytes, and a 16-row tile is one contiguous run.  A
// persistent CTA streams its tiles through a ring of shared-memory stages
// filled by bulk asynchronous copies (cp.async.bulk, completion on an
// mbarrier), so every packed byte crosses HBM once, several stages are in
// flight per CTA, and no registers are held by loads in flight.
//
// Each of the 8 warps takes one group of a stage.  Nibbles become bf16 with one
// LOP3 per pair (0x4300 | q == 128 + q exactly) and feed the warp-level
// tensor-core MMA (m16n8k16, bf16 x bf16 -> f32) with the 16 weight rows as
// the A operand and up to 8 tokens as the B operand, straight from registers.
// The zero point is applied by a second MMA whose A operand is the constant
// -(128 + z) (exact in bf16; up to 8 tokens the tensor pipe has room and the
// integer pipe does not) or, for 9..16 tokens, by an exact bf16x2 add on the A
// registers, so each group's accumulator holds sum_k x_k (q_k - z) up to f32
// accumulation; the bf16 scale is applied once per group in f32.  CUDA-core FMA cannot keep
// up with HBM here (fewer than 3 issue slots per weight are available at full
// bandwidth), which is why the tensor path is used even for one token.
//
// Every mbarrier wait is bounded; a wait that runs out records
// AB2_ERR_TIMEOUT in the status word and the CTA returns.
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
// Bounded wait: false when the phase did not complete within the limit.  The
// first probe is kept out of the loop so the common case costs one instruction.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    if (mbar_try_wait(addr, parity)) return true;
    for (int spin = 0; spin < (1 << 22); ++spin)
        if (mbar_try_wait(addr, parity)) return true;
    return false;
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
constexpr int W4_GROUPS_PER_STAGE = 8;   // one group per warp
constexpr int W4_STAGE_WORDS = W4_GROUPS_PER_STAGE * W4_BLOCK_WORDS;

// NT = number of 8-token tiles (1 or 2).  Token rows at or beyond M are read
// from row M-1 instead (their output columns are never stored), so the loop
// carries no predicates.  grid.x <= number of 16-row tiles.
//
// The 8 warps of a CTA each own one group of a stage and keep their own f32
// partial sums of the tile; at the end of a tile each warp publishes its
// partials and the warp that arrives last adds the eight in fixed order and
// stores the outputs, so there is no CTA-wide barrier in the steady state and
// the result does not depend on arrival order.  Two partial buffers suffice
// because a warp can run at most `stages` <= chunks items ahead of another.
//
// EPI selects what the reducing warp stores: the projection (W4_EPI_STORE), the
// residual plus the projection (W4_EPI_ADD; `resid` may alias `y`), or
// silu(gate) * up for a weight whose 16-row tiles hold 8 gate rows followed by
// the 8 matching up rows (W4_EPI_SWIGLU; y is [M][N/2]).
// W4_EPI_F32 stores the f32 sums ([M][N] floats at `y`): the partial result of a
// row-parallel shard, summed across ranks before it is rounded.
enum { W4_EPI_STORE = 0, W4_EPI_ADD = 1, W4_EPI_SWIGLU = 2, W4_EPI_F32 = 3 };

template <int NT, int EPI>
__global__ void __launch_bounds__(256)
gemv_w4a16_stream_kernel(const uint32_t *__restrict__ wt, const __nv_bfloat16 *__restrict__ x,
                         __nv_bfloat16 *y, const __nv_bfloat16 *resid, int N, int K, int M,
                         int *status) {
    constexpr int MAX_STAGES = NT == 1 ? 4 : 3;  // keeps static shared memory under 48 KB
    __shared__ alignas(128) uint32_t ring[MAX_STAGES][W4_STAGE_WORDS];
    __shared__ float red[2][8][16][8 * NT + 1];
    __shared__ alignas(8) uint64_t full_bar[MAX_STAGES];
    __shared__ alignas(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ int arrivals[2];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int G = K >> 7, chunks = (G + 7) >> 3, tiles = (N + 15) >> 4;
    const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int items = my_tiles * chunks;
    const int stages = min(MAX_STAGES, chunks);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 8);
        }
        arrivals[0] = 0;
        arrivals[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    // Producer state (thread 0): next item to load, as (tile index, chunk, slot).
    const bool producer = threadIdx.x == 0;
    int p_item = 0, p_tile = blockIdx.x, p_chunk = 0, p_slot = 0;
    auto issue_next = [&]() {
        const int ng = min(W4_GROUPS_PER_STAGE, G - p_chunk * W4_GROUPS_PER_STAGE);
        const uint32_t bytes = (uint32_t)ng * W4_BLOCK_WORDS * 4;
        const uint32_t *src =
            wt + ((size_t)p_tile * G + (size_t)p_chunk * W4_GROUPS_PER_STAGE) * W4_BLOCK_WORDS;
        mbar_arrive_expect_tx(&full_bar[p_slot], bytes);
        bulk_g2s(&ring[p_slot][0], src, bytes, &full_bar[p_slot]);
        ++p_item;
        if (++p_chunk == chunks) { p_chunk = 0; p_tile += gridDim.x; }
        if (++p_slot == stages) p_slot = 0;
    };
    if (producer)
        for (int j = 0; j < min(stages, items); ++j) issue_next();

    // The weights are constant, so their first stages are already in flight; the
    // activations (and the residual) come from the preceding kernel.
    pdl_wait();
    pdl_launch_dependents();

    // Opaque register copies of the two constants of the nibble extraction.
    uint32_t k_mask = 0x000F000Fu, k_magic = 0x43004300u;
    asm volatile("" : "+r"(k_mask), "+r"(k_magic));

    const uint32_t lane_words = r * 16 + c * 4;  // this thread's 4 words of row r in a block
    int slot = 0, prev_slot = 0;
    uint32_t parity = 0, prev_parity = 0;
    int buf = 0, item = 0;

    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
        const __nv_bfloat16 *xp[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t)
            xp[t] = x + (size_t)min(r + 8 * t, M - 1) * K + c * 32 + warp * 128;

        for (int chunk = 0; chunk < chunks; ++chunk, ++item) {
            if (!mbar_wait(&full_bar[slot], parity)) {
                atomicExch(status, (int)AB2_ERR_TIMEOUT);
                return;
            }
            // Warps beyond the last group of a short final stage run on block 0 of
            // the stage with their scales forced to zero (no divergent branch).
            const bool active = chunk * W4_GROUPS_PER_STAGE + warp < G;
            const uint32_t *blk = &ring[slot][(active ? warp : 0) * W4_BLOCK_WORDS];
            const uint4 wa = *reinterpret_cast<const uint4 *>(blk + lane_words);
            const uint4 wb = *reinterpret_cast<const uint4 *>(blk + lane_words + 128);
            uint32_t pa = blk[256 + r], pb = blk[256 + r + 8];
            if (!active) { pa &= 0xffff0000u; pb &= 0xffff0000u; }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[slot]);
            // Refill the slot released one step ago (so this thread does not wait
            // on the slowest warp of the current step).
            if (producer && item >= 1 && p_item < items) {
                if (!mbar_wait(&empty_bar[prev_slot], prev_parity)) {
                    atomicExch(status, (int)AB2_ERR_TIMEOUT);
                    return;
                }
                issue_next();
            }
            prev_slot = slot;
            prev_parity = parity;
            if (++slot == stages) { slot = 0; parity ^= 1; }

            uint4 xw[NT][4];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const __nv_bfloat16 *src = active ? xp[t] : xp[t] - warp * 128;
#pragma unroll
                for (int wi = 0; wi < 4; ++wi)
                    xw[t][wi] = *reinterpret_cast<const uint4 *>(src + wi * 8);
                xp[t] += W4_GROUPS_PER_STAGE * 128;
            }

            const float sa = __uint_as_float(pa << 16), sb = __uint_as_float(pb << 16);
            const uint32_t nza = __byte_perm(pa, pa, 0x3232), nzb = __byte_perm(pb, pb, 0x3232);
            // two independent accumulation chains: codes, and the zero point
            float d[NT][4], dz[NT][4];
            const uint32_t words_a[4] = {wa.x, wa.y, wa.z, wa.w};
            const uint32_t words_b[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                uint32_t a[8];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    a[2 * jj] = w4_pair_bf16(words_a[wi], jj, k_mask, k_magic);
                    a[2 * jj + 1] = w4_pair_bf16(words_b[wi], jj, k_mask, k_magic);
                }
                if (NT == 2) {
                    // 9..16 tokens: the tensor pipe is the scarce one, so the zero
                    // point is removed by an exact bf16x2 add: (128 + q) - (128 + z)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        a[2 * jj] = bf16x2_add(a[2 * jj], nza);
                        a[2 * jj + 1] = bf16x2_add(a[2 * jj + 1], nzb);
                    }
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    // two independent accumulation chains (even / odd k-steps, or
                    // codes / zero point when the zero point rides the tensor pipe)
                    if (wi == 0) {
                        mma_bf16_16816_init(d[t], a[0], a[1], a[2], a[3], xw[t][wi].x, xw[t][wi].y);
                        if (NT == 1)
                            mma_bf16_16816_init(dz[t], nza, nzb, nza, nzb, xw[t][wi].x, xw[t][wi].y);
                        else
                            mma_bf16_16816_init(dz[t], a[4], a[5], a[6], a[7], xw[t][wi].z, xw[t][wi].w);
                    } else {
                        mma_bf16_16816(d[t], a[0], a[1], a[2], a[3], xw[t][wi].x, xw[t][wi].y);
                        if (NT == 1)
                            mma_bf16_16816(dz[t], nza, nzb, nza, nzb, xw[t][wi].x, xw[t][wi].y);
                        else
                            mma_bf16_16816(dz[t], a[4], a[5], a[6], a[7], xw[t][wi].z, xw[t][wi].w);
                    }
                    if (NT == 1) {
                        mma_bf16_16816(d[t], a[4], a[5], a[6], a[7], xw[t][wi].z, xw[t][wi].w);
                        mma_bf16_16816(dz[t], nza, nzb, nza, nzb, xw[t][wi].z, xw[t][wi].w);
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                acc[t][0] = fmaf(sa, d[t][0] + dz[t][0], acc[t][0]);
                acc[t][1] = fmaf(sa, d[t][1] + dz[t][1], acc[t][1]);
                acc[t][2] = fmaf(sb, d[t][2] + dz[t][2], acc[t][2]);
                acc[t][3] = fmaf(sb, d[t][3] + dz[t][3], acc[t][3]);
            }
        }

        // End of the tile: publish this warp's partials; the last warp to arrive
        // adds the 8 K-slices in fixed order and stores.
        // D fragment: [0],[1] -> (row r, tokens 2c, 2c+1); [2],[3] -> (row r+8, same)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            red[buf][warp][r][8 * t + 2 * c] = acc[t][0];
            red[buf][warp][r][8 * t + 2 * c + 1] = acc[t][1];
            red[buf][warp][r + 8][8 * t + 2 * c] = acc[t][2];
            red[buf][warp][r + 8][8 * t + 2 * c + 1] = acc[t][3];
        }
        __threadfence_block();
        __syncwarp();
        int arrived = 0;
        if (lane == 0) arrived = atomicAdd(&arrivals[buf], 1);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == 7) {
            __threadfence_block();
            const int row0 = tile * 16;
            for (int idx = lane; idx < 16 * 8 * NT; idx += 32) {
                const int tok = idx >> 4, row = idx & 15;
                if (EPI == W4_EPI_SWIGLU) {
                    // rows 0..7 of the tile are gate rows, rows 8..15 the matching up rows
                    const int half_n = N >> 1, col = tile * 8 + row;
                    if (row < 8 && tok < M && col < half_n) {
                        float g = 0.f, u = 0.f;
#pragma unroll
                        for (int w = 0; w < 8; ++w) { g += red[buf][w][row][tok]; u += red[buf][w][row + 8][tok]; }
                        // the reference rounds gate and up to the activation type first
                        g = __bfloat162float(__float2bfloat16_rn(g));
                        u = __bfloat162float(__float2bfloat16_rn(u));
                        y[(size_t)tok * half_n + col] = __float2bfloat16_rn(swiglu_value(g, u));
                    }
                } else if (tok < M && row0 + row < N) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < 8; ++w) v += red[buf][w][row][tok];
                    const size_t o = (size_t)tok * N + row0 + row;
                    if (EPI == W4_EPI_F32) {  // unrounded partial sum of a row-parallel shard
                        reinterpret_cast<float *>(y)[o] = v;
                    } else {
                        if (EPI == W4_EPI_ADD)  // residual + bf16(projection), as residual + x does
                            v = __bfloat162float(resid[o]) + __bfloat162float(__float2bfloat16_rn(v));
                        y[o] = __float2bfloat16_rn(v);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) arrivals[buf] = 0;
        }
        buf ^= 1;
    }
}

}  // namespace ab2
