// W4A16 (group 128, bf16 activations) decode GEMV for 1..16 tokens: every warp
// streams its own contiguous run of weight blocks.
//
// The weight is a sequence of 1088-byte blocks ordered [16-row tile][group]
// (w4a16_layout.cuh).  The sequence is cut into one contiguous range per warp
// of the grid, equal to within one block, so every SM streams the same number
// of bytes whatever N and K are.  A warp owns a private ring of shared-memory
// stages that lane 0 fills with bulk asynchronous copies (cp.async.bulk,
// completion on an mbarrier per stage): there is no CTA-wide barrier, no shared
// producer and no cross-warp reduction in shared memory.
//
// Arithmetic per block is that of gemv_w4a16_mma.cuh: nibbles become bf16 with
// one shift and one LOP3 per pair (0x4300 | q == 128 + q exactly) and feed
// mma.sync.m16n8k16 (bf16 x bf16 -> f32) with the 16 weight rows as A and up to
// 8 tokens as B; the zero point leaves by an exact bf16x2 add on the A registers;
// the bf16 scale is applied per group in f32.
//
// A tile whose groups all lie inside one warp's range is finished by that warp.
// A tile cut by a range boundary is finished by whichever of its contributors
// arrives last: every contributor writes its f32 partial sums to its own slot
// of a global scratch buffer, bumps the tile's counter, and the last one adds
// the slots in contributor order (so the sum does not depend on arrival order),
// runs the epilogue and resets the counter.  Nobody waits on anybody.
//
// Every mbarrier wait is bounded; a wait that runs out records AB2_ERR_TIMEOUT
// in the status word and the warp returns.
#pragma once

#include "gemv_w4a16_mma.cuh"
#include "tp.cuh"

namespace ab2 {

constexpr int W4W_STAGES = 5;
constexpr int W4W_WARPS = 8;
// f32 partial sums of one tile as one warp holds them: 32 lanes x 4 x NT (NT <= 2)
constexpr int W4W_SLOT_FLOATS = 32 * 8;

template <int NT, int EPI>
__device__ __forceinline__ void w4w_store_tile(const float (&acc)[NT][4], int tile, int r, int c,
                                               __nv_bfloat16 *y, const __nv_bfloat16 *resid, int N,
                                               int M) {
    // peer exchange: buffer (epoch + 1) & 1, slot of this rank, in every rank's inbox
    const ab2_tp_peer_desc *peers = nullptr;
    size_t peer_off = 0;
    int peer_world = 0;
    uint32_t exchange = 0;
    if (EPI == W4_EPI_F32_PEER) {
        peers = reinterpret_cast<const ab2_tp_peer_desc *>(y);
        peer_world = peers->world;
        exchange = *peers->epoch + 1;
        peer_off = ((size_t)(exchange & 1u) * peer_world + peers->rank) * peers->max_elems;
    }
    // The residual may alias the output (the stream is updated in place), so loads left between
    // the stores could not be moved ahead of them: all residual values are read first.
    float rv[NT][4];
    if (EPI == W4_EPI_ADD) {
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int tok = 8 * t + 2 * c + (q & 1), row = tile * 16 + r + 8 * (q >> 1);
                rv[t][q] = (tok < M && row < N) ? __bfloat162float(resid[(size_t)tok * N + row]) : 0.f;
            }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int tok = 8 * t + 2 * c + i;
            if (tok >= M) continue;
            if (EPI == W4_EPI_SWIGLU) {
                // rows 0..7 of the tile are gate rows, rows 8..15 the matching up rows
                const int half_n = N >> 1, col = tile * 8 + r;
                if (col < half_n) {
                    // the reference rounds gate and up to the activation type first
                    const float g = __bfloat162float(__float2bfloat16_rn(acc[t][i]));
                    const float u = __bfloat162float(__float2bfloat16_rn(acc[t][2 + i]));
                    y[(size_t)tok * half_n + col] = __float2bfloat16_rn(swiglu_value(g, u));
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = tile * 16 + r + 8 * h;
                    if (row >= N) continue;
                    float v = acc[t][2 * h + i];
                    const size_t o = (size_t)tok * N + row;
                    if (EPI == W4_EPI_F32) {  // unrounded partial sum of a row-parallel shard
                        reinterpret_cast<float *>(y)[o] = v;
                    } else if (EPI == W4_EPI_F32_PEER) {  // the same, stored over NVLink with every rank
                        const unsigned long long word = tp_ll_pack(v, exchange);  // the sum and its arrival signal in one store
                        for (int p = 0; p < peer_world; ++p) tp_ll_store(peers->inbox[p] + peer_off + o, word);
                    } else {
                        if (EPI == W4_EPI_ADD)  // residual + bf16(projection), as residual + x does
                            v = rv[t][2 * h + i] + __bfloat162float(__float2bfloat16_rn(v));
                        y[o] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
}

// Bounded wait on an mbarrier phase (two seconds of wall clock).  Returns 0 when the
// limit ran out.  The first probe is kept out of the loop so the common case costs
// one instruction.
__device__ __forceinline__ uint32_t mbar_wait_addr(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return 1u;
    unsigned long long t0 = 0;  // read only once a wait has lasted: the timer is a slow register
    for (int spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return 1u;
        if ((spin & 31) == 31) {
            const unsigned long long now = mbar_wall_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) return 0u;
        }
    }
}

// When `go` is non-zero: arm `bar` for `bytes` and start the bulk copy of one
// block into shared memory.  Predicated, so a single lane can issue it without a
// divergent branch.
__device__ __forceinline__ void bulk_g2s_if(uint32_t go, uint32_t dst, const void *src, uint32_t bytes,
                                            uint32_t bar) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.u32 p, %0, 0;\n"
        " @p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%4], %3;\n"
        " @p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%1], [%2], %3, [%4];\n"
        "}\n" ::"r"(go),
        "r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

// partials: [gridDim.x * 8 warps][2][W4W_SLOT_FLOATS] floats; counters: one int
// per 16-row tile, zero on entry and on exit.
//
template <int NT, int EPI>
__global__ void __launch_bounds__(256, 3)
gemv_w4a16_warp_kernel(const uint32_t *__restrict__ wt, const __nv_bfloat16 *__restrict__ x,
                       __nv_bfloat16 *y, const __nv_bfloat16 *resid, int N, int K, int M,
                       float *partials, int *counters, int *status) {
    __shared__ alignas(128) uint32_t ring[W4W_WARPS][W4W_STAGES][W4_BLOCK_WORDS];
    __shared__ alignas(8) uint64_t full_bar[W4W_WARPS][W4W_STAGES];
    constexpr uint32_t BLOCK_BYTES = W4_BLOCK_WORDS * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int G = K >> 7, tiles = (N + 15) >> 4;
    const int total = tiles * G;
    const int nwarps = (int)gridDim.x * W4W_WARPS, wid = (int)blockIdx.x * W4W_WARPS + warp;
    // ranges: the first `rem` warps take base + 1 blocks, the others base
    const int base = total / nwarps, rem = total - base * nwarps;
    const int b0 = wid * base + min(wid, rem);
    const int nblk = base + (wid < rem ? 1 : 0);
    const int b1 = b0 + nblk;

    const uint32_t ring0 = smem_addr(&ring[warp][0][0]), bar0 = smem_addr(&full_bar[warp][0]);
    const uint32_t lane0 = lane == 0 ? 1u : 0u;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < W4W_STAGES; ++s) mbar_init(&full_bar[warp][s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncwarp();
    // the weights are constant: the first stages are in flight before the
    // preceding kernel has finished
    const uint32_t *src = wt + (size_t)b0 * W4_BLOCK_WORDS;  // next block to fetch
    int to_fetch = nblk;
#pragma unroll
    for (int j = 0; j < W4W_STAGES; ++j) {
        bulk_g2s_if(lane0 & (to_fetch > 0 ? 1u : 0u), ring0 + j * BLOCK_BYTES, src, BLOCK_BYTES, bar0 + j * 8);
        src += W4_BLOCK_WORDS;
        --to_fetch;
    }

    // activations (and the residual) come from the preceding kernel
    pdl_wait();
    pdl_launch_dependents();
    if (nblk == 0) return;

    const uint32_t hidden_zero = (uint32_t)K & 1u;  // K is a multiple of 128
    // Opaque register copies of the two constants of the nibble extraction.
    uint32_t k_mask = 0x000F000Fu, k_magic = 0x43004300u;
    asm volatile("" : "+r"(k_mask), "+r"(k_magic));

    const uint32_t code_off = (r * 16 + c * 4) * 4;  // this thread's 4 words of row r in a block
    const uint32_t param_off = (256 + r) * 4;
    const __nv_bfloat16 *xrow[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) xrow[t] = x + (size_t)min(r + 8 * t, M - 1) * K + c * 32;

    int tile = b0 / G, g = b0 - tile * G;
    uint32_t cur = ring0, bar = bar0, parity = 0;
    const uint32_t ring_end = ring0 + W4W_STAGES * BLOCK_BYTES;

    for (int b = b0; b < b1;) {
        const int n = min(G - g, b1 - b);  // blocks of this tile inside the range
        const bool whole = n == G;
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
        const __nv_bfloat16 *xp[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) xp[t] = xrow[t] + g * 128;

        for (int it = 0; it < n; ++it) {
            if (!mbar_wait_addr(bar, parity)) {
                if (lane == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
                return;
            }
            const uint4 wa = lds128(cur + code_off);
            const uint4 wb = lds128(cur + code_off + 512);
            const uint32_t pa = lds32(cur + param_off), pb = lds32(cur + param_off + 32);
            uint4 xw[NT][4];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
#pragma unroll
                for (int wi = 0; wi < 4; ++wi)
                    xw[t][wi] = *reinterpret_cast<const uint4 *>(xp[t] + wi * 8);
                xp[t] += 128;
            }

            const float sa = __uint_as_float(pa << 16), sb = __uint_as_float(pb << 16);
            const uint32_t nza = __byte_perm(pa, pa, 0x3232), nzb = __byte_perm(pb, pb, 0x3232);
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
                // the zero point leaves by an exact bf16x2 add: (128 + q) - (128 + z)
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    a[2 * jj] = bf16x2_add(a[2 * jj], nza);
                    a[2 * jj + 1] = bf16x2_add(a[2 * jj + 1], nzb);
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    // two independent accumulation chains (even / odd k-steps)
                    if (wi == 0) {
                        mma_bf16_16816_init(d[t], a[0], a[1], a[2], a[3], xw[t][wi].x, xw[t][wi].y);
                        mma_bf16_16816_init(dz[t], a[4], a[5], a[6], a[7], xw[t][wi].z, xw[t][wi].w);
                    } else {
                        mma_bf16_16816(d[t], a[0], a[1], a[2], a[3], xw[t][wi].x, xw[t][wi].y);
                        mma_bf16_16816(dz[t], a[4], a[5], a[6], a[7], xw[t][wi].z, xw[t][wi].w);
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

            // Refill this stage with the block W4W_STAGES ahead.  The copy must not be issued while a
            // load of the stage is still under way (a shared-memory load can wait behind other traffic
            // for longer than a bulk copy out of L2 takes to land): its source address takes in the
            // running sums, which every load of the stage has fed, masked with a zero the compiler
            // cannot see.
            uint32_t held = 0;
#pragma unroll
            for (int t = 0; t < NT; ++t) held ^= __float_as_uint(acc[t][0]) ^ __float_as_uint(acc[t][2]);
            __syncwarp();
            bulk_g2s_if(lane0 & (to_fetch > 0 ? 1u : 0u), cur, src + (held & hidden_zero), BLOCK_BYTES, bar);
            src += W4_BLOCK_WORDS;
            --to_fetch;
            cur += BLOCK_BYTES;
            bar += 8;
            if (cur == ring_end) { cur = ring0; bar = bar0; parity ^= 1; }
        }
        b += n;

        // ---- end of this warp's share of the tile ---------------------------
        if (whole) {
            w4w_store_tile<NT, EPI>(acc, tile, r, c, y, resid, N, M);
        } else {
            // contributors of the tile: the warps whose ranges meet [tile*G, tile*G + G)
            const int cut = rem * (base + 1);
            const int first_b = tile * G, last_b = first_b + G - 1;
            const int w_first = first_b < cut ? first_b / (base + 1) : rem + (first_b - cut) / base;
            const int w_last = last_b < cut ? last_b / (base + 1) : rem + (last_b - cut) / base;
            // a warp has at most two cut tiles: the one its range starts inside (slot
            // 0) and the one its range ends inside (slot 1)
            float *mine = partials + ((size_t)wid * 2 + (wid == w_first ? 1 : 0)) * W4W_SLOT_FLOATS +
                          lane * 4 * NT;
#pragma unroll
            for (int t = 0; t < NT; ++t)
                *reinterpret_cast<float4 *>(mine + 4 * t) =
                    make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
            __threadfence();
            __syncwarp();
            int arrived = 0;
            if (lane == 0) arrived = atomicAdd(&counters[tile], 1);
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            if (arrived == w_last - w_first) {
                __threadfence();
                float sum[NT][4];
#pragma unroll
                for (int t = 0; t < NT; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sum[t][i] = 0.f;
                for (int w = w_first; w <= w_last; ++w) {
                    const float *p = partials + ((size_t)w * 2 + (w == w_first ? 1 : 0)) * W4W_SLOT_FLOATS +
                                     lane * 4 * NT;
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const float4 v = __ldcg(reinterpret_cast<const float4 *>(p + 4 * t));
                        sum[t][0] += v.x; sum[t][1] += v.y; sum[t][2] += v.z; sum[t][3] += v.w;
                    }
                }
                w4w_store_tile<NT, EPI>(sum, tile, r, c, y, resid, N, M);
                if (lane == 0) counters[tile] = 0;
            }
        }
        g = 0;
        ++tile;
    }
}

}  // namespace ab2
