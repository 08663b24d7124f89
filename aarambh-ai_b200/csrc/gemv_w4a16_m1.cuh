// W4A16 (group 128) decode GEMV for ONE token: the warp-streaming kernel of
// gemv_w4a16_warp.cuh with the activation side prepared once per CTA so that
// the per-weight work is one logic op per pair of weights.
//
// Prologue (after the preceding kernel has finished): the CTA reads the K bf16
// activations, finds their largest magnitude, and writes them to shared memory
// as f16 scaled by a power of two 2^e that puts the largest value just below
// 2^15 (exact: bf16 has fewer significand bits than f16, and values more than
// 2^25 below the largest one are the only ones that can lose bits).  Elements
// whose position in their 8-element word is 2, 3, 6 or 7 are scaled by a
// further 2^-4.  Per group of 128 it also keeps P = sum of the stored values
// and T = 2^e * sum of the activations, both in f32.
//
// Main loop: a code word holds 8 nibbles; (w & 0x000F000F) | 0x64006400 is the
// f16 pair (1024 + q, 1024 + q') of two of them and (w & 0x00F000F0) |
// 0x64006400 is (1024 + 16 q, 1024 + 16 q') of two others, exactly, with no
// shift; one shift by 8 gives the other four.  The factor 16 meets the 2^-4 of
// the activation, so the f16 MMA (m16n8k16, f32 accumulate) returns
//     d = 1024 P + 2^e sum_k x_k q_k
// and the group's contribution to the output is  s (d - 1024 P - z T) / 2^e.
// Only lanes 0..3 hold activations (token 0 is column 0 of the B operand); the
// other columns of the MMA are zero and ignored.
//
// Ranges, rings, bounded waits and the finishing of cut tiles are those of
// gemv_w4a16_warp.cuh.
#pragma once

#include "gemv_w4a16_warp.cuh"

namespace ab2 {

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816_init(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                   uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// (word & mask) | magic as one three-input logic op (all operands in registers).
__device__ __forceinline__ uint32_t and_or(uint32_t word, uint32_t mask, uint32_t magic) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(word), "r"(mask), "r"(magic));
    return d;
}

// 16 bytes from shared memory into v when `go` is non-zero (v keeps its value otherwise).
__device__ __forceinline__ void lds128_if(uint32_t go, uint32_t addr, uint4 &v) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.u32 p, %4, 0;\n"
        " @p ld.shared.v4.u32 {%0,%1,%2,%3}, [%5];\n"
        "}\n"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(go), "r"(addr));
}

// Dynamic shared memory: rings [8][STAGES][2 x 1088 B], activations [K] f16, group
// constants [K/128] float2, barriers [8][STAGES].
// A bulk copy costs its issuing warp (and the SM's copy engine) about 50 cycles whatever its size,
// so a ring stage holds two consecutive blocks fetched by one copy.
constexpr int W4M1_COPY_BLOCKS = 2;
template <int STAGES>
__host__ __device__ constexpr size_t w4m1_smem_bytes(int K) {
    return (size_t)W4W_WARPS * STAGES * W4M1_COPY_BLOCKS * W4_BLOCK_WORDS * 4 + (size_t)K * 2 + (size_t)(K >> 7) * 8 +
           (size_t)W4W_WARPS * STAGES * 8;
}

constexpr int W4M1_LOCAL_TILES = 64;  // cut tiles a CTA can finish through shared memory

// NORM: the activations are RMS-normalised first (x * rsqrt(mean(x^2) + eps) *
// norm_w, rounded to bf16 as the stand-alone kernel does), so the normalisation
// costs no launch of its own.  NV = vectors of 8 activations a thread keeps in
// registers between the two passes of the prologue (K <= 2048 * NV).
//
// PEER_IN (tensor parallel, with NORM): the input is the residual stream plus
// the sum over ranks of the partial sums arriving in this rank's inbox of the
// peer exchange (tp.cuh).  Every inbox word carries the number of its exchange,
// so each thread simply waits (bounded) until the words it needs show the
// current number, adds the partials in rank order and rounds as the stand-alone
// reduce does; CTA 0 also writes the new residual stream to `x_out` (not `x`:
// other CTAs still read it), and the CTA that finishes its prologue last
// advances the exchange count.
template <int EPI, int STAGES, int NV, bool NORM, bool PEER_IN = false>
__global__ void __launch_bounds__(256, 3)
gemv_w4a16_m1_kernel(const uint32_t *__restrict__ wt, const __nv_bfloat16 *__restrict__ x,
                     const float *__restrict__ norm_w, float eps, __nv_bfloat16 *y,
                     const __nv_bfloat16 *resid, int N, int K, float *partials, int *counters,
                     int *status, const ab2_tp_peer_desc *peers = nullptr, __nv_bfloat16 *x_out = nullptr) {
    static_assert(!PEER_IN || NORM, "the peer exchange is consumed by the normalising kernels");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float2 warp_part[W4W_WARPS];                 // (sum of squares, largest magnitude)
    __shared__ float2 cta_part[W4W_WARPS][2][8];            // partial sums of cut tiles, rows (r, r + 8)
    __shared__ int cta_cnt[W4M1_LOCAL_TILES];
    constexpr uint32_t BLOCK_BYTES = W4_BLOCK_WORDS * 4, STAGE_BYTES = W4M1_COPY_BLOCKS * BLOCK_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int G = K >> 7, tiles = (N + 15) >> 4;
    const int total = tiles * G;
    const int nwarps = (int)gridDim.x * W4W_WARPS, wid = (int)blockIdx.x * W4W_WARPS + warp;
    const int base = total / nwarps, rem = total - base * nwarps;
    const int b0 = wid * base + min(wid, rem);
    const int nblk = base + (wid < rem ? 1 : 0);
    const int b1 = b0 + nblk;

    const uint32_t smem0 = smem_addr(smem_raw);
    const uint32_t xs0 = smem0 + W4W_WARPS * STAGES * STAGE_BYTES;  // f16 activations
    const uint32_t gs0 = xs0 + K * 2;                               // (C2, T) per group
    const uint32_t bars0 = gs0 + G * 8;
    const uint32_t ring0 = smem0 + warp * STAGES * STAGE_BYTES, bar0 = bars0 + warp * STAGES * 8;
    const uint32_t lane0 = lane == 0 ? 1u : 0u;
    if (threadIdx.x < W4M1_LOCAL_TILES) cta_cnt[threadIdx.x] = 0;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar0 + s * 8));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncwarp();
    // the weights are constant: the first stages are in flight before the
    // preceding kernel has finished
    const uint32_t *src = wt + (size_t)b0 * W4_BLOCK_WORDS;  // next block to fetch
    int to_fetch = nblk;
#pragma unroll
    for (int j = 0; j < STAGES; ++j) {
        bulk_g2s_if(lane0 & (to_fetch > 0 ? 1u : 0u), ring0 + j * STAGE_BYTES, src,
                    (uint32_t)min(to_fetch, W4M1_COPY_BLOCKS) * BLOCK_BYTES, bar0 + j * 8);
        src += W4M1_COPY_BLOCKS * W4_BLOCK_WORDS;
        to_fetch -= W4M1_COPY_BLOCKS;
    }

    // the norm weights are constant too, and a step's weight stream has long evicted them from L2:
    // request them now so that the prologue does not wait for DRAM
    if (NORM) {
#pragma unroll
        for (int it = 0; it < NV; ++it) {
            const int i = threadIdx.x + it * 256;
            if (i < (K >> 3)) asm volatile("prefetch.global.L1 [%0];\n" ::"l"(norm_w + 8 * i));
        }
    }

    // activations (and the residual) come from the preceding kernel
    pdl_wait();
    pdl_launch_dependents();

    // ---- tensor parallel: the partial sums of every rank wait in this rank's inbox ----
    const unsigned long long *box = nullptr;
    size_t box_stride = 0;
    int box_world = 0;
    uint32_t exchange = 0;
    unsigned long long wait_limit = 0;
    __shared__ int peer_failed;
    if (PEER_IN) {
        const ab2_tp_peer_desc d = *peers;
        exchange = *d.epoch + 1;
        if (threadIdx.x == 0) peer_failed = 0;
        box = d.inbox[d.rank] + (size_t)(exchange & 1u) * d.world * d.max_elems;
        box_stride = d.max_elems;
        box_world = d.world;
        wait_limit = d.wait_limit_ns;
        __syncthreads();
    }

    // ---- prologue, pass 1: sum of squares and largest magnitude ---------------
    const uint4 *x4 = reinterpret_cast<const uint4 *>(x);
    const int nvec = K >> 3;
    uint4 xv[NV];
    float ss = 0.f, amax = 0.f;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
        const int i = threadIdx.x + it * 256;
        xv[it] = i < nvec ? __ldcg(x4 + i) : make_uint4(0u, 0u, 0u, 0u);
        if (PEER_IN && i < nvec) {
            // residual + bf16(sum over ranks), element by element as the stand-alone reduce does
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int rk = 0; rk < box_world; ++rk) {
                // every word carries its exchange number: wait (bounded) until this thread's eight have arrived
                float pv[8];
                if (!tp_ll_wait8(box + (size_t)rk * box_stride + 8 * (size_t)i, exchange, wait_limit, pv)) {
                    peer_failed = 1;
#pragma unroll
                    for (int j = 0; j < 8; ++j) pv[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[j] += pv[j];
            }
            uint32_t w[4] = {xv[it].x, xv[it].y, xv[it].z, xv[it].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float f0 = __uint_as_float(w[j] << 16) + __bfloat162float(__float2bfloat16_rn(sum[2 * j]));
                const float f1 = __uint_as_float(w[j] & 0xffff0000u) + __bfloat162float(__float2bfloat16_rn(sum[2 * j + 1]));
                w[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f0)) |
                       ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f1)) << 16);
            }
            xv[it] = make_uint4(w[0], w[1], w[2], w[3]);
            if (blockIdx.x == 0) reinterpret_cast<uint4 *>(x_out)[i] = xv[it];
        }
        const uint32_t w[4] = {xv[it].x, xv[it].y, xv[it].z, xv[it].w};
        float nw[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
        if (NORM && i < nvec) {
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i);
            const float4 w1 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i + 1);
            nw[0] = w0.x; nw[1] = w0.y; nw[2] = w0.z; nw[3] = w0.w;
            nw[4] = w1.x; nw[5] = w1.y; nw[6] = w1.z; nw[7] = w1.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xffff0000u);
            if (NORM) {
                ss = fmaf(f0, f0, ss);
                ss = fmaf(f1, f1, ss);
            }
            amax = fmaxf(amax, fmaxf(fabsf(f0 * nw[2 * j]), fabsf(f1 * nw[2 * j + 1])));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
    if (lane == 0) warp_part[warp] = make_float2(ss, amax);
    __syncthreads();
    if (PEER_IN && peer_failed) {
        // a peer's sums did not arrive within the limit: record it and stop (the exchange count is
        // left as it was; ab2_tp_peer_reset puts the ranks back in step)
        if (threadIdx.x == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
        return;
    }
    {
        const float2 t = lane < W4W_WARPS ? warp_part[lane] : make_float2(0.f, 0.f);
        ss = t.x;
        amax = t.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        }
    }
    float inv = 1.f;
    if (NORM) {
        inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
        amax = amax * inv * 1.0078125f;  // bound on |bf16(x inv w)|
    }
    // 2^e puts the largest magnitude in [2^14, 2^15); e is kept where 2^e, 2^(e-4)
    // and 2^-e are normal f32 (an all-zero or non-finite input takes the clamp)
    int e = 141 - (int)((__float_as_uint(amax) >> 23) & 0xffu);
    e = max(-100, min(100, e));
    const float sc_lo = __uint_as_float((uint32_t)(e + 127) << 23);
    const float sc_hi = __uint_as_float((uint32_t)(e - 4 + 127) << 23);
    const float unscale = __uint_as_float((uint32_t)(127 - e) << 23);

    // ---- prologue, pass 2: f16 copy and group sums ----------------------------
#pragma unroll
    for (int it = 0; it < NV; ++it) {
        const int i = threadIdx.x + it * 256;
        if (i < nvec) {  // uniform over each aligned group of 16 lanes (nvec is a multiple of 16)
            const uint32_t w[4] = {xv[it].x, xv[it].y, xv[it].z, xv[it].w};
            float nw[8];
            if (NORM) {
                const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i);
                const float4 w1 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i + 1);
                nw[0] = w0.x; nw[1] = w0.y; nw[2] = w0.z; nw[3] = w0.w;
                nw[4] = w1.x; nw[5] = w1.y; nw[6] = w1.z; nw[7] = w1.w;
            }
            uint32_t h[4];
            float p = 0.f, sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xffff0000u);
                if (NORM) {
                    f0 = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__fmul_rn(f0, inv), nw[2 * j])));
                    f1 = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__fmul_rn(f1, inv), nw[2 * j + 1])));
                }
                const float sc = (j & 1) ? sc_hi : sc_lo;  // words 1 and 3 hold elements 2,3 and 6,7
                const __half2 hh = __floats2half2_rn(f0 * sc, f1 * sc);
                h[j] = *reinterpret_cast<const uint32_t *>(&hh);
                const float2 back = __half22float2(hh);
                p += back.x + back.y;
                sum += f0 + f1;
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(xs0 + i * 16), "r"(h[0]), "r"(h[1]),
                         "r"(h[2]), "r"(h[3])
                         : "memory");
            // a group is 16 consecutive vectors = 16 consecutive lanes
            const uint32_t half_mask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                p += __shfl_xor_sync(half_mask, p, o);
                sum += __shfl_xor_sync(half_mask, sum, o);
            }
            if ((lane & 15) == 0) {
                const float T = sum * sc_lo;
                const float C2 = 1024.f * p - 128.f * T;
                asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(gs0 + (i >> 4) * 8), "f"(C2), "f"(T)
                             : "memory");
            }
        }
    }
    __syncthreads();
    if (PEER_IN && threadIdx.x == 0) {
        // every CTA has read the exchange count and its inbox: the last one closes the exchange
        const ab2_tp_peer_desc d = *peers;
        if (atomicAdd(d.done, 1u) == gridDim.x - 1) {
            *d.done = 0;
            __threadfence();
            *d.epoch = exchange;
        }
    }
    if (nblk == 0) return;

    const uint32_t hidden_zero = (uint32_t)K & 1u;  // K is a multiple of 128
    // Opaque register copies of the constants of the nibble extraction.
    uint32_t k_lo = 0x000F000Fu, k_hi = 0x00F000F0u, k_magic = 0x64006400u;
    asm volatile("" : "+r"(k_lo), "+r"(k_hi), "+r"(k_magic));

    const uint32_t code_off = (r * 16 + c * 4) * 4;  // this thread's 4 words of row r in a block
    const uint32_t param_off = (256 + r) * 4;
    const uint32_t has_x = r == 0 ? 1u : 0u;
    const uint32_t xlane = xs0 + c * 64;
    // first tile this CTA touches (warp 0's range starts there)
    const int cta_w0 = (int)blockIdx.x * W4W_WARPS;
    const int cta_tile0 = (cta_w0 * base + min(cta_w0, rem)) / G;

    int tile = b0 / G, g = b0 - tile * G;
    // cur: the stage of the next block; second: its first block has been consumed already
    uint32_t cur = ring0, bar = bar0, parity = 0, second = 0;
    const uint32_t ring_end = ring0 + STAGES * STAGE_BYTES;
    uint4 xw[4];
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) xw[wi] = make_uint4(0u, 0u, 0u, 0u);

    for (int b = b0; b < b1;) {
        const int n = min(G - g, b1 - b);  // blocks of this tile inside the range
        const bool whole = n == G;
        float acc_a = 0.f, acc_b = 0.f;  // rows r and r + 8 of the tile, token 0 (lanes c == 0)
        uint32_t xaddr = xlane + g * 256, gaddr = gs0 + g * 8;

        // one block at `addr` of the ring: unpack, 8 MMAs, the group's scale and zero point
        auto block = [&](uint32_t addr) {
            const uint4 wa = lds128(addr + code_off);
            const uint4 wb = lds128(addr + code_off + 512);
            const uint32_t pa = lds32(addr + param_off), pb = lds32(addr + param_off + 32);
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) lds128_if(has_x, xaddr + wi * 16, xw[wi]);
            float C2, T;
            asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(C2), "=f"(T) : "r"(gaddr));
            xaddr += 256;
            gaddr += 8;

            float d[4], d2[4];
            const uint32_t words_a[4] = {wa.x, wa.y, wa.z, wa.w};
            const uint32_t words_b[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t ua = words_a[wi], ub = words_b[wi];
                const uint32_t ua8 = ua >> 8, ub8 = ub >> 8;
                // pair j of a word = elements (2j, 2j+1); even j as 1024 + q, odd j as 1024 + 16 q
                const uint32_t a0 = and_or(ua, k_lo, k_magic), a1 = and_or(ub, k_lo, k_magic);
                const uint32_t a2 = and_or(ua, k_hi, k_magic), a3 = and_or(ub, k_hi, k_magic);
                const uint32_t a4 = and_or(ua8, k_lo, k_magic), a5 = and_or(ub8, k_lo, k_magic);
                const uint32_t a6 = and_or(ua8, k_hi, k_magic), a7 = and_or(ub8, k_hi, k_magic);
                if (wi == 0) {
                    mma_f16_16816_init(d, a0, a1, a2, a3, xw[wi].x, xw[wi].y);
                    mma_f16_16816_init(d2, a4, a5, a6, a7, xw[wi].z, xw[wi].w);
                } else {
                    mma_f16_16816(d, a0, a1, a2, a3, xw[wi].x, xw[wi].y);
                    mma_f16_16816(d2, a4, a5, a6, a7, xw[wi].z, xw[wi].w);
                }
            }
            // s (d - 1024 P - z T) with -(128 + z) taken from the parameter word
            const float sa = __uint_as_float(pa << 16), sb = __uint_as_float(pb << 16);
            const float nza = __uint_as_float(pa & 0xffff0000u), nzb = __uint_as_float(pb & 0xffff0000u);
            acc_a = fmaf(sa, (d[0] + d2[0]) - fmaf(-nza, T, C2), acc_a);
            acc_b = fmaf(sb, (d[2] + d2[2]) - fmaf(-nzb, T, C2), acc_b);
        };
        // The stage `cur` points into has been consumed: refill it with the two blocks STAGES stages
        // ahead (every lane's loads of it were issued above and have been consumed) and move on.
        auto next_stage = [&]() {
            // The copy must not be issued while a load of the stage is still under way (a shared-memory load
            // can wait behind other traffic for longer than a bulk copy out of L2 takes to land): its source
            // address takes in the running sums, which every load of the stage has fed, masked with a zero the
            // compiler cannot see.
            const uint32_t held = (__float_as_uint(acc_a) ^ __float_as_uint(acc_b)) & hidden_zero;
            __syncwarp();
            bulk_g2s_if(lane0 & (to_fetch > 0 ? 1u : 0u), cur, src + held, (uint32_t)min(to_fetch, W4M1_COPY_BLOCKS) * BLOCK_BYTES, bar);
            src += W4M1_COPY_BLOCKS * W4_BLOCK_WORDS;
            to_fetch -= W4M1_COPY_BLOCKS;
            cur += STAGE_BYTES;
            bar += 8;
            if (cur == ring_end) { cur = ring0; bar = bar0; parity ^= 1; }
        };
        int it = 0;
        if (second) {  // the tile starts at the second block of a stage whose first block closed the previous tile
            block(cur + BLOCK_BYTES);
            next_stage();
            second = 0;
            it = 1;
        }
        for (; it + 2 <= n; it += 2) {  // whole stages: one wait, two blocks, one refill
            if (!mbar_wait_addr(bar, parity)) {
                if (lane == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
                return;
            }
#pragma unroll 1
            for (uint32_t h = 0; h < W4M1_COPY_BLOCKS * BLOCK_BYTES; h += BLOCK_BYTES) block(cur + h);
            next_stage();
        }
        if (it < n) {  // the tile (or the range) ends on the first block of a stage
            if (!mbar_wait_addr(bar, parity)) {
                if (lane == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
                return;
            }
            block(cur);
            second = 1;
        }
        b += n;

        // ---- end of this warp's share of the tile ---------------------------
        float acc[1][4] = {{acc_a * unscale, 0.f, acc_b * unscale, 0.f}};
        if (whole) {
            w4w_store_tile<1, EPI>(acc, tile, r, c, y, resid, N, 1);
        } else {
            // contributors of the tile: the warps whose ranges meet [tile*G, tile*G + G)
            const int cut = rem * (base + 1);
            const int first_b = tile * G, last_b = first_b + G - 1;
            const int w_first = first_b < cut ? first_b / (base + 1) : rem + (first_b - cut) / base;
            const int w_last = last_b < cut ? last_b / (base + 1) : rem + (last_b - cut) / base;
            const int which = wid == w_first ? 1 : 0;  // slot 1: the tile my range ends inside
            const int li = tile - cta_tile0;
            float sum[1][4] = {{0.f, 0.f, 0.f, 0.f}};
            bool last = false;
            if ((w_first >> 3) == (int)blockIdx.x && (w_last >> 3) == (int)blockIdx.x && li < W4M1_LOCAL_TILES) {
                // every contributor is a warp of this CTA: finish through shared memory
                if (c == 0) cta_part[warp][which][r] = make_float2(acc[0][0], acc[0][2]);
                __threadfence_block();
                __syncwarp();
                int arrived = 0;
                if (lane == 0) arrived = atomicAdd(&cta_cnt[li], 1);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                last = arrived == w_last - w_first;
                if (last) {
                    __threadfence_block();
                    for (int w = w_first; w <= w_last; ++w) {
                        const float2 v = cta_part[w & 7][w == w_first ? 1 : 0][r];
                        sum[0][0] += v.x;
                        sum[0][2] += v.y;
                    }
                }
            } else {
                float *mine = partials + ((size_t)wid * 2 + which) * W4W_SLOT_FLOATS + r * 2;
                if (c == 0) *reinterpret_cast<float2 *>(mine) = make_float2(acc[0][0], acc[0][2]);
                __threadfence();
                __syncwarp();
                int arrived = 0;
                if (lane == 0) arrived = atomicAdd(&counters[tile], 1);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                last = arrived == w_last - w_first;
                if (last) {
                    __threadfence();
                    for (int w = w_first; w <= w_last; ++w) {
                        const float *p = partials + ((size_t)w * 2 + (w == w_first ? 1 : 0)) * W4W_SLOT_FLOATS + r * 2;
                        const float2 v = __ldcg(reinterpret_cast<const float2 *>(p));
                        sum[0][0] += v.x;
                        sum[0][2] += v.y;
                    }
                    if (lane == 0) counters[tile] = 0;
                }
            }
            if (last) w4w_store_tile<1, EPI>(sum, tile, r, c, y, resid, N, 1);
        }
        g = 0;
        ++tile;
    }
}

}  // namespace ab2
