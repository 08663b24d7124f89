// The one-token decode step of one sequence as ONE persistent kernel: embedding,
// every block {RMSNorm + QKV, RoPE + KV append + attention, O + residual, RMSNorm +
// gate|up + SwiGLU, down + residual}, final norm + LM head, greedy argmax and the
// length commit (AarambhModel::forward_decode_batch at one row,
// crates/aarambh-studio-model/src/model.rs:590-641, with the sampling of
// crates/aarambh-studio-inference/src/sampler.rs:217-224).
//
// Why one kernel: at one token every phase of a block is a few microseconds of
// HBM time, and as separate launches each phase pays a kernel boundary, a cold
// ramp of its weight stream and its own tail.  Here one CTA per SM stays resident
// for the whole step (cooperative launch), the phases are separated by a grid
// barrier (one release add + acquire poll per CTA), and - the point of it - every
// warp's ring of weight blocks keeps streaming across the barriers: the weights
// are constants, so while a warp waits for the activations of the next phase its
// ring already holds that phase's first blocks.
//
// The projection phases are the one-token W4A16 GEMV of gemv_w4a16_m1.cuh (same
// layout, same arithmetic, same contributor-ordered finishing of cut tiles), with
// the CTA's prologue (RMSNorm, f16 copy of the activations, group sums) run once
// per SM and phase.  The attention phase gives every KV head `nsplit` CTAs; a CTA
// scores its slice of the cached tokens (one warp per token, a lane per four
// dimensions), normalises within the CTA, accumulates P.V, leaves its partial
// (max, sum, accumulator) in global memory, and the last CTA of a head to arrive
// merges the partials (log-sum-exp) and writes the head's output.
//
// Status: opt-in (AB2_PERSISTENT_STEP=1).  Measured on the Large-class decoder (one B200, context
// 512): 1.98 ms per step against 1.82 ms for the graph-replayed chain of kernels.  What a phase
// costs here besides its weight stream: the grid barrier (1.3 us), the projection prologue on
// 768 threads (2 to 3.5 us, every CTA converts the whole activation vector), the attention phase
// (10 us: a chain of dependent L2 round trips through three CTA barriers, the split merge and an
// atomic), and the one-tile imbalance of dealing 16-row tiles to 148 CTAs.  The weight rings do
// stream across the barriers as intended (the first blocks of a phase are resident when it
// starts), but the fixed costs above outweigh the kernel boundaries they replace.
//
// Every wait is bounded (two seconds of wall clock): a barrier or copy that never
// completes records AB2_ERR_TIMEOUT in the status word, the CTA waits (bounded)
// for its own copies in flight and returns.
#include <algorithm>
#include <cfloat>
#include <vector>

#include "common.cuh"
#include "kv_cache.cuh"
#include "ops.cuh"
#include "gemv_w4a16_m1.cuh"
#include "decode_step_persistent.cuh"

using namespace ab2;

namespace ab2 {
int device_sm_count();
int device_status_word(int **out);
int device_recovery_epoch();

namespace {

constexpr int PS_WARPS = 24;
constexpr int PS_THREADS = PS_WARPS * 32;
constexpr int PS_STAGES = 6;
constexpr int PS_NV = 3;           // vectors of 8 activations a thread holds between the prologue passes
constexpr int PS_MAX_K = 16384;    // <= PS_THREADS * 8 * PS_NV
constexpr int PS_LOCAL_TILES = 128;  // tiles of one projection a CTA may own
constexpr int PS_HD = 128;
constexpr int PS_TRACE = 10;         // timestamps kept per phase and traced CTA
constexpr int PS_MAX_CTA_TOKENS = 520;  // cached tokens one CTA attends (context bound / splits + the new one)
constexpr uint32_t PS_BLOCK_BYTES = W4_BLOCK_WORDS * 4;

enum { PS_GEMV = 0, PS_ATTN = 1, PS_EMBED = 2, PS_TAIL = 3 };

struct PsOp {
    int kind, epi, N, K;
    const uint32_t *wt;
    const __nv_bfloat16 *x;      // activations of the projection
    const float *norm_w;         // RMSNorm weight fused into the prologue, or null
    __nv_bfloat16 *y;            // output (null: the logits buffer of the call)
    const __nv_bfloat16 *resid;  // W4_EPI_ADD
    int layer, pad;
};

struct PsArgs {
    const PsOp *ops;
    int nops;
    float eps, scale;
    const float *cos_t, *sin_t;
    const uint32_t *emb;   // embedding table, W4A16 tile-major
    int emb_N, emb_K;
    const uint32_t *ids;   // the token (device)
    __nv_bfloat16 *x;      // residual stream [d]
    const __nv_bfloat16 *qkv;
    __nv_bfloat16 *attn;
    KvView kv;             // layer 0
    size_t kv_layer_tokens;
    int row, h, rep, nsplit;
    float *apart_acc;      // [kvh][nsplit][rep][128]
    float *apart_ml;       // [kvh][nsplit][rep][2]
    int *acount;           // [kvh], zero at rest
    unsigned int *bar;     // grid barrier: arrivals since the scratch was made
    unsigned int bar_base; // arrivals before this launch
    int *status;
    __nv_bfloat16 *logits;
    int vocab;
    uint32_t *argmax_out;  // or null
    unsigned long long *trace;  // [3 CTAs][nops][4] timestamps (ns): phase start, prologue done, CTA done, barrier passed
};

__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16 *p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];\n" : "=h"(v) : "l"(p));
    return __uint_as_float((uint32_t)v << 16);
}
__device__ __forceinline__ uint32_t ldcg_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];\n" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void i8x4_to_f32(uint32_t w, float (&f)[4]) {
    const uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
}

__device__ __forceinline__ long long ps_argmax_key(float v, int idx) {
    int b = __float_as_int(v);
    b ^= (int)(((unsigned)(b >> 31)) >> 1);
    return ((long long)b << 32) | (unsigned)idx;
}

// floor(n / d) for small non-negative n and positive d without the integer-division sequence
// (this runs once per cut tile, in code that is fetched cold every phase).
__device__ __forceinline__ int ps_div_floor(int n, int d) {
    int q = (int)__fdividef((float)n + 0.5f, (float)d);
    if (q * d > n) --q;
    else if ((q + 1) * d <= n) ++q;
    return q;
}
// The warp whose contiguous run holds block b when nb = 24 * base + rem blocks are dealt to 24
// warps, the first `rem` of them taking base + 1.
__device__ __forceinline__ int ps_warp_of_block(int b, int base, int rem) {
    const int cut = rem * (base + 1);
    return b < cut ? ps_div_floor(b, base + 1) : rem + ps_div_floor(b - cut, base);
}

// Shared memory of the attention phase; it aliases the activation area of the
// projection phases (a grid barrier lies between any two uses).
struct PsAttnSmem {
    float qs[4][PS_HD];                 // rotated queries of the KV head's query heads
    float sc[PS_MAX_CTA_TOKENS][4];     // scores, then probabilities x V scale
    float vscale[PS_MAX_CTA_TOKENS];
    float newk[PS_HD], newv[PS_HD];     // the new token as the cache will return it
    float pacc[PS_WARPS][PS_HD];        // P.V per (token subset, head) warp
    float hm[4], hl[4];                 // this CTA's running max and sum per head
    float mlbuf[4][16][2];              // (max, sum) of every split of the head, for the merge
};

__host__ __device__ constexpr size_t ps_act_bytes() {
    size_t gemv = (size_t)PS_MAX_K * 2 + (size_t)(PS_MAX_K >> 7) * 8;
    return gemv > sizeof(PsAttnSmem) ? gemv : sizeof(PsAttnSmem);
}
// rings, activation / attention area, mbarriers, then a copy of the op list
__host__ __device__ constexpr size_t ps_smem_bytes(int nops) {
    return (size_t)PS_WARPS * PS_STAGES * PS_BLOCK_BYTES + ((ps_act_bytes() + 127) / 128) * 128 +
           (size_t)PS_WARPS * PS_STAGES * 8 + (size_t)nops * sizeof(PsOp);
}


// Named barrier over `count` threads (a multiple of 32).
__device__ __forceinline__ void ps_bar(int id, int count) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// The projection prologue of one CTA: the K bf16 activations at `x` (optionally RMS-normalised,
// x * rsqrt(mean(x^2) + eps) * norm_w rounded to bf16) become, in shared memory, f16 values
// scaled by a power of two 2^e that puts the largest magnitude in [2^14, 2^15) (elements 2, 3,
// 6, 7 of every eight by a further 2^-4), plus (C2, T) per group of 128 for the main loop
// (gemv_w4a16_m1.cuh explains the arithmetic).  Returns 2^-e.
//
// Measured: 2 to 3.5 us per phase on 768 threads, of which about 1 us is the instruction fetch
// of code that the weight loop evicted in between (a second call right after the first takes
// 1.5 to 2 us).  Calling it once on stale data while the CTA waits at the grid barrier, to warm
// the instruction cache, was tried (hence the barrier id and thread count arguments): the dry
// call outlasts the barrier wait, and the step got slower (2.17 against 2.03 ms).
__device__ __forceinline__ float ps_prologue(const __nv_bfloat16 *x, const float *norm_w, int K, float eps, uint32_t xs0,
                                          uint32_t gs0, float2 *warp_part, int tid, int bar_id, int bar_count) {
    const int warp = tid >> 5, lane = tid & 31;
    const uint4 *x4 = reinterpret_cast<const uint4 *>(x);
    const int nvec = K >> 3;  // a multiple of 32: the guards below are uniform per warp
    {
        uint4 xv[PS_NV];
#pragma unroll
        for (int it = 0; it < PS_NV; ++it) {
            const int i = tid + it * PS_THREADS;
            if (i < nvec) xv[it] = __ldcg(x4 + i);
        }
#pragma unroll
        for (int it = 0; it < PS_NV; ++it) {
            const int i = tid + it * PS_THREADS;
            if (i < nvec)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(xs0 + i * 16), "r"(xv[it].x), "r"(xv[it].y),
                             "r"(xv[it].z), "r"(xv[it].w)
                             : "memory");
        }
    }
    // pass 1: sum of squares and largest magnitude (each thread re-reads what it stored)
    float ss = 0.f, amax = 0.f;
#pragma unroll 1
    for (int i = tid; i < nvec; i += PS_THREADS) {
        const uint4 v = lds128(xs0 + i * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        if (norm_w) {
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i);
            const float4 w1 = __ldg(reinterpret_cast<const float4 *>(norm_w) + 2 * i + 1);
            const float nw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float f0 = __uint_as_float(w[j] << 16), f1 = __uint_as_float(w[j] & 0xffff0000u);
                ss = fmaf(f0, f0, ss);
                ss = fmaf(f1, f1, ss);
                amax = fmaxf(amax, fmaxf(fabsf(f0 * nw[2 * j]), fabsf(f1 * nw[2 * j + 1])));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xffff0000u))));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
    if (lane == 0) warp_part[warp] = make_float2(ss, amax);
    ps_bar(bar_id, bar_count);
    {
        const float2 t = lane < PS_WARPS ? warp_part[lane] : make_float2(0.f, 0.f);
        ss = t.x;
        amax = t.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        }
    }
    float inv = 1.f;
    if (norm_w) {
        inv = rsqrtf(fmaf(ss, 1.0f / (float)K, eps));  // within 2 ulp of the separately rounded form
        amax = amax * inv * 1.0078125f;                // bound on |bf16(x inv w)|
    }
    int e = 141 - (int)((__float_as_uint(amax) >> 23) & 0xffu);
    e = max(-100, min(100, e));
    const float sc_lo = __uint_as_float((uint32_t)(e + 127) << 23);
    const float sc_hi = __uint_as_float((uint32_t)(e - 4 + 127) << 23);

    // pass 2: f16 copy (in place) and group sums
#pragma unroll 1
    for (int i = tid; i < nvec; i += PS_THREADS) {
        const uint4 v = lds128(xs0 + i * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float nw[8];
        if (norm_w) {
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
            if (norm_w) {
                f0 = bf16_round(__fmul_rn(__fmul_rn(f0, inv), nw[2 * j]));
                f1 = bf16_round(__fmul_rn(__fmul_rn(f1, inv), nw[2 * j + 1]));
            }
            const float sc = (j & 1) ? sc_hi : sc_lo;  // words 1 and 3 hold elements 2,3 and 6,7
            const __half2 hh = __floats2half2_rn(f0 * sc, f1 * sc);
            h[j] = *reinterpret_cast<const uint32_t *>(&hh);
            const float2 back = __half22float2(hh);
            p += back.x + back.y;
            sum += f0 + f1;
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(xs0 + i * 16), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3])
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
            asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(gs0 + (i >> 4) * 8), "f"(C2), "f"(T) : "memory");
        }
    }
    ps_bar(bar_id, bar_count);
    return __uint_as_float((uint32_t)(127 - e) << 23);
}

template <bool TRACE>
__global__ void __launch_bounds__(PS_THREADS, 1) decode_step_persistent_kernel(const PsArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float2 warp_part[PS_WARPS];
    __shared__ float2 cta_part[PS_WARPS][2][8];
    __shared__ int cta_cnt[PS_LOCAL_TILES];
    __shared__ int s_abort, s_last;
    __shared__ long long warp_best[PS_WARPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, c = lane & 3;

    const uint32_t smem0 = smem_addr(smem_raw);
    const uint32_t act0 = smem0 + PS_WARPS * PS_STAGES * PS_BLOCK_BYTES;  // activations / attention area
    unsigned char *act_ptr = smem_raw + (size_t)PS_WARPS * PS_STAGES * PS_BLOCK_BYTES;
    const uint32_t bars0 = act0 + (uint32_t)(((ps_act_bytes() + 127) / 128) * 128);
    const uint32_t ring0 = smem0 + warp * PS_STAGES * PS_BLOCK_BYTES, bar0 = bars0 + warp * PS_STAGES * 8;
    const uint32_t ring_end = ring0 + PS_STAGES * PS_BLOCK_BYTES;
    const uint32_t lane0 = lane == 0 ? 1u : 0u;

    // the op list lives in shared memory: a phase must not start with a round trip for its descriptor
    const PsOp *ops = reinterpret_cast<const PsOp *>(smem_raw + (size_t)PS_WARPS * PS_STAGES * PS_BLOCK_BYTES +
                                                      ((ps_act_bytes() + 127) / 128) * 128 + (size_t)PS_WARPS * PS_STAGES * 8);
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.ops);
        uint4 *dst = reinterpret_cast<uint4 *>(const_cast<PsOp *>(ops));
        for (int i = tid; i < a.nops * (int)(sizeof(PsOp) / 16); i += PS_THREADS) dst[i] = src[i];
    }
    // A projection's 16-row tiles are dealt to the CTAs in contiguous runs (equal to within one
    // tile) and the blocks of a CTA's tiles to its warps in contiguous runs (equal to within one
    // block): a tile is finished inside one CTA, through shared memory.
    auto cta_tiles = [&](int N, int &tile_lo, int &ntile) {
        const int tiles = (N + 15) >> 4;
        const int tb = tiles / (int)gridDim.x, tr = tiles - tb * (int)gridDim.x;
        tile_lo = (int)blockIdx.x * tb + min((int)blockIdx.x, tr);
        ntile = tb + ((int)blockIdx.x < tr ? 1 : 0);
    };

    if (tid == 0) s_abort = 0;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < PS_STAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar0 + s * 8));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    // ---- the fetch cursor: walks this warp's block ranges of every projection, in order
    int f_op = -1, f_left = 0;
    const uint32_t *f_src = nullptr;
    int in_flight = 0;
    auto next_range = [&]() {
        while (f_left == 0 && f_op < a.nops) {
            ++f_op;
            if (f_op >= a.nops) break;
            if (ops[f_op].kind != PS_GEMV) continue;
            int tile_lo, ntile;
            cta_tiles(ops[f_op].N, tile_lo, ntile);
            const int G = ops[f_op].K >> 7, nb = ntile * G;
            const int base = nb / PS_WARPS, rem = nb - base * PS_WARPS;
            f_left = base + (warp < rem ? 1 : 0);
            f_src = ops[f_op].wt + ((size_t)tile_lo * G + warp * base + min(warp, rem)) * W4_BLOCK_WORDS;
        }
    };
    // `after`: a value the copy must wait for (the sums that the loads of the stage have fed): it enters the
    // source address masked with a zero the compiler cannot see, so the copy is not issued while a load of
    // the stage is still under way.
    const uint32_t hidden_zero = (uint32_t)a.nops >> 30;
    auto refill = [&](uint32_t stage, uint32_t bar, uint32_t after = 0u) {
        const uint32_t go = f_left > 0 ? 1u : 0u;
        bulk_g2s_if(lane0 & go, stage, f_src + (after & hidden_zero), PS_BLOCK_BYTES, bar);
        if (go) {
            f_src += W4_BLOCK_WORDS;
            ++in_flight;
            if (--f_left == 0) next_range();
        }
    };
    next_range();
#pragma unroll 1
    for (int j = 0; j < PS_STAGES; ++j) refill(ring0 + j * PS_BLOCK_BYTES, bar0 + j * 8);

    // ---- attention geometry: the same in every block (one sequence, one new token)
    const int att_on = (int)blockIdx.x < a.kv.kvh * a.nsplit ? 1 : 0;
    const int att_kvhead = (int)blockIdx.x / a.nsplit, att_rank = (int)blockIdx.x % a.nsplit;
    const int att_pos = a.kv.lens[a.row];
    const int att_chunk = (att_pos + a.nsplit - 1) / a.nsplit;
    const int att_c0 = min(att_pos, att_rank * att_chunk);
    const int att_ncached = att_on ? min(att_pos, att_c0 + att_chunk) - att_c0 : 0;
    const size_t att_head_base = ((size_t)a.row * a.kv.kvh + (att_on ? att_kvhead : 0)) * a.kv.cap;

    uint32_t cur = ring0, bar = bar0, parity = 0;
    bool dead = false;  // a copy of this warp never arrived: it only keeps the barriers company
    uint32_t k_lo = 0x000F000Fu, k_hi = 0x00F000F0u, k_magic = 0x64006400u;
    asm volatile("" : "+r"(k_lo), "+r"(k_hi), "+r"(k_magic));
    unsigned int barrier_no = 0;
    // phase timestamps of the first, the middle and the last CTA (thread 0 of each)
    const int trace_slot = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x / 2 ? 1 : (blockIdx.x == gridDim.x - 1 ? 2 : -1));
    auto stamp = [&](int oi, int which) {
        if (TRACE && trace_slot >= 0 && tid == 0) a.trace[((size_t)trace_slot * a.nops + oi) * PS_TRACE + which] = mbar_wall_ns();
    };

    for (int oi = 0; oi < a.nops; ++oi) {
        const PsOp &op = ops[oi];
        const int kind = op.kind;
        stamp(oi, 0);
        if (kind != PS_GEMV) stamp(oi, 1);
        if (kind == PS_EMBED) {
            // TokenEmbedding::forward: x = dequant(table[id, :]), one element per thread
            const int k = (int)blockIdx.x * PS_THREADS + tid;
            if (k < a.emb_K) {
                uint32_t id = a.ids[0];
                if (id >= (uint32_t)a.emb_N) id = a.emb_N - 1;
                W4Layout L{a.emb_N, a.emb_K, 128};
                const uint32_t word = a.emb[L.code_index((int)id, k >> 3)];
                const int e = k & 7, slot = (e >> 1) + 4 * (e & 1);
                const uint32_t p = a.emb[L.param_index((int)id, k >> 7)];
                const float v = __fmul_rn(__fsub_rn((float)((word >> (4 * slot)) & 0xFu), (float)((p >> 16) & 0xFu)),
                                          bf16_bits_to_f32((uint16_t)(p & 0xffffu)));
                a.x[k] = __float2bfloat16_rn(v);
            }
        } else if (kind == PS_GEMV) {
            const int K = op.K, N = op.N, G = K >> 7;
            int tile_lo, ntile;
            cta_tiles(N, tile_lo, ntile);
            const int nb = ntile * G;  // blocks of this CTA, numbered from its first tile
            const int base = nb / PS_WARPS, rem = nb - base * PS_WARPS;
            const int b0 = warp * base + min(warp, rem);
            const int nblk = base + (warp < rem ? 1 : 0);
            const int b1 = b0 + nblk;
            const uint32_t xs0 = act0, gs0 = act0 + K * 2;
            const float *norm_w = op.norm_w;
            if (tid < PS_LOCAL_TILES) cta_cnt[tid] = 0;
          if (ntile > 0) {  // a CTA without tiles of this projection has nothing to prepare

            // ---- prologue (one shared instance of the code: see ps_prologue)
            const float unscale = ps_prologue(op.x, norm_w, K, a.eps, xs0, gs0, warp_part, tid, 0, PS_THREADS);
            stamp(oi, 1);

            // ---- main loop: this warp's blocks ------------------------------------
            const uint32_t code_off = (r * 16 + c * 4) * 4;
            const uint32_t param_off = (256 + r) * 4;
            const uint32_t has_x = r == 0 ? 1u : 0u;
            const uint32_t xlane = xs0 + c * 64;
            __nv_bfloat16 *y = op.y ? op.y : a.logits;
            const int epi = op.epi;

            int lt = b0 / G, g = b0 - lt * G;  // tile of the CTA, group

            uint4 xw[4];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) xw[wi] = make_uint4(0u, 0u, 0u, 0u);

#pragma unroll 1
            for (int b = b0; b < b1 && !dead;) {
                const int n = min(G - g, b1 - b);
                const bool whole = n == G;
                float acc_a = 0.f, acc_b = 0.f;
                uint32_t xaddr = xlane + g * 256, gaddr = gs0 + g * 8;

#pragma unroll 1
                for (int it = 0; it < n; ++it) {
                    if (!mbar_wait_addr(bar, parity)) {
                        if (lane == 0) atomicExch(a.status, (int)AB2_ERR_TIMEOUT);
                        dead = true;
                        break;
                    }
                    const uint4 wa = lds128(cur + code_off);
                    const uint4 wb = lds128(cur + code_off + 512);
                    const uint32_t pa = lds32(cur + param_off), pb = lds32(cur + param_off + 32);
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
                    const float sa = __uint_as_float(pa << 16), sb = __uint_as_float(pb << 16);
                    const float nza = __uint_as_float(pa & 0xffff0000u), nzb = __uint_as_float(pb & 0xffff0000u);
                    acc_a = fmaf(sa, (d[0] + d2[0]) - fmaf(-nza, T, C2), acc_a);
                    acc_b = fmaf(sb, (d[2] + d2[2]) - fmaf(-nzb, T, C2), acc_b);

                    // refill this stage with the next block of the cursor (this phase or a later one)
                    __syncwarp();
                    --in_flight;
                    refill(cur, bar, __float_as_uint(acc_a) ^ __float_as_uint(acc_b));
                    cur += PS_BLOCK_BYTES;
                    bar += 8;
                    if (cur == ring_end) { cur = ring0; bar = bar0; parity ^= 1; }
                }
                if (dead) break;
                b += n;

                // ---- end of this warp's share of the tile ---------------------------
                float va = acc_a * unscale, vb = acc_b * unscale;
                bool store = whole;
                if (!whole) {
                    // The tile is shared with other warps of this CTA: the warps whose ranges meet
                    // [lt*G, lt*G + G).  Each leaves its partial in a slot (slot 1: the tile its range
                    // ends inside) and bumps the tile's counter; the last to arrive sums the slots in
                    // warp order (= block order), so the result does not depend on arrival order.
                    const int w_first = ps_warp_of_block(lt * G, base, rem);
                    const int w_last = ps_warp_of_block(lt * G + G - 1, base, rem);
                    const int which = warp == w_first ? 1 : 0;
                    if (c == 0) cta_part[warp][which][r] = make_float2(va, vb);
                    __threadfence_block();
                    __syncwarp();
                    int arrived = 0;
                    if (lane == 0) arrived = atomicAdd(&cta_cnt[lt], 1);
                    arrived = __shfl_sync(0xffffffffu, arrived, 0);
                    store = arrived == w_last - w_first;
                    if (store) {
                        __threadfence_block();
                        va = 0.f;
                        vb = 0.f;
#pragma unroll 1
                        for (int w = w_first; w <= w_last; ++w) {
                            const float2 v = cta_part[w][w == w_first ? 1 : 0][r];
                            va += v.x;
                            vb += v.y;
                        }
                    }
                }
                const int tile = tile_lo + lt;
                if (store && c == 0) {
                    if (epi == W4_EPI_SWIGLU) {
                        const int col = tile * 8 + r;
                        if (col < (N >> 1)) {  // silu(gate) * up on the rounded projections; fast exp / divide (1e-6 relative)
                            const float gt = bf16_round(va);
                            y[col] = __float2bfloat16_rn(__fdividef(gt, 1.0f + __expf(-gt)) * bf16_round(vb));
                        }
                    } else {
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int row = tile * 16 + r + 8 * hh;
                            if (row < N) {
                                float v = hh ? vb : va;
                                if (epi == W4_EPI_ADD) v = ldcg_bf16(op.resid + row) + bf16_round(v);
                                y[row] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                }
                g = 0;
                ++lt;
            }
            stamp(oi, 7);  // warp 0 is through its blocks
          }  // ntile > 0
        } else if (kind == PS_ATTN) {
            const int nsplit = a.nsplit, rep = a.rep, kvh = a.kv.kvh;
            if (att_on) {
                PsAttnSmem &S = *reinterpret_cast<PsAttnSmem *>(act_ptr);
                const int kvhead = att_kvhead, rank = att_rank;
                constexpr int half = PS_HD / 2;
                const int pos = att_pos;
                const size_t layer_off = (size_t)op.layer * a.kv_layer_tokens;
                const int8_t *kc = (const int8_t *)a.kv.k + layer_off * PS_HD;
                const int8_t *vc = (const int8_t *)a.kv.v + layer_off * PS_HD;
                float *ksc = a.kv.ks + layer_off, *vsc = a.kv.vs + layer_off;
                const size_t head_base = att_head_base;
                const float *cs = a.cos_t + (size_t)pos * half, *sn = a.sin_t + (size_t)pos * half;
                // cached tokens of this CTA; the last split also owns the new token
                const int c0 = att_c0, ncached = att_ncached;
                const bool owns_new = rank == nsplit - 1;
                const int ntok = ncached + (owns_new ? 1 : 0);

                // ---- rotated queries (one pair per thread), rounded to bf16
                for (int i = tid; i < rep * half; i += PS_THREADS) {
                    const int hh = i / half, qd = i % half;
                    const __nv_bfloat16 *qp = a.qkv + (size_t)(kvhead * rep + hh) * PS_HD;
                    float o1, o2;
                    rope_rotate(ldcg_bf16(qp + qd), ldcg_bf16(qp + half + qd), cs[qd], sn[qd], o1, o2);
                    S.qs[hh][qd] = bf16_round(o1);
                    S.qs[hh][half + qd] = bf16_round(o2);
                }
                // ---- the new token: rotation, per-token absmax INT8, store into the cache
                if (owns_new && warp == PS_WARPS - 1) {
                    const __nv_bfloat16 *kp = a.qkv + (size_t)(a.h + kvhead) * PS_HD;
                    const __nv_bfloat16 *vp = a.qkv + (size_t)(a.h + kvh + kvhead) * PS_HD;
                    const uint32_t klo = ldcg_u32(kp + 2 * lane), khi = ldcg_u32(kp + half + 2 * lane);
                    const uint32_t vlo = ldcg_u32(vp + 2 * lane), vhi = ldcg_u32(vp + half + 2 * lane);
                    const float2 nc = *reinterpret_cast<const float2 *>(cs + 2 * lane);
                    const float2 ns = *reinterpret_cast<const float2 *>(sn + 2 * lane);
                    float kd[4], vd[4], o1, o2;
                    rope_rotate(__uint_as_float(klo << 16), __uint_as_float(khi << 16), nc.x, ns.x, o1, o2);
                    kd[0] = bf16_round(o1); kd[2] = bf16_round(o2);
                    rope_rotate(__uint_as_float(klo & 0xffff0000u), __uint_as_float(khi & 0xffff0000u), nc.y, ns.y, o1, o2);
                    kd[1] = bf16_round(o1); kd[3] = bf16_round(o2);
                    vd[0] = __uint_as_float(vlo << 16); vd[1] = __uint_as_float(vlo & 0xffff0000u);
                    vd[2] = __uint_as_float(vhi << 16); vd[3] = __uint_as_float(vhi & 0xffff0000u);
                    float ka = fmaxf(fmaxf(fabsf(kd[0]), fabsf(kd[1])), fmaxf(fabsf(kd[2]), fabsf(kd[3])));
                    float va = fmaxf(fmaxf(fabsf(vd[0]), fabsf(vd[1])), fmaxf(fabsf(vd[2]), fabsf(vd[3])));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
                        va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o));
                    }
                    const float kscale = (ka <= FLT_EPSILON) ? 1.0f : __fdiv_rn(ka, 127.0f);
                    const float vscale = (va <= FLT_EPSILON) ? 1.0f : __fdiv_rn(va, 127.0f);
                    auto enc = [](float x, float sc) -> float {
                        float q = roundf(__fdiv_rn(x, sc));
                        q = q < -127.f ? -127.f : (q > 127.f ? 127.f : q);
                        return (q != q) ? 0.f : q;
                    };
                    float kq[4], vq[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        kq[i] = enc(kd[i], kscale);
                        vq[i] = enc(vd[i], vscale);
                        kd[i] = __fmul_rn(kq[i], kscale);
                        vd[i] = __fmul_rn(vq[i], vscale);
                    }
                    if (pos < a.kv.cap) {
                        const size_t trow = head_base + pos;
                        auto pack2 = [](float x, float y) -> uint16_t {
                            return (uint16_t)((uint32_t)(uint8_t)(int8_t)x | ((uint32_t)(uint8_t)(int8_t)y << 8));
                        };
                        uint16_t *kw = reinterpret_cast<uint16_t *>(const_cast<int8_t *>(kc) + trow * PS_HD);
                        uint16_t *vw = reinterpret_cast<uint16_t *>(const_cast<int8_t *>(vc) + trow * PS_HD);
                        kw[lane] = pack2(kq[0], kq[1]);
                        kw[32 + lane] = pack2(kq[2], kq[3]);
                        vw[lane] = pack2(vq[0], vq[1]);
                        vw[32 + lane] = pack2(vq[2], vq[3]);
                        if (lane == 0) { ksc[trow] = kscale; vsc[trow] = vscale; }
                    }
                    S.newk[2 * lane] = kd[0]; S.newk[2 * lane + 1] = kd[1];
                    S.newk[half + 2 * lane] = kd[2]; S.newk[half + 2 * lane + 1] = kd[3];
                    S.newv[2 * lane] = vd[0]; S.newv[2 * lane + 1] = vd[1];
                    S.newv[half + 2 * lane] = vd[2]; S.newv[half + 2 * lane + 1] = vd[3];
                }
                __syncthreads();
                stamp(oi, 4);

                // ---- scores: a warp per token, a lane per four dimensions.  Loops are kept rolled:
                // this code runs once per block and is fetched cold each time, so its length counts.
                {
                    // the next token's row is requested before the current one is reduced
                    auto fetch = [&](int t, uint32_t &kraw, float &ksv, float &vsv) {
                        kraw = 0u; ksv = 1.f; vsv = 1.f;
                        if (t < ncached) {
                            const size_t trow = head_base + c0 + t;
                            kraw = __ldg(reinterpret_cast<const uint32_t *>(kc + trow * PS_HD + lane * 4));
                            ksv = __ldg(ksc + trow);
                            vsv = __ldg(vsc + trow);
                        }
                    };
                    uint32_t kraw_n;
                    float ks_n, vs_n;
                    fetch(warp, kraw_n, ks_n, vs_n);
#pragma unroll 1
                    for (int t = warp; t < ntok; t += PS_WARPS) {
                        const uint32_t kraw = kraw_n;
                        const float ksv = ks_n, vsv = vs_n;
                        fetch(t + PS_WARPS, kraw_n, ks_n, vs_n);
                        float kf[4];
                        i8x4_to_f32(kraw, kf);
                        if (t >= ncached) {  // the new token, already dequantised
                            const float4 nk = *reinterpret_cast<const float4 *>(&S.newk[lane * 4]);
                            kf[0] = nk.x; kf[1] = nk.y; kf[2] = nk.z; kf[3] = nk.w;
                        }
#pragma unroll 1
                        for (int hh = 0; hh < rep; ++hh) {
                            const float4 q = *reinterpret_cast<const float4 *>(&S.qs[hh][lane * 4]);
                            float dot = q.x * kf[0];
                            dot = fmaf(q.y, kf[1], dot);
                            dot = fmaf(q.z, kf[2], dot);
                            dot = fmaf(q.w, kf[3], dot);
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                            if (lane == 0) S.sc[t][hh] = dot * ksv * a.scale;
                        }
                        if (lane == 0) S.vscale[t] = vsv;
                    }
                }
                __syncthreads();
                stamp(oi, 5);
                // ---- softmax within the CTA: warp hh normalises head hh
                if (warp < rep) {
                    float m = -INFINITY;
#pragma unroll 1
                    for (int t = lane; t < ntok; t += 32) m = fmaxf(m, S.sc[t][warp]);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                    float l = 0.f;
#pragma unroll 1
                    for (int t = lane; t < ntok; t += 32) {
                        const float p = __expf(S.sc[t][warp] - m);
                        l += p;
                        S.sc[t][warp] = p * S.vscale[t];
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
                    if (lane == 0) { S.hm[warp] = m; S.hl[warp] = l; }
                }
                __syncthreads();
                stamp(oi, 6);
                // ---- P.V: warp = (token subset, head), a lane per four dimensions; four tokens in flight
                {
                    const int hh = warp % rep, ts = warp / rep, nts = PS_WARPS / rep;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                    for (int t0 = ts; t0 < ntok; t0 += 4 * nts) {
                        uint32_t raw[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int t = min(t0 + u * nts, max(ncached - 1, 0));
                            raw[u] = __ldg(reinterpret_cast<const uint32_t *>(vc + (head_base + c0 + t) * PS_HD + lane * 4));
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int t = t0 + u * nts;
                            float vf[4];
                            i8x4_to_f32(raw[u], vf);
                            if (t >= ncached && t < ntok) {  // the new token (past the end the clamped row stands, times 0)
                                const float4 nv = *reinterpret_cast<const float4 *>(&S.newv[lane * 4]);
                                vf[0] = nv.x; vf[1] = nv.y; vf[2] = nv.z; vf[3] = nv.w;
                            }
                            const float pv = t < ntok ? S.sc[t][hh] : 0.f;
#pragma unroll
                            for (int j = 0; j < 4; ++j) acc[j] = fmaf(pv, vf[j], acc[j]);
                        }
                    }
                    *reinterpret_cast<float4 *>(&S.pacc[warp][lane * 4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                }
                __syncthreads();
                stamp(oi, 7);
                // ---- this CTA's partial -> global memory
                const size_t pbase = ((size_t)kvhead * nsplit + rank) * rep;
                for (int i = tid; i < rep * PS_HD; i += PS_THREADS) {
                    const int hh = i / PS_HD, d = i % PS_HD;
                    float A = 0.f;
#pragma unroll 1
                    for (int ts = 0; ts < PS_WARPS / rep; ++ts) A += S.pacc[ts * rep + hh][d];
                    a.apart_acc[(pbase + hh) * PS_HD + d] = A;
                    if (d == 0) *reinterpret_cast<float2 *>(&a.apart_ml[(pbase + hh) * 2]) = make_float2(S.hm[hh], S.hl[hh]);
                }
                __threadfence();
                __syncthreads();
                if (tid == 0) s_last = atomicAdd(&a.acount[kvhead], 1) == nsplit - 1 ? 1 : 0;
                __syncthreads();
                stamp(oi, 8);
                if (s_last) {
                    // the last CTA of the head to arrive merges the splits (log-sum-exp)
                    __threadfence();
                    if (tid < rep * nsplit) {
                        const int hh = tid / nsplit, s2 = tid % nsplit;
                        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(&a.apart_ml[(((size_t)kvhead * nsplit + s2) * rep + hh) * 2]));
                        S.mlbuf[hh][s2][0] = ml.x;
                        S.mlbuf[hh][s2][1] = ml.y;
                    }
                    __syncthreads();
                    for (int i = tid; i < rep * PS_HD; i += PS_THREADS) {
                        const int hh = i / PS_HD, d = i % PS_HD;
                        float M = -INFINITY;
#pragma unroll 1
                        for (int s2 = 0; s2 < nsplit; ++s2) M = fmaxf(M, S.mlbuf[hh][s2][0]);
                        float L = 0.f, A = 0.f;
                        const float *accp = a.apart_acc + ((size_t)kvhead * nsplit * rep + hh) * PS_HD + d;
#pragma unroll 4
                        for (int s2 = 0; s2 < nsplit; ++s2) {
                            const float e2 = __expf(S.mlbuf[hh][s2][0] - M);  // exp(-inf) = 0 for an empty split
                            L = fmaf(e2, S.mlbuf[hh][s2][1], L);
                            A = fmaf(e2, __ldcg(accp + (size_t)s2 * rep * PS_HD), A);
                        }
                        a.attn[(size_t)(kvhead * rep + hh) * PS_HD + d] = __float2bfloat16_rn(L > 0.f ? A * (1.0f / L) : A);
                    }
                    if (tid == 0) a.acount[kvhead] = 0;
                }
            }
        } else {  // PS_TAIL: greedy token (last maximum under the f32 total order) and the length commit
            if (blockIdx.x == 0) {
                if (a.argmax_out) {
                    long long best = LLONG_MIN;
                    const int nvec = a.vocab >> 3;
                    const uint4 *row4 = reinterpret_cast<const uint4 *>(a.logits);
                    for (int i = tid; i < nvec; i += PS_THREADS) {
                        const uint4 v = __ldcg(row4 + i);
                        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            best = max(best, ps_argmax_key(__uint_as_float(w[j] << 16), i * 8 + 2 * j));
                            best = max(best, ps_argmax_key(__uint_as_float(w[j] & 0xffff0000u), i * 8 + 2 * j + 1));
                        }
                    }
                    for (int i = (nvec << 3) + tid; i < a.vocab; i += PS_THREADS) best = max(best, ps_argmax_key(ldcg_bf16(a.logits + i), i));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
                    if (lane == 0) warp_best[warp] = best;
                    __syncthreads();
                    if (warp == 0) {
                        long long v = lane < PS_WARPS ? warp_best[lane] : LLONG_MIN;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
                        if (lane == 0) a.argmax_out[0] = (uint32_t)(v & 0xffffffffll);
                    }
                }
                if (tid == 0) a.kv.lens[a.row] += 1;
            }
        }

        // ---- grid barrier: the next phase reads what this one wrote ------------------
        if (oi + 1 < a.nops) {
            ++barrier_no;
            // what the next phase reads and this launch never writes is pulled into L2 while the
            // CTA waits: the RMSNorm weight, or the cached K / V rows of this CTA's tokens
            {
                const PsOp &nx = ops[oi + 1];
                if (nx.kind == PS_GEMV && nx.norm_w) {
                    for (int i = tid; i < nx.K >> 5; i += PS_THREADS)
                        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(nx.norm_w + (size_t)i * 32));
                } else if (nx.kind == PS_ATTN && att_ncached > 0) {
                    const size_t layer_off = (size_t)nx.layer * a.kv_layer_tokens;
                    const size_t trow0 = layer_off + att_head_base + att_c0;
                    if (tid < att_ncached) {
                        asm volatile("prefetch.global.L2 [%0];\n" ::"l"((const int8_t *)a.kv.k + (trow0 + tid) * PS_HD));
                        asm volatile("prefetch.global.L2 [%0];\n" ::"l"((const int8_t *)a.kv.v + (trow0 + tid) * PS_HD));
                    }
                    if (tid * 32 < att_ncached) {  // scale words: 32 per line
                        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(a.kv.ks + trow0 + tid * 32));
                        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(a.kv.vs + trow0 + tid * 32));
                    }
                }
            }
            __syncthreads();
            stamp(oi, 2);
            if (tid == 0) {
                const unsigned int target = a.bar_base + barrier_no * gridDim.x;
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(a.bar) : "memory");
                bool ok = false;
                unsigned long long t_start = 0;
                for (int spin = 0;; ++spin) {
                    unsigned int v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(a.bar) : "memory");
                    if ((int)(v - target) >= 0) { ok = true; break; }
                    if ((spin & 255) == 255) {
                        const unsigned long long now = mbar_wall_ns();
                        if (t_start == 0) t_start = now;
                        else if (now - t_start > 2000000000ull) break;  // two seconds
                    }
                }
                if (!ok) {
                    atomicExch(a.status, (int)AB2_ERR_TIMEOUT);
                    s_abort = 1;
                }
            }
            __syncthreads();
            stamp(oi, 3);
            if (s_abort) break;
        }
    }

    // ---- leave: nothing of this warp may still be in flight towards shared memory.  After a
    // normal step the cursor has run out and every copy was consumed; after a timeout the
    // stages still pending are waited for (bounded).
    for (; in_flight > 0 && !dead; --in_flight) {
        if (!mbar_wait_addr(bar, parity)) break;
        cur += PS_BLOCK_BYTES;
        bar += 8;
        if (cur == ring_end) { cur = ring0; bar = bar0; parity ^= 1; }
    }
}

}  // namespace

struct PersistentStep {
    PsOp *ops_dev = nullptr;
    int nops = 0, grid = 0, nsplit = 1, device = 0;
    PsModelDesc desc;
    float *apart_acc = nullptr, *apart_ml = nullptr;
    int *acount = nullptr;
    unsigned int *bar = nullptr;
    unsigned int bar_total = 0;  // arrivals the barrier word has seen once every launch so far has finished
    int max_tiles = 0, recovery_epoch = 0;
    unsigned long long *trace = nullptr;
    bool traced = false;
};

static bool ps_weight_ok(const ab2_qweight *w) {
    return w && w->fmt == FMT_W4A16 && w->group == 128 && w->K % 128 == 0 && w->K <= PS_MAX_K;
}

int persistent_step_create(PersistentStep **out, const PsModelDesc &d) {
    *out = nullptr;
    // Opt-in (AB2_PERSISTENT_STEP=1, read when a model is finalised): on the Large-class decoder the
    // graph-replayed chain of kernels is still the faster of the two (1.82 against 1.98 ms per step).
    const char *on = getenv("AB2_PERSISTENT_STEP");
    if (!on || on[0] == '0') return AB2_OK;
    if (d.head_dim != PS_HD || d.n_heads % d.n_kv_heads != 0) return AB2_OK;
    const int rep = d.n_heads / d.n_kv_heads;
    if (rep != 1 && rep != 2 && rep != 4) return AB2_OK;
    if (!ps_weight_ok(d.embedding) || d.embedding->K != d.d_model || !ps_weight_ok(d.lm_head)) return AB2_OK;
    for (int l = 0; l < d.n_layers; ++l) {
        const PsLayerDesc &L = d.layers[l];
        if (!ps_weight_ok(L.wqkv) || !ps_weight_ok(L.wo) || !ps_weight_ok(L.wgu) || !ps_weight_ok(L.wdown)) return AB2_OK;
    }
    int dev = 0, coop = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return AB2_OK;
    const int nops_of_model = 1 + 5 * d.n_layers + 2;
    const size_t smem = ps_smem_bytes(nops_of_model);
    if (smem > 220 * 1024) return AB2_OK;  // too many blocks for the shared copy of the op list
    if (cudaFuncSetAttribute(decode_step_persistent_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(decode_step_persistent_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return AB2_OK;
    }
    int per_sm = 0;
    AB2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_persistent_kernel<true>, PS_THREADS, smem));
    if (per_sm < 1) return AB2_OK;
    const int grid = device_sm_count();
    if (d.n_kv_heads > grid) return AB2_OK;

    PersistentStep *ps = new PersistentStep();
    ps->desc = d;
    ps->grid = grid;
    ps->device = dev;
    ps->nsplit = std::max(1, std::min(16, grid / d.n_kv_heads));
    std::vector<PsOp> ops;
    auto gemv = [&](const ab2_qweight *w, const void *x, const float *norm_w, void *y, const void *resid, int epi) {
        PsOp o = {};
        o.kind = PS_GEMV; o.epi = epi; o.N = w->N; o.K = w->K;
        o.wt = (const uint32_t *)w->codes; o.x = (const __nv_bfloat16 *)x; o.norm_w = norm_w;
        o.y = (__nv_bfloat16 *)y; o.resid = (const __nv_bfloat16 *)resid;
        ops.push_back(o);
        ps->max_tiles = std::max(ps->max_tiles, (w->N + 15) / 16);
    };
    PsOp e = {};
    e.kind = PS_EMBED;
    ops.push_back(e);
    for (int l = 0; l < d.n_layers; ++l) {
        const PsLayerDesc &L = d.layers[l];
        gemv(L.wqkv, d.x, L.norm1, d.qkv, nullptr, W4_EPI_STORE);
        PsOp at = {};
        at.kind = PS_ATTN; at.layer = l;
        ops.push_back(at);
        gemv(L.wo, d.attn, nullptr, d.x, d.x, W4_EPI_ADD);
        gemv(L.wgu, d.x, L.norm2, d.hid, nullptr, W4_EPI_SWIGLU);
        gemv(L.wdown, d.hid, nullptr, d.x, d.x, W4_EPI_ADD);
    }
    gemv(d.lm_head, d.x, d.final_norm, nullptr, nullptr, W4_EPI_STORE);
    PsOp t = {};
    t.kind = PS_TAIL;
    ops.push_back(t);
    ps->nops = (int)ops.size();
    if ((ps->max_tiles + grid - 1) / grid > PS_LOCAL_TILES) {  // a CTA finishes its tiles through a fixed table
        delete ps;
        return AB2_OK;
    }

    const size_t parts = (size_t)d.n_kv_heads * ps->nsplit * rep;
    cudaError_t err = cudaMalloc((void **)&ps->ops_dev, ops.size() * sizeof(PsOp));
    if (err == cudaSuccess) err = cudaMemcpy(ps->ops_dev, ops.data(), ops.size() * sizeof(PsOp), cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = cudaMalloc((void **)&ps->apart_acc, parts * PS_HD * sizeof(float));
    if (err == cudaSuccess) err = cudaMalloc((void **)&ps->apart_ml, parts * 2 * sizeof(float));
    if (err == cudaSuccess) err = cudaMalloc((void **)&ps->acount, (size_t)d.n_kv_heads * sizeof(int));
    if (err == cudaSuccess) err = cudaMemset(ps->acount, 0, (size_t)d.n_kv_heads * sizeof(int));
    if (err == cudaSuccess) err = cudaMalloc((void **)&ps->trace, (size_t)3 * ops.size() * PS_TRACE * sizeof(unsigned long long));
    if (err == cudaSuccess) err = cudaMemset(ps->trace, 0, (size_t)3 * ops.size() * PS_TRACE * sizeof(unsigned long long));
    if (err == cudaSuccess) err = cudaMalloc((void **)&ps->bar, sizeof(unsigned int));
    if (err == cudaSuccess) err = cudaMemset(ps->bar, 0, sizeof(unsigned int));
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        persistent_step_destroy(ps);
        return fail(AB2_ERR_CUDA, "persistent decode step set-up failed: %s", cudaGetErrorString(err));
    }
    ps->recovery_epoch = device_recovery_epoch();
    *out = ps;
    return AB2_OK;
}

void persistent_step_destroy(PersistentStep *ps) {
    if (!ps) return;
    cudaFree(ps->ops_dev); cudaFree(ps->apart_acc); cudaFree(ps->apart_ml); cudaFree(ps->acount);
    cudaFree(ps->bar); cudaFree(ps->trace);
    delete ps;
}

int persistent_step_trace(const PersistentStep *ps, unsigned long long *out, int capacity, int *nphases) {
    AB2_REQUIRE(ps && out && nphases, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(ps->traced, AB2_ERR_UNSUPPORTED, "phase timestamps are recorded only when AB2_PS_TRACE is set in the environment");
    *nphases = ps->nops;
    AB2_REQUIRE(capacity >= 3 * ps->nops * PS_TRACE, AB2_ERR_CAPACITY, "the trace needs room for %d values", 3 * ps->nops * PS_TRACE);
    AB2_CUDA(cudaDeviceSynchronize());
    AB2_CUDA(cudaMemcpy(out, ps->trace, (size_t)3 * ps->nops * PS_TRACE * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return AB2_OK;
}

bool persistent_step_serves(const PersistentStep *ps, const ab2_kv *kv, int len_bound) {
    if (!ps || !kv) return false;
    const PsModelDesc &d = ps->desc;
    return kv->dtype == AB2_KV_INT8 && kv->hd == PS_HD && kv->kvh == d.n_kv_heads && kv->h == d.n_heads &&
           kv->L == d.n_layers && (len_bound + ps->nsplit - 1) / ps->nsplit + 1 <= PS_MAX_CTA_TOKENS;
}

int persistent_step_launch(PersistentStep *ps, ab2_kv *kv, const uint32_t *ids_dev, int row, void *logits_dev,
                           uint32_t *argmax_dev, cudaStream_t s) {
    const PsModelDesc &d = ps->desc;
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    if (ps->recovery_epoch != device_recovery_epoch()) {
        // a wait ran out in some earlier kernel on this device: counters may hold partial
        // counts; put them back to rest before the next step relies on them
        AB2_CUDA(cudaStreamSynchronize(s));
        AB2_CUDA(cudaMemset(ps->acount, 0, (size_t)d.n_kv_heads * sizeof(int)));
        AB2_CUDA(cudaMemcpy(ps->bar, &ps->bar_total, sizeof(unsigned int), cudaMemcpyHostToDevice));
        ps->recovery_epoch = device_recovery_epoch();
    }
    PsArgs a = {};
    a.ops = ps->ops_dev; a.nops = ps->nops;
    a.eps = d.eps; a.scale = (float)(1.0 / std::sqrt((double)d.head_dim));
    a.cos_t = d.cos_t; a.sin_t = d.sin_t;
    a.emb = (const uint32_t *)d.embedding->codes; a.emb_N = d.embedding->N; a.emb_K = d.embedding->K;
    a.ids = ids_dev;
    a.x = (__nv_bfloat16 *)d.x; a.qkv = (const __nv_bfloat16 *)d.qkv; a.attn = (__nv_bfloat16 *)d.attn;
    a.kv = kv_view(kv, 0);
    a.kv_layer_tokens = (size_t)kv->B * kv->kvh * kv->cap;
    a.row = row; a.h = d.n_heads; a.rep = d.n_heads / d.n_kv_heads; a.nsplit = ps->nsplit;
    a.apart_acc = ps->apart_acc; a.apart_ml = ps->apart_ml; a.acount = ps->acount;
    a.bar = ps->bar; a.bar_base = ps->bar_total;
    a.status = status;
    a.logits = (__nv_bfloat16 *)logits_dev; a.vocab = d.vocab; a.argmax_out = argmax_dev;
    a.trace = ps->trace;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ps->grid); cfg.blockDim = dim3(PS_THREADS);
    cfg.dynamicSmemBytes = ps_smem_bytes(ps->nops); cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    // AB2_PS_TRACE=1 runs the build of the kernel that records phase timestamps (ab2_model_step_trace)
    static const bool trace = getenv("AB2_PS_TRACE") != nullptr;
    ps->traced = trace;
    cudaError_t e = trace ? cudaLaunchKernelEx(&cfg, decode_step_persistent_kernel<true>, a)
                          : cudaLaunchKernelEx(&cfg, decode_step_persistent_kernel<false>, a);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(AB2_ERR_CUDA, "persistent decode step launch failed: %s", cudaGetErrorString(e));
    }
    ps->bar_total += (unsigned int)(ps->nops - 1) * (unsigned int)ps->grid;
    return AB2_OK;
}

}  // namespace ab2
