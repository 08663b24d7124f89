// W4A16 (group 128, bf16 activations) decode GEMM for 9..32 tokens per pass on the
// warp MMA, register-tiled: a warp multiplies a strip of 64 output rows (4 tiles
// of 16) by all tokens, so the activation fragments it loads serve four weight
// blocks and the codes of a block are unpacked once for every token.
//
// The 8 warps of a CTA are WS strips x WK slices of K (WS WK = 8): the WS warps of
// a slice walk the same groups of neighbouring strips and share one ring of
// activation stages, so a CTA reads the activations once per 64 WS rows.  Work is
// cut in units of (WS strips, quantisation group); the units, ordered
// [strips][group], are cut into one contiguous range per CTA, equal to within one
// unit.  A CTA walks its range strip set by strip set; the groups of a set that
// lie inside the range are shared out among the WK slices (contiguous shares), and
// the slices' sums are added through shared memory in slice order.  A strip set
// whose groups all lie inside one CTA is finished there; one cut by a range
// boundary goes through one f32 partial tile per contributing CTA and a counter
// in global memory: the last CTA to arrive adds the partial tiles in CTA order
// and stores.  Nobody waits on another CTA, and the sums do not depend on arrival
// order.
//
// Weights: every warp owns a ring of stages (one group of its strip each: 4
// blocks of 1088 bytes of the tile-major layout, w4a16_layout.cuh) filled by bulk
// asynchronous copies, lane t copying the block of tile t, completion on an
// mbarrier per stage; the codes go to registers at the start of a group, so the
// stage is refilled at once.
// Activations: a stage holds one group of every token in fragment order (the 16
// bytes of token r + 8t at k = 32c + 8i sit where lane (r, c) loads B operand i of
// token tile t).  Each warp of the slice copies its share of the tokens with
// cp.async, two whole 256-byte rows per instruction, and the copies' completion
// arrives on the stage's "full" mbarrier; a warp that has consumed a stage arrives
// on its "empty" mbarrier, and the stage is refilled one group later, so the
// warps of a slice may drift apart by a group.
//
// Arithmetic per block is that of gemv_w4a16_warp.cuh: 0x4300 | q == 128 + q as
// bf16, the zero point leaves by an exact bf16x2 add, mma.sync.m16n8k16 with f32
// accumulation over the group, the bf16 scale applied per group in f32.
//
// Every mbarrier wait is bounded; a wait that runs out records AB2_ERR_TIMEOUT,
// and the warp stops waiting but keeps taking part in the CTA's barriers, so the
// kernel still ends.
#pragma once

#include "gemv_w4a16_warp.cuh"

namespace ab2 {

constexpr int W4S_WSTAGES = 3;  // weight stages of a warp (one group of its strip each)
constexpr int W4S_XSTAGES = 3;  // activation stages of a slice (one group of every token each)
constexpr uint32_t W4S_BLOCK_BYTES = W4_BLOCK_WORDS * 4;

// Shape of a CTA: NT token tiles of 8, strips of RT tiles of 16 rows, WS strips x WK slices of K
// (one warp each).
template <int NT_, int RT_, int WS_, int WK_>
struct W4sShape {
    static constexpr int NT = NT_, RT = RT_, WS = WS_, WK = WK_, WARPS = WS_ * WK_, FRAGS = RT_ * NT_;
    static constexpr uint32_t WSTAGE = RT_ * W4S_BLOCK_BYTES;
    static constexpr uint32_t XSTAGE = NT_ * 2048;  // 4 B operands x NT token tiles x 32 lanes x 16 bytes
    // fragments (tile, token tile) of a strip that the other slices hand to the owning slice
    static constexpr uint32_t REDUCE = WS_ * RT_ * NT_ * (WK_ - 1) * 512;
    static constexpr size_t SMEM = (size_t)WARPS * W4S_WSTAGES * WSTAGE + (size_t)WK_ * W4S_XSTAGES * XSTAGE + REDUCE +
                                   (WARPS * W4S_WSTAGES + 2 * WK_ * W4S_XSTAGES) * 8 + 128;
    // f32 partial tiles of a strip set: WS strips x RT tiles x NT token tiles x 32 lanes x 4
    static constexpr int SLOT_FLOATS = WS_ * RT_ * NT_ * 128;
};
constexpr int W4S_MAX_SLOT_FLOATS = 8192;

// Walks the groups of one K slice of a CTA in the order its warps consume them: strip set by strip
// set, the slice's share of the groups of the set that lie inside the CTA's range [u0, u1).
// `g < ge` while a group is left.
template <int WK>
struct W4sCursor {
    int s, g, ge;
    __device__ __forceinline__ bool valid() const { return g < ge; }
    static __device__ __forceinline__ void share(int s, int u0, int u1, int G, int wk, int &a, int &b) {
        const int ga = max(u0 - s * G, 0), gb = min(u1 - s * G, G);
        const int n = gb - ga, base = n / WK, rem = n - base * WK;
        a = ga + wk * base + min(wk, rem);
        b = a + base + (wk < rem ? 1 : 0);
    }
    // first group at or after strip set `from`
    __device__ __forceinline__ void seek(int from, int u0, int u1, int G, int wk) {
        for (s = from; s * G < u1; ++s) {
            share(s, u0, u1, G, wk, g, ge);
            if (g < ge) return;
        }
        g = ge = 0;
    }
    __device__ __forceinline__ void next(int u0, int u1, int G, int wk) {
        if (++g < ge) return;
        seek(s + 1, u0, u1, G, wk);
    }
};

template <int EPI>
__device__ __forceinline__ void w4s_store_frag(const float (&v)[4], int tile, int tok0, int r, int c,
                                               __nv_bfloat16 *y, const __nv_bfloat16 *resid, int N, int M) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int tok = tok0 + 2 * c + i;
        if (tok >= M) continue;
        if (EPI == W4_EPI_SWIGLU) {
            // rows 0..7 of the tile are gate rows, rows 8..15 the matching up rows
            const int half_n = N >> 1, col = tile * 8 + r;
            if (col < half_n) {
                const float g = __bfloat162float(__float2bfloat16_rn(v[i]));
                const float u = __bfloat162float(__float2bfloat16_rn(v[2 + i]));
                y[(size_t)tok * half_n + col] = __float2bfloat16_rn(swiglu_value(g, u));
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = tile * 16 + r + 8 * h;
                if (row >= N) continue;
                float val = v[2 * h + i];
                const size_t o = (size_t)tok * N + row;
                if (EPI == W4_EPI_F32) {
                    reinterpret_cast<float *>(y)[o] = val;
                } else {
                    if (EPI == W4_EPI_ADD)  // residual + bf16(projection), as residual + x does
                        val = __bfloat162float(resid[o]) + __bfloat162float(__float2bfloat16_rn(val));
                    y[o] = __float2bfloat16_rn(val);
                }
            }
        }
    }
}

// partials: [gridDim.x][2][SLOT_FLOATS] floats; counters: one int per strip set, zero on entry and on exit.
template <class S, int EPI>
__global__ void __launch_bounds__(S::WARPS * 32, 1)
gemv_w4a16_strip_kernel(const uint32_t *__restrict__ wt, const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *y,
                        const __nv_bfloat16 *resid, int N, int K, int M, float *partials, int *counters,
                        int *status) {
    constexpr int NT = S::NT, RT = S::RT, WS = S::WS, WK = S::WK, FRAGS = S::FRAGS, WARPS = S::WARPS;
    constexpr int OWN = (FRAGS + WK - 1) / WK;  // fragments of a strip one slice finishes
    constexpr int TOK_PER_WARP = 8 * NT / WS;   // rows of a stage this warp copies (two per instruction)
    static_assert(TOK_PER_WARP >= 2 && TOK_PER_WARP % 2 == 0 && TOK_PER_WARP * WS == 8 * NT, "token rows are copied in pairs");
    constexpr uint32_t XSTAGE = S::XSTAGE, WSTAGE = S::WSTAGE;
    using Cursor = W4sCursor<WK>;
    extern __shared__ uint8_t w4s_smem_raw[];
    const uint32_t smem0 = (smem_addr(w4s_smem_raw) + 127u) & ~127u;
    __shared__ int last_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ws = warp % WS, wk = warp / WS;  // strip of the set, slice of K
    const int r = lane >> 2, c = lane & 3;
    const int G = K >> 7, tiles = (N + 15) >> 4;
    const int sets = (tiles + WS * RT - 1) / (WS * RT);
    const int total = sets * G;
    const int nc = (int)gridDim.x, cta = (int)blockIdx.x;
    const int base = total / nc, rem = total - base * nc;
    const int u0 = cta * base + min(cta, rem), u1 = u0 + base + (cta < rem ? 1 : 0);

    const uint32_t wring0 = smem0 + warp * (W4S_WSTAGES * WSTAGE);
    const uint32_t xring0 = smem0 + WARPS * (W4S_WSTAGES * WSTAGE) + wk * (W4S_XSTAGES * XSTAGE);
    const uint32_t red0 = smem0 + WARPS * (W4S_WSTAGES * WSTAGE) + WK * (W4S_XSTAGES * XSTAGE);
    const uint32_t bars = red0 + S::REDUCE;
    const uint32_t wbar0 = bars + warp * (W4S_WSTAGES * 8);
    const uint32_t xfull0 = bars + WARPS * W4S_WSTAGES * 8 + wk * (W4S_XSTAGES * 8);
    const uint32_t xempty0 = xfull0 + WK * W4S_XSTAGES * 8;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < W4S_WSTAGES; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(wbar0 + s * 8));
        if (ws == 0) {
#pragma unroll
            for (int s = 0; s < W4S_XSTAGES; ++s) {
                // full: every lane of the slice's warps arrives when its copies have landed; empty: one arrival per warp
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(xfull0 + s * 8), "n"(WS * 32));
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(xempty0 + s * 8), "n"(WS));
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    const int tile0 = ws * RT;  // first tile of this warp's strip inside a set
    // one group of this warp's strip into a weight stage: lane 0 arms the barrier for the blocks
    // that exist, lane t copies tile t's
    // `after` is a value the copies must wait for: it enters their source address masked with a zero the
    // compiler cannot see (K is a multiple of 128), so the copies cannot be issued before it is known.
    const uint32_t hidden_zero = (uint32_t)K & 1u;
    auto fetch_w = [&](const Cursor &cu, uint32_t stage, uint32_t bar, uint32_t after) {
        const int t0 = cu.s * (WS * RT) + tile0;
        const int nv = max(0, min(RT, tiles - t0));
        const uint32_t go = (cu.valid() && nv > 0) ? 1u : 0u;
        const uint32_t arm = go & (lane == 0 ? 1u : 0u), copy = go & (lane < nv ? 1u : 0u);
        const uint32_t *src = wt + ((size_t)(t0 + lane) * G + cu.g) * W4_BLOCK_WORDS + (after & hidden_zero);
        asm volatile(
            "{\n"
            " .reg .pred p, q;\n"
            " setp.ne.u32 p, %0, 0;\n"
            " setp.ne.u32 q, %1, 0;\n"
            " @p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%5], %4;\n"
            " @q cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%2], [%3], %6, [%5];\n"
            "}\n" ::"r"(arm),
            "r"(copy), "r"(stage + (uint32_t)lane * W4S_BLOCK_BYTES), "l"(src), "r"((uint32_t)nv * W4S_BLOCK_BYTES),
            "r"(bar), "n"(W4S_BLOCK_BYTES)
            : "memory");
    };

    const int s_first = u0 / G, s_last = (u1 - 1) / G;
    // the weights are constant: the first stages are in flight before the preceding kernel has finished
    Cursor wcur;
    wcur.seek(s_first, u0, u1, G, wk);
#pragma unroll
    for (int j = 0; j < W4S_WSTAGES; ++j) {
        fetch_w(wcur, wring0 + j * WSTAGE, wbar0 + j * 8, 0u);
        if (wcur.valid()) wcur.next(u0, u1, G, wk);
    }

    // activations (and the residual) come from the preceding kernel
    pdl_wait();
    pdl_launch_dependents();

    // This warp's share of an activation stage: rows ws TOK_PER_WARP .. of the token tile set, two
    // rows of 256 bytes per instruction (lane: row lane / 16, 16-byte piece lane % 16).  Piece p of
    // a row holds k = 8p ..: it is B operand p % 4 of lane column p / 4.
    const int xpiece = lane & 15;
    const __nv_bfloat16 *xsrc[TOK_PER_WARP / 2];
    uint32_t xdst[TOK_PER_WARP / 2], xbytes[TOK_PER_WARP / 2];  // rows past the last token are filled with zeros
#pragma unroll
    for (int j = 0; j < TOK_PER_WARP / 2; ++j) {
        const int tok = ws * TOK_PER_WARP + 2 * j + (lane >> 4);
        xbytes[j] = tok < M ? 16u : 0u;
        xsrc[j] = x + (size_t)min(tok, M - 1) * K + xpiece * 8;
        xdst[j] = (uint32_t)((xpiece & 3) * (NT * 512) + (tok >> 3) * 512 + ((tok & 7) * 4 + (xpiece >> 2)) * 16);
    }
    Cursor xcur;
    xcur.seek(s_first, u0, u1, G, wk);
    auto fetch_x = [&](uint32_t stage, uint32_t full) {
        if (xcur.valid()) {
#pragma unroll
            for (int j = 0; j < TOK_PER_WARP / 2; ++j)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(stage + xdst[j]),
                             "l"(xsrc[j] + xcur.g * 128), "r"(xbytes[j])
                             : "memory");
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(full) : "memory");
            xcur.next(u0, u1, G, wk);
        }
    };
#pragma unroll
    for (int j = 0; j < W4S_XSTAGES; ++j) fetch_x(xring0 + j * XSTAGE, xfull0 + j * 8);

    // Opaque register copies of the two constants of the nibble extraction.
    uint32_t k_mask = 0x000F000Fu, k_magic = 0x43004300u;
    asm volatile("" : "+r"(k_mask), "+r"(k_magic));

    const uint32_t code_off = (r * 16 + c * 4) * 4;  // this thread's 4 words of row r in a block
    const uint32_t param_off = (256 + r) * 4;
    uint32_t wstage = wring0, wbar = wbar0, wparity = 0;
    const uint32_t wring_end = wring0 + W4S_WSTAGES * WSTAGE;
    // activation stage of the group being consumed, and of the one consumed before it (refilled now)
    int xs = 0, xs_prev = W4S_XSTAGES - 1;
    uint32_t xparity = 0, xparity_prev = 0;
    bool first_group = true;
    bool dead = false;  // a wait ran out: stop waiting, finish the walk

    for (int s = s_first; s <= s_last; ++s) {
        int ga, gb;
        Cursor::share(s, u0, u1, G, wk, ga, gb);
        const bool has_w = s * (WS * RT) + tile0 < tiles;  // the last set may have fewer strips
        float acc[RT][NT][4];
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[rt][t][i] = 0.f;

        for (int g = ga; g < gb; ++g) {
            uint32_t wa[RT][4], wb[RT][4], pa[RT], pb[RT];
            if (has_w) {
                if (!dead && !mbar_wait_addr(wbar, wparity)) {
                    if (lane == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
                    dead = true;
                }
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    const uint4 va = lds128(wstage + rt * W4S_BLOCK_BYTES + code_off);
                    const uint4 vb = lds128(wstage + rt * W4S_BLOCK_BYTES + code_off + 512);
                    wa[rt][0] = va.x; wa[rt][1] = va.y; wa[rt][2] = va.z; wa[rt][3] = va.w;
                    wb[rt][0] = vb.x; wb[rt][1] = vb.y; wb[rt][2] = vb.z; wb[rt][3] = vb.w;
                    pa[rt] = lds32(wstage + rt * W4S_BLOCK_BYTES + param_off);
                    pb[rt] = lds32(wstage + rt * W4S_BLOCK_BYTES + param_off + 32);
                }
                // The stage takes the group W4S_WSTAGES ahead once every lane HOLDS its words.  The loads above
                // have only been issued (a shared-memory load can wait behind other traffic for longer than a
                // bulk copy out of L2 takes to land), so the refill is made to wait for one word of every load:
                // a 16-byte load completes as a whole.
                uint32_t held = 0;
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) held ^= wa[rt][0] ^ wb[rt][0] ^ pa[rt] ^ pb[rt];
                __syncwarp();
                fetch_w(wcur, wstage, wbar, held);
                wstage += WSTAGE;
                wbar += 8;
                if (wstage == wring_end) { wstage = wring0; wbar = wbar0; wparity ^= 1; }
            } else {
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) wa[rt][i] = wb[rt][i] = 0u;
                    pa[rt] = pb[rt] = 0u;
                }
            }
            if (wcur.valid()) wcur.next(u0, u1, G, wk);
            uint32_t nza[RT], nzb[RT];  // -(128 + zero point) of rows r and r + 8 in both halves
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                nza[rt] = __byte_perm(pa[rt], pa[rt], 0x3232);
                nzb[rt] = __byte_perm(pb[rt], pb[rt], 0x3232);
            }

            // The stage consumed one group ago is refilled with the group W4S_XSTAGES - 1 ahead, once
            // every warp of the slice has left it.
            if (!first_group) {
                if (xcur.valid() && !dead && !mbar_wait_addr(xempty0 + xs_prev * 8, xparity_prev)) {
                    if (lane == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
                    dead = true;
                }
                fetch_x(xring0 + xs_prev * XSTAGE, xfull0 + xs_prev * 8);
            }
            first_group = false;

            if (!dead && !mbar_wait_addr(xfull0 + xs * 8, xparity)) {
                if (lane == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
                dead = true;
            }
            const uint32_t xstage = xring0 + xs * XSTAGE;
            float d[RT][NT][4];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                uint4 xw[NT];
#pragma unroll
                for (int t = 0; t < NT; ++t) xw[t] = lds128(xstage + wi * (NT * 512) + t * 512 + lane * 16);
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    uint32_t a[8];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        // the zero point leaves by an exact bf16x2 add: (128 + q) - (128 + z)
                        a[2 * jj] = bf16x2_add(w4_pair_bf16(wa[rt][wi], jj, k_mask, k_magic), nza[rt]);
                        a[2 * jj + 1] = bf16x2_add(w4_pair_bf16(wb[rt][wi], jj, k_mask, k_magic), nzb[rt]);
                    }
                    // the two K steps of a token tile depend on each other: all token tiles of one step first
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        if (wi == 0)
                            mma_bf16_16816_init(d[rt][t], a[0], a[1], a[2], a[3], xw[t].x, xw[t].y);
                        else
                            mma_bf16_16816(d[rt][t], a[0], a[1], a[2], a[3], xw[t].x, xw[t].y);
                    }
#pragma unroll
                    for (int t = 0; t < NT; ++t) mma_bf16_16816(d[rt][t], a[4], a[5], a[6], a[7], xw[t].z, xw[t].w);
                }
            }
            // The stage is handed back once every load of it has returned: the address of the arrival takes
            // in the sums that the last loads of every token tile have fed (masked with the hidden zero).
            uint32_t xheld = 0;
#pragma unroll
            for (int t = 0; t < NT; ++t) xheld ^= __float_as_uint(d[RT - 1][t][0]);
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(xempty0 + xs * 8 + (xheld & hidden_zero)) : "memory");
            xs_prev = xs;
            xparity_prev = xparity;
            if (++xs == W4S_XSTAGES) { xs = 0; xparity ^= 1; }

#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                const float sa = __uint_as_float(pa[rt] << 16), sb = __uint_as_float(pb[rt] << 16);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    acc[rt][t][0] = fmaf(sa, d[rt][t][0], acc[rt][t][0]);
                    acc[rt][t][1] = fmaf(sa, d[rt][t][1], acc[rt][t][1]);
                    acc[rt][t][2] = fmaf(sb, d[rt][t][2], acc[rt][t][2]);
                    acc[rt][t][3] = fmaf(sb, d[rt][t][3], acc[rt][t][3]);
                }
            }
        }

        // ---- the set's groups inside this CTA are done: add the slices' sums in slice order ----
        // Fragment e of a strip is finished by slice e % WK; the other slices hand theirs over.
        const bool whole = u0 <= s * G && (s + 1) * G <= u1;
        // contributors of a cut set: the CTAs whose ranges meet [s G, s G + G)
        const int cut = rem * (base + 1);
        const int first_u = s * G, last_u = first_u + G - 1;
        const int c_first = first_u < cut ? first_u / (base + 1) : rem + (first_u - cut) / base;
        const int c_last = last_u < cut ? last_u / (base + 1) : rem + (last_u - cut) / base;
        // a CTA has at most two cut sets: the one its range starts inside (slot 0) and the one its
        // range ends inside (slot 1)
        float *mine = partials + ((size_t)cta * 2 + (cta == c_first ? 1 : 0)) * S::SLOT_FLOATS +
                      (size_t)ws * FRAGS * 128;
        float sum[OWN][4];
        if (WK > 1) {
            __syncthreads();  // the hand-over buffer is free
#pragma unroll
            for (int e = 0; e < FRAGS; ++e) {
                const int owner = e % WK;
                if (wk != owner) {
                    const int pos = wk < owner ? wk : wk - 1;
                    const float *v = acc[e / NT][e % NT];
                    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(
                                     red0 + (((ws * FRAGS + e) * (WK - 1) + pos) * 32 + lane) * 16),
                                 "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
                                 : "memory");
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int e = 0; e < FRAGS; ++e) {
            if (e % WK != wk) continue;
            float *o = sum[e / WK];
            o[0] = o[1] = o[2] = o[3] = 0.f;
#pragma unroll
            for (int k = 0; k < WK; ++k) {
                float4 v;
                if (k == wk) {
                    v = make_float4(acc[e / NT][e % NT][0], acc[e / NT][e % NT][1], acc[e / NT][e % NT][2],
                                    acc[e / NT][e % NT][3]);
                } else {
                    const int pos = k < wk ? k : k - 1;
                    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                                 : "r"(red0 + (((ws * FRAGS + e) * (WK - 1) + pos) * 32 + lane) * 16));
                }
                o[0] += v.x; o[1] += v.y; o[2] += v.z; o[3] += v.w;
            }
            if (whole)
                w4s_store_frag<EPI>(sum[e / WK], s * (WS * RT) + tile0 + e / NT, 8 * (e % NT), r, c, y, resid, N, M);
            else
                *reinterpret_cast<float4 *>(mine + (e * 32 + lane) * 4) = make_float4(o[0], o[1], o[2], o[3]);
        }
        if (!whole) {
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) last_flag = atomicAdd(&counters[s], 1) == c_last - c_first ? 1 : 0;
            __syncthreads();
            if (last_flag) {
                __threadfence();
                // the partial tiles of every contributor, in CTA order; the loads of a few CTAs are in flight together
                float t4[OWN][4];
#pragma unroll
                for (int o = 0; o < OWN; ++o) t4[o][0] = t4[o][1] = t4[o][2] = t4[o][3] = 0.f;
#pragma unroll 4
                for (int cc = c_first; cc <= c_last; ++cc) {
                    const float *p = partials + ((size_t)cc * 2 + (cc == c_first ? 1 : 0)) * S::SLOT_FLOATS +
                                     (size_t)ws * FRAGS * 128 + lane * 4;
#pragma unroll
                    for (int e = 0; e < FRAGS; ++e) {
                        if (e % WK != wk) continue;
                        const float4 v = __ldcg(reinterpret_cast<const float4 *>(p + e * 128));
                        t4[e / WK][0] += v.x; t4[e / WK][1] += v.y; t4[e / WK][2] += v.z; t4[e / WK][3] += v.w;
                    }
                }
#pragma unroll
                for (int e = 0; e < FRAGS; ++e) {
                    if (e % WK != wk) continue;
                    w4s_store_frag<EPI>(t4[e / WK], s * (WS * RT) + tile0 + e / NT, 8 * (e % NT), r, c, y, resid, N, M);
                }
                if (threadIdx.x == 0) counters[s] = 0;
            }
        }
    }
    asm volatile("cp.async.wait_all;\n" ::: "memory");
}

}  // namespace ab2
