// INT8-KV flash-decode attention on the warp-level tensor cores (head_dim 128,
// up to 8 query heads per kv head): the throughput path for long contexts and
// large batches, where the CUDA-core kernel is bound by int8 -> float conversion
// rather than by HBM.
//
// Per 16 cached tokens a warp issues 16 MMAs for Q.K^T (A = the group's query
// heads as the 16 rows, constant in registers; B = K^T straight from the 128-byte
// token rows) and 8 MMAs for P.V (A = V^T obtained from the natural [token][d]
// rows with ldmatrix.trans on byte pairs; B = P^T, which is exactly the score
// fragment the first MMA left in this thread's registers).  int8 codes become
// fp16 by one byte-permute each (0x6400 | (code ^ 0x80) = 1152 + code, exact)
// and one exact fp16 subtraction of 1152 on the otherwise idle FMA pipe; the
// per-token K scale multiplies the f32 score, the per-token V scale is folded
// into P.  Accumulation is f32; softmax is the same online form as the reference
// (crates/aarambh-studio-kernel/src/cpu/parallel_attn.rs:189-234), in blocks of
// 16 keys.  Context splits are merged by the log-sum-exp kernel of attention.cu.
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "kv_cache.cuh"

using namespace ab2;

namespace ab2 {
namespace {

struct MmaAttnArgs {
    KvView kv;
    const void *q;  // head (row, head) at row * q_stride + head * 128
    long long q_stride;
    int row0, h, rep, nsplit, dtype;
    int pending;    // appended, not yet committed tokens per row: they are attended too
    float scale;
    float *part_acc, *part_ml;
    void *out;      // used when nsplit == 1
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t f16x2_sub1152(uint32_t v) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(v), "r"(0xE480E480u));  // + (-1152, -1152)
    return d;
}
// bytes i and j of the sign-flipped word as fp16x2 (code_i, code_j), exact
template <int I, int J>
__device__ __forceinline__ uint32_t i8_pair_f16(uint32_t flipped) {
    return f16x2_sub1152(__byte_perm(flipped, 0x64646464u, (4 << 12) | (J << 8) | (4 << 4) | I));
}
__device__ __forceinline__ float q_as_f32(const void *p, int dtype, size_t i) {
    if (dtype == AB2_F32) return ((const float *)p)[i];
    if (dtype == AB2_F16) return __half2float(((const __half *)p)[i]);
    return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void st_out(void *p, int dtype, size_t i, float v) {
    if (dtype == AB2_F32) ((float *)p)[i] = v;
    else if (dtype == AB2_F16) ((__half *)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
}

// grid (nsplit, kv heads, rows), 128 threads; head_dim 128, INT8 cache.
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(MmaAttnArgs a) {
    constexpr int HD = 128;
    __shared__ alignas(128) uint8_t vst[4][2][16 * HD];  // per warp, double-buffered V block (swizzled 16-byte chunks)
    __shared__ float wm[4][8], wl[4][8];
    __shared__ float wacc[4][8][HD];
    pdl_wait();  // inputs come from the preceding kernel of the step
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int split = blockIdx.x, kvhead = blockIdx.y, rrow = blockIdx.z, row = kv_row(a.kv, a.row0, rrow);
    const int len = a.kv.lens[row] + a.pending;
    int per = (len + a.nsplit - 1) / a.nsplit;
    per = (per + 63) & ~63;  // whole 16-token blocks for each of the four warps
    const int t0 = split * per, t1 = min(len, t0 + per);
    const size_t head_base = ((size_t)row * a.kv.kvh + kvhead) * a.kv.cap;
    const int8_t *kbase = (const int8_t *)a.kv.k + head_base * HD;
    const int8_t *vbase = (const int8_t *)a.kv.v + head_base * HD;
    const float *ksc = a.kv.ks + head_base, *vsc = a.kv.vs + head_base;

    // ---- Q fragments (A operand): row g = query head g of the group; k-step s
    // covers d = c*32 + 4s + {0,1} (a0) and {2,3} (a2).  Rows >= rep are zero.
    uint32_t qa0[8], qa2[8];
    {
        const size_t qb = (size_t)rrow * a.q_stride + ((size_t)kvhead * a.rep + g) * HD + c * 32;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
            if (g < a.rep) {
                v0 = q_as_f32(a.q, a.dtype, qb + 4 * s); v1 = q_as_f32(a.q, a.dtype, qb + 4 * s + 1);
                v2 = q_as_f32(a.q, a.dtype, qb + 4 * s + 2); v3 = q_as_f32(a.q, a.dtype, qb + 4 * s + 3);
            }
            qa0[s] = pack_f16(v0, v1);
            qa2[s] = pack_f16(v2, v3);
        }
    }

    float m_run = -INFINITY, l_run = 0.f;  // of head g (replicated over c)
    float o[8][4];                          // [d chunk][fragment]: rows d, columns heads 2c, 2c+1
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    auto stage_v = [&](int base, int buf) {
        // 16 tokens x 128 bytes; chunk (token, ch) lands at token*128 + ((ch ^ (token & 7)) << 4)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = lane + 32 * i, tok = idx >> 3, ch = idx & 7;
            const int src_tok = min(base + tok, t1 - 1);
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&vst[warp][buf][tok * HD + ((ch ^ (tok & 7)) << 4)]);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(vbase + (size_t)src_tok * HD + ch * 16));
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    auto load_k = [&](int base, uint4 (&kr)[4], float (&sc)[8]) {
        // n-tile nt: token base + nt*8 + g, this thread's 32 bytes d = c*32 .. c*32+31
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int tok = min(base + nt * 8 + g, t1 - 1);
            const uint4 *p = reinterpret_cast<const uint4 *>(kbase + (size_t)tok * HD + c * 32);
            kr[2 * nt] = p[0];
            kr[2 * nt + 1] = p[1];
        }
        // scales of the tokens this thread's score / probability columns belong to
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = min(base + nt * 8 + 2 * c + e, t1 - 1);
                sc[nt * 2 + e] = ksc[tok];
                sc[4 + nt * 2 + e] = vsc[tok];
            }
    };

    int buf = 0;
    const int first = t0 + warp * 16;
    uint4 kr[4];
    float sc[8];
    if (first < t1) { stage_v(first, 0); load_k(first, kr, sc); }

    for (int base = first; base < t1; base += 64) {
        // prefetch the next block of this warp
        uint4 kr_n[4];
        float sc_n[8];
        const int nxt = base + 64;
        if (nxt < t1) { stage_v(nxt, buf ^ 1); load_k(nxt, kr_n, sc_n); }

        // ---- S = Q.K^T for two 8-token tiles
        float s_frag[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s_frag[nt][j] = 0.f;
            const uint32_t w[8] = {kr[2 * nt].x ^ 0x80808080u, kr[2 * nt].y ^ 0x80808080u, kr[2 * nt].z ^ 0x80808080u,
                                   kr[2 * nt].w ^ 0x80808080u, kr[2 * nt + 1].x ^ 0x80808080u, kr[2 * nt + 1].y ^ 0x80808080u,
                                   kr[2 * nt + 1].z ^ 0x80808080u, kr[2 * nt + 1].w ^ 0x80808080u};
#pragma unroll
            for (int s = 0; s < 8; ++s)
                mma_f16_16816(s_frag[nt], qa0[s], 0u, qa2[s], 0u, i8_pair_f16<0, 1>(w[s]), i8_pair_f16<2, 3>(w[s]));
        }
        // ---- online softmax for head g over the 16 tokens (this thread: tokens nt*8 + 2c + e)
        float sv[4];
        float bm = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool valid = base + nt * 8 + 2 * c + e < t1;
                sv[nt * 2 + e] = valid ? s_frag[nt][e] * sc[nt * 2 + e] * a.scale : -INFINITY;
                bm = fmaxf(bm, sv[nt * 2 + e]);
            }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        const float m_new = fmaxf(m_run, bm);
        const float corr = expf(m_run - m_new);
        float pv[4], psum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            pv[i] = expf(sv[i] - m_new);  // exp(-inf) = 0 for tokens past the end
            psum += pv[i];
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l_run = l_run * corr + psum;
        m_run = m_new;
        // P^T fragments (B operand of P.V): probabilities times the V scale of their token
        const uint32_t pb0 = pack_f16(pv[0] * sc[4], pv[1] * sc[5]);
        const uint32_t pb1 = pack_f16(pv[2] * sc[6], pv[3] * sc[7]);
        // rescale factors of the heads this thread's output columns belong to
        const float c0 = __shfl_sync(0xffffffffu, corr, (2 * c) * 4), c1 = __shfl_sync(0xffffffffu, corr, (2 * c + 1) * 4);

        // ---- O += V^T . P^T  (V block staged in shared memory)
        if (nxt < t1) asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncwarp();
        const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(&vst[warp][buf][0]);
        // ldmatrix x4.trans: matrices (tokens 0-7, chunk dc), (8-15, dc), (0-7, dc+1), (8-15, dc+1)
        const int lm = lane >> 3, lr = lane & 7, ltok = (lm & 1) * 8 + lr;
#pragma unroll
        for (int dp = 0; dp < 4; ++dp) {
            const int ch = 2 * dp + (lm >> 1);
            const uint32_t addr = vs_base + ltok * HD + ((ch ^ (ltok & 7)) << 4);
            uint32_t r0, r1, r2, r3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
            r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
                const uint32_t lo = hc ? r2 : r0, hi = hc ? r3 : r1;  // tokens 0-7 / 8-15 of chunk 2*dp + hc
                float (&acc)[4] = o[2 * dp + hc];
                acc[0] *= c0; acc[1] *= c1; acc[2] *= c0; acc[3] *= c1;
                // rows g: d = chunk*16 + 2g (bytes 0, 2); rows g+8: d + 1 (bytes 1, 3)
                mma_f16_16816(acc, i8_pair_f16<0, 2>(lo), i8_pair_f16<1, 3>(lo), i8_pair_f16<0, 2>(hi), i8_pair_f16<1, 3>(hi), pb0, pb1);
            }
        }
        __syncwarp();
        if (nxt < t1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) kr[i] = kr_n[i];
#pragma unroll
            for (int i = 0; i < 8; ++i) sc[i] = sc_n[i];
        }
        buf ^= 1;
    }

    // ---- merge the four warps
    if (c == 0 && g < 8) { wm[warp][g] = m_run; wl[warp][g] = l_run; }
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        const int d = ch * 16 + 2 * g;
        if (2 * c < 8) { wacc[warp][2 * c][d] = o[ch][0]; wacc[warp][2 * c][d + 1] = o[ch][2]; }
        if (2 * c + 1 < 8) { wacc[warp][2 * c + 1][d] = o[ch][1]; wacc[warp][2 * c + 1][d + 1] = o[ch][3]; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.rep * HD; i += 128) {
        const int hh = i / HD, d = i % HD;
        const float M = fmaxf(fmaxf(wm[0][hh], wm[1][hh]), fmaxf(wm[2][hh], wm[3][hh]));
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float e = (wm[w][hh] == -INFINITY) ? 0.f : expf(wm[w][hh] - M);
            L += e * wl[w][hh];
            A += e * wacc[w][hh][d];
        }
        const int head = kvhead * a.rep + hh;
        if (a.nsplit == 1) {
            st_out(a.out, a.dtype, ((size_t)rrow * a.h + head) * HD + d, L > 0.f ? A * (1.0f / L) : A);
        } else {
            const size_t pi = ((size_t)row * a.h + head) * a.nsplit + split;
            a.part_acc[pi * HD + d] = A;
            if (d == 0) { a.part_ml[pi * 2] = M; a.part_ml[pi * 2 + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------
// Causal attention of S new queries per sequence over the INT8 cache (prefill
// chunks, speculative verification): GroupedQueryAttention::forward at S > 1
// (crates/aarambh-studio-nn/src/attention.rs:170-226) with the causal cut of
// dispatch.rs:145-160 (query i sees keys up to kv_len - q_len + i).
//
// Same tensor-core arithmetic as the decode kernel above with the roles of the
// MMA rows changed: a warp owns 16 consecutive queries of ONE query head (the A
// rows of Q.K^T), walks the keys 16 at a time up to the causal limit of its last
// query, keeps the online softmax of its 16 rows in registers and accumulates
// O^T = V^T . P^T for queries 0-7 and 8-15 with the same V^T fragments.  The warps
// of a CTA are the query heads of one KV head on the same 16 queries, so the K
// rows and V blocks they fetch are the same bytes (cache hits after the first).
// No cross-warp merge and no context split: every (head, query tile) is a warp.
// ---------------------------------------------------------------------------
struct PrefillAttnArgs {
    KvView kv;
    const void *q;
    void *out;
    AttnStrides st;
    int S, pending, row0, rep, dtype;
    float scale;
};

__global__ void __launch_bounds__(128) attn_prefill_mma_kernel(PrefillAttnArgs a) {
    constexpr int HD = 128;
    __shared__ alignas(128) uint8_t vst[4][2][16 * HD];  // per warp, double-buffered V block (swizzled 16-byte chunks)
    pdl_wait();
    pdl_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    if (warp >= a.rep) return;  // no barrier below: a spare warp may leave
    const int qt = blockIdx.x, kvhead = blockIdx.y, rrow = blockIdx.z, row = kv_row(a.kv, a.row0, rrow);
    const int head = kvhead * a.rep + warp;
    const int q_lo = qt * 16;
    // keys visible to query i: [0, first + i]; first = cached + appended - S
    const int first = a.kv.lens[row] + a.pending - a.S;
    const int kmax = first + min(a.S, q_lo + 16);  // keys the tile's last query sees
    const size_t head_base = ((size_t)row * a.kv.kvh + kvhead) * a.kv.cap;
    const int8_t *kbase = (const int8_t *)a.kv.k + head_base * HD;
    const int8_t *vbase = (const int8_t *)a.kv.v + head_base * HD;
    const float *ksc = a.kv.ks + head_base, *vsc = a.kv.vs + head_base;

    // ---- Q fragments: rows g and g + 8 = queries q_lo + g, q_lo + g + 8; k-step s covers
    // d = c*32 + 4s + {0,1} (a0 / a1) and {2,3} (a2 / a3)
    uint32_t qa0[8], qa1[8], qa2[8], qa3[8];
    {
        const int qa = q_lo + g, qb = q_lo + g + 8;
        const size_t ba = (size_t)((long long)rrow * a.st.q_b + (long long)qa * a.st.q_s + (long long)head * a.st.q_h) + c * 32;
        const size_t bb = (size_t)((long long)rrow * a.st.q_b + (long long)qb * a.st.q_s + (long long)head * a.st.q_h) + c * 32;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (qa < a.S)
                for (int j = 0; j < 4; ++j) v[j] = q_as_f32(a.q, a.dtype, ba + 4 * s + j);
            if (qb < a.S)
                for (int j = 0; j < 4; ++j) v[4 + j] = q_as_f32(a.q, a.dtype, bb + 4 * s + j);
            qa0[s] = pack_f16(v[0], v[1]); qa2[s] = pack_f16(v[2], v[3]);
            qa1[s] = pack_f16(v[4], v[5]); qa3[s] = pack_f16(v[6], v[7]);
        }
    }
    const int end_a = first + q_lo + g + 1, end_b = end_a + 8;  // exclusive key limits of this thread's two rows

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[8][2][4];  // [d chunk][queries 0-7 / 8-15][fragment]: rows d, d + 1; columns queries 2c, 2c + 1
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
            for (int j = 0; j < 4; ++j) o[i][h2][j] = 0.f;

    auto stage_v = [&](int base, int buf) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = lane + 32 * i, tok = idx >> 3, ch = idx & 7;
            const int src_tok = min(base + tok, kmax - 1);
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&vst[warp][buf][tok * HD + ((ch ^ (tok & 7)) << 4)]);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(vbase + (size_t)src_tok * HD + ch * 16));
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    auto load_k = [&](int base, uint4 (&kr)[4], float (&sc)[8]) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int tok = min(base + nt * 8 + g, kmax - 1);
            const uint4 *p = reinterpret_cast<const uint4 *>(kbase + (size_t)tok * HD + c * 32);
            kr[2 * nt] = p[0];
            kr[2 * nt + 1] = p[1];
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int tok = min(base + nt * 8 + 2 * c + e, kmax - 1);
                sc[nt * 2 + e] = ksc[tok];
                sc[4 + nt * 2 + e] = vsc[tok];
            }
    };

    int buf = 0;
    uint4 kr[4];
    float sc[8];
    if (kmax > 0) { stage_v(0, 0); load_k(0, kr, sc); }
    for (int base = 0; base < kmax; base += 16) {
        uint4 kr_n[4];
        float sc_n[8];
        const int nxt = base + 16;
        if (nxt < kmax) { stage_v(nxt, buf ^ 1); load_k(nxt, kr_n, sc_n); }

        // ---- S = Q.K^T for two 8-token tiles (rows g: fragments 0,1; rows g + 8: fragments 2,3)
        float s_frag[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s_frag[nt][j] = 0.f;
            const uint32_t w[8] = {kr[2 * nt].x ^ 0x80808080u, kr[2 * nt].y ^ 0x80808080u, kr[2 * nt].z ^ 0x80808080u,
                                   kr[2 * nt].w ^ 0x80808080u, kr[2 * nt + 1].x ^ 0x80808080u, kr[2 * nt + 1].y ^ 0x80808080u,
                                   kr[2 * nt + 1].z ^ 0x80808080u, kr[2 * nt + 1].w ^ 0x80808080u};
#pragma unroll
            for (int s = 0; s < 8; ++s)
                mma_f16_16816(s_frag[nt], qa0[s], qa1[s], qa2[s], qa3[s], i8_pair_f16<0, 1>(w[s]), i8_pair_f16<2, 3>(w[s]));
        }
        // ---- online softmax of rows g and g + 8 over the 16 tokens (causal: token < row limit)
        float pv[2][4], corr[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int lim = h2 ? end_b : end_a;
            float sv[4], bm = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const bool valid = base + nt * 8 + 2 * c + e < lim;
                    sv[nt * 2 + e] = valid ? s_frag[nt][2 * h2 + e] * sc[nt * 2 + e] * a.scale : -INFINITY;
                    bm = fmaxf(bm, sv[nt * 2 + e]);
                }
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
            const float m_new = fmaxf(m_run[h2], bm);
            // a row with no visible key yet keeps m = -inf; exp(-inf - -inf) must not become NaN
            corr[h2] = m_new == -INFINITY ? 1.f : expf(m_run[h2] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pv[h2][i] = m_new == -INFINITY ? 0.f : expf(sv[i] - m_new);
                psum += pv[h2][i];
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l_run[h2] = l_run[h2] * corr[h2] + psum;
            m_run[h2] = m_new;
        }
        // P^T fragments (B operand of P.V) for queries 0-7 and 8-15, times the V scale of their token
        uint32_t pb0[2], pb1[2];
        float c0[2], c1[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            pb0[h2] = pack_f16(pv[h2][0] * sc[4], pv[h2][1] * sc[5]);
            pb1[h2] = pack_f16(pv[h2][2] * sc[6], pv[h2][3] * sc[7]);
            // rescale factors of the queries this thread's output columns belong to (rows 2c, 2c + 1 of the half)
            c0[h2] = __shfl_sync(0xffffffffu, corr[h2], (2 * c) * 4);
            c1[h2] = __shfl_sync(0xffffffffu, corr[h2], (2 * c + 1) * 4);
        }

        // ---- O^T += V^T . P^T  (V block staged in shared memory)
        if (nxt < kmax) asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncwarp();
        const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(&vst[warp][buf][0]);
        const int lm = lane >> 3, lr = lane & 7, ltok = (lm & 1) * 8 + lr;
#pragma unroll
        for (int dp = 0; dp < 4; ++dp) {
            const int ch = 2 * dp + (lm >> 1);
            const uint32_t addr = vs_base + ltok * HD + ((ch ^ (ltok & 7)) << 4);
            uint32_t r0, r1, r2, r3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
            r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
                const uint32_t lo = hc ? r2 : r0, hi = hc ? r3 : r1;
                const uint32_t va0 = i8_pair_f16<0, 2>(lo), va1 = i8_pair_f16<1, 3>(lo), va2 = i8_pair_f16<0, 2>(hi), va3 = i8_pair_f16<1, 3>(hi);
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    float (&acc)[4] = o[2 * dp + hc][h2];
                    acc[0] *= c0[h2]; acc[1] *= c1[h2]; acc[2] *= c0[h2]; acc[3] *= c1[h2];
                    mma_f16_16816(acc, va0, va1, va2, va3, pb0[h2], pb1[h2]);
                }
            }
        }
        __syncwarp();
        if (nxt < kmax) {
#pragma unroll
            for (int i = 0; i < 4; ++i) kr[i] = kr_n[i];
#pragma unroll
            for (int i = 0; i < 8; ++i) sc[i] = sc_n[i];
        }
        buf ^= 1;
    }

    // ---- normalise and store: this thread holds dims (d, d + 1), d = ch*16 + 2g, of queries 2c, 2c + 1 of each half
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const float l0 = __shfl_sync(0xffffffffu, l_run[h2], (2 * c) * 4), l1 = __shfl_sync(0xffffffffu, l_run[h2], (2 * c + 1) * 4);
        const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int qi = q_lo + 8 * h2 + 2 * c + e;
            if (qi >= a.S) continue;
            const size_t ob = (size_t)((long long)rrow * a.st.o_b + (long long)qi * a.st.o_s + (long long)head * a.st.o_h);
            const float inv = e ? i1 : i0;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                const int d = ch * 16 + 2 * g;
                st_out(a.out, a.dtype, ob + d, o[ch][h2][e] * inv);
                st_out(a.out, a.dtype, ob + d + 1, o[ch][h2][2 + e] * inv);
            }
        }
    }
}

}  // namespace

// Returns AB2_ERR_UNSUPPORTED when the cache or head layout is not the one this
// kernel serves (the caller then uses the general kernel).
int attention_decode_mma_device(const ab2_kv *kv, int layer, const void *q, void *out, int row0, int nrows,
                                float scale, ab2_dtype dtype, int nsplit, float *part_acc, float *part_ml,
                                int pending, long long q_stride, cudaStream_t s) {
    if (kv->dtype != AB2_KV_INT8 || kv->hd != 128 || kv->h / kv->kvh > 8) return AB2_ERR_UNSUPPORTED;
    MmaAttnArgs a;
    a.kv = kv_view(kv, layer);
    a.q = q; a.out = out; a.row0 = row0; a.h = kv->h; a.rep = kv->h / kv->kvh; a.nsplit = nsplit;
    a.dtype = (int)dtype; a.scale = scale; a.part_acc = part_acc; a.part_ml = part_ml;
    a.pending = pending; a.q_stride = q_stride;
    cudaError_t e = launch_kernel(attn_decode_mma_kernel, dim3(nsplit, kv->kvh, nrows), dim3(128), 0, s, a);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "decode attention launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

// S > 1 queries per row over an INT8 cache, head_dim 128, 1..4 query heads per KV head: the
// tensor-core causal kernel.  AB2_ERR_UNSUPPORTED otherwise (the caller keeps the general kernel).
int attention_prefill_mma_device(const ab2_kv *kv, int layer, const void *q, void *out, int S, int pending, int row0,
                                 int nrows, float scale, ab2_dtype dtype, AttnStrides st, cudaStream_t s) {
    const int rep = kv->h / kv->kvh;
    if (kv->dtype != AB2_KV_INT8 || kv->hd != 128 || rep > 4 || S < 2) return AB2_ERR_UNSUPPORTED;
    PrefillAttnArgs a;
    a.kv = kv_view(kv, layer);
    a.q = q; a.out = out; a.st = st; a.S = S; a.pending = pending; a.row0 = row0; a.rep = rep;
    a.dtype = (int)dtype; a.scale = scale;
    cudaError_t e = launch_kernel(attn_prefill_mma_kernel, dim3((S + 15) / 16, kv->kvh, nrows), dim3(128), 0, s, a);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "prefill attention launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

}  // namespace ab2
