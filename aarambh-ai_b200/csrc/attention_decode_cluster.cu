// Decode attention for the decoder step over an INT8 cache, one thread-block
// cluster per (row, kv head): RoPE on the new token's Q and K, quantise + append
// of its K/V, grouped-query attention over the cache and the new token, and the
// log-sum-exp merge of the context splits.
//
// Same arithmetic as attention_decode_fused.cu (which serves the other cache
// types, head sizes and long contexts).  What differs is how the splits meet:
// the CTAs of a cluster each take a slice of the context, leave their partial
// (max, sum, accumulator) in their own shared memory, and after one cluster
// barrier every CTA merges a slice of the output by reading its peers' shared
// memory directly.  No partials travel through global memory and nothing waits
// on a global counter, which at a few hundred cached tokens is most of the time
// of the split kernel.
//
// 256 threads.  Every warp of the cluster takes a contiguous run of cached
// tokens, except warp 7 of CTA 0, which owns the new token (rotation, per-token
// absmax quantisation, the store into the cache, and its score).
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "kv_cache.cuh"
#include "ops.cuh"

using namespace ab2;

namespace ab2 {
int device_sm_count();
namespace {

constexpr int HD = 128;

__device__ __forceinline__ void i8x4_f32(uint32_t w, float (&f)[4]) {
    const uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// f32 at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ float ld_peer(const float *p, uint32_t rank) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

struct ClusterArgs {
    KvView kv;
    const __nv_bfloat16 *qkv;  // [rows][stride]: q heads, then k heads, then v heads
    __nv_bfloat16 *out;        // [rows][h * hd]
    long long stride;
    const float *cos_t, *sin_t;
    const int *rope_pos;  // explicit positions per cache row, or nullptr (= cache length)
    int row0, h, nsplit;
    float scale;
};

template <int REP>
__global__ void __launch_bounds__(256) attn_decode_cluster_kernel(ClusterArgs a) {
    __shared__ alignas(16) float qs[REP][HD];
    __shared__ alignas(16) float ps[8][32][REP];
    __shared__ float wm[8][REP], wl[8][REP];
    __shared__ alignas(16) float wacc[8][REP][HD];
    __shared__ float cm[REP], cl[REP];      // this CTA's partial, read by its peers
    __shared__ alignas(16) float cacc[REP][HD];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int rank = (int)cluster_rank(), nsplit = a.nsplit;
    const int kvhead = blockIdx.y, rrow = blockIdx.z, row = kv_row(a.kv, a.row0, rrow);
    constexpr int half = HD / 2;
    const int pos = a.kv.lens[row];                       // cached tokens; the new one lands here
    const int rpos = a.rope_pos ? a.rope_pos[row] : pos;  // RoPE position of the new token
    const float *cs = a.cos_t + (size_t)rpos * half, *sn = a.sin_t + (size_t)rpos * half;
    const size_t head_base = ((size_t)row * a.kv.kvh + kvhead) * a.kv.cap;
    const size_t tok_base = (size_t)rrow * a.stride;
    const bool new_token_warp = rank == 0 && warp == 7;

    // contiguous run of cached tokens of this warp
    const int workers = nsplit * 8 - 1;
    const int widx = rank * 8 + warp - (rank > 0 ? 1 : 0);
    const int tpw = (pos + workers - 1) / workers;
    const int t0 = new_token_warp ? 0 : min(pos, widx * tpw);
    const int t1 = new_token_warp ? 0 : min(pos, t0 + tpw);

    // The cached K/V do not depend on the preceding kernel: the raw bytes of the
    // first chunk are requested before waiting for it, all at once.
    uint4 kraw[8];
    uint32_t vraw[32];
    float kscale_c = 1.f, vscale_c = 1.f;
    auto stage_chunk = [&](int base, int n) {
        const size_t trow = head_base + min(base + lane, t1 - 1);
        const uint4 *kp = reinterpret_cast<const uint4 *>((const char *)a.kv.k + trow * HD);
#pragma unroll
        for (int i = 0; i < 8; ++i) kraw[i] = kp[i];
        kscale_c = a.kv.ks[trow];
        vscale_c = a.kv.vs[trow];
#pragma unroll
        for (int t = 0; t < 32; ++t)
            if (t < n)
                vraw[t] = *reinterpret_cast<const uint32_t *>((const char *)a.kv.v + (head_base + base + t) * HD + lane * 4);
    };
    // Short runs (at most 16 tokens per warp, the usual case at a few hundred cached
    // tokens): LPT = 4 or 2 lanes share a token, each holding 32 or 64 of its 128 K
    // bytes, so the score costs 1/LPT of the lane-per-token form and no lane idles.
    const int lpt = tpw <= 8 ? 4 : (tpw <= 16 ? 2 : 1);
    uint4 kq[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) kq[i] = make_uint4(0u, 0u, 0u, 0u);
    if (t0 < t1) {
        if (lpt > 1) {
            const int n = t1 - t0;
            const int qj = lpt == 4 ? lane >> 2 : lane >> 1, qp = lpt == 4 ? lane & 3 : lane & 1;
            const size_t trow = head_base + t0 + min(qj, n - 1);
            const uint4 *kp = reinterpret_cast<const uint4 *>((const char *)a.kv.k + trow * HD + qp * (HD / lpt));
            kq[0] = kp[0];
            kq[1] = kp[1];
            if (lpt == 2) { kq[2] = kp[2]; kq[3] = kp[3]; }
            kscale_c = a.kv.ks[trow];
            vscale_c = a.kv.vs[trow];
#pragma unroll
            for (int t = 0; t < 16; ++t)
                if (t < n)
                    vraw[t] = *reinterpret_cast<const uint32_t *>((const char *)a.kv.v + (head_base + t0 + t) * HD + lane * 4);
        } else {
            stage_chunk(t0, min(32, t1 - t0));
        }
    }
    // rotation table entries of this thread's pair (the position is known already)
    const int qh = tid >> 6, qd = tid & 63;
    const float qc = cs[qd], qsn = sn[qd];
    float2 nc = make_float2(1.f, 1.f), ns = make_float2(0.f, 0.f);
    if (new_token_warp) {
        nc = *reinterpret_cast<const float2 *>(cs + 2 * lane);
        ns = *reinterpret_cast<const float2 *>(sn + 2 * lane);
    }

    pdl_wait();  // q, k, v of the new token come from the preceding projection
    pdl_launch_dependents();

    // ---- Q: one rotation pair per thread (4 heads x 64 pairs), rounded to bf16
    for (int hh = qh; hh < REP; hh += 4) {
        const __nv_bfloat16 *qp = a.qkv + tok_base + (size_t)(kvhead * REP + hh) * HD;
        float o1, o2;
        rope_rotate(__bfloat162float(qp[qd]), __bfloat162float(qp[half + qd]), qc, qsn, o1, o2);
        qs[hh][qd] = bf16_round(o1);
        qs[hh][half + qd] = bf16_round(o2);
    }
    // ---- the new token (warp 7 of CTA 0): lane owns dims 2l, 2l+1, 64+2l, 64+2l+1
    float kd[4] = {0.f, 0.f, 0.f, 0.f}, vd[4] = {0.f, 0.f, 0.f, 0.f};
    if (new_token_warp) {
        const __nv_bfloat16 *kp = a.qkv + tok_base + (size_t)(a.h + kvhead) * HD;
        const __nv_bfloat16 *vp = a.qkv + tok_base + (size_t)(a.h + a.kv.kvh + kvhead) * HD;
        const uint32_t klo = *reinterpret_cast<const uint32_t *>(kp + 2 * lane);
        const uint32_t khi = *reinterpret_cast<const uint32_t *>(kp + half + 2 * lane);
        const uint32_t vlo = *reinterpret_cast<const uint32_t *>(vp + 2 * lane);
        const uint32_t vhi = *reinterpret_cast<const uint32_t *>(vp + half + 2 * lane);
        float o1, o2;
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
            kd[i] = __fmul_rn(kq[i], kscale);  // what the cache will return
            vd[i] = __fmul_rn(vq[i], vscale);
        }
        if (pos < a.kv.cap) {
            const size_t trow = head_base + pos;
            auto pack2 = [](float x, float y) -> uint16_t {
                return (uint16_t)((uint32_t)(uint8_t)(int8_t)x | ((uint32_t)(uint8_t)(int8_t)y << 8));
            };
            uint16_t *kc = reinterpret_cast<uint16_t *>((int8_t *)a.kv.k + trow * HD);
            uint16_t *vc = reinterpret_cast<uint16_t *>((int8_t *)a.kv.v + trow * HD);
            kc[lane] = pack2(kq[0], kq[1]);
            kc[32 + lane] = pack2(kq[2], kq[3]);
            vc[lane] = pack2(vq[0], vq[1]);
            vc[32 + lane] = pack2(vq[2], vq[3]);
            if (lane == 0) { a.kv.ks[trow] = kscale; a.kv.vs[trow] = vscale; }
        }
    }
    __syncthreads();

    float m_run[REP], l_run[REP], acc[REP][4];
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) {
        m_run[hh] = -INFINITY;
        l_run[hh] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[hh][j] = 0.f;
    }

    if (new_token_warp) {
        // score of the new token; this warp's accumulator uses its own dim ownership
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) {
            float dot = qs[hh][2 * lane] * kd[0];
            dot = fmaf(qs[hh][2 * lane + 1], kd[1], dot);
            dot = fmaf(qs[hh][half + 2 * lane], kd[2], dot);
            dot = fmaf(qs[hh][half + 2 * lane + 1], kd[3], dot);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) { wm[warp][hh] = dot * a.scale; wl[warp][hh] = 1.f; }
            wacc[warp][hh][2 * lane] = vd[0];
            wacc[warp][hh][2 * lane + 1] = vd[1];
            wacc[warp][hh][half + 2 * lane] = vd[2];
            wacc[warp][hh][half + 2 * lane + 1] = vd[3];
        }
    } else {
        if (lpt > 1 && t0 < t1) {
            const int n = t1 - t0;
            const int qj = lpt == 4 ? lane >> 2 : lane >> 1, qp = lpt == 4 ? lane & 3 : lane & 1;
            const int dims = HD / lpt;  // dims of this lane's part of the token
            const bool valid = qj < n;
            float sc[REP];
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) sc[hh] = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                if (w * 16 < dims) {
                    const uint32_t w4[4] = {kq[w].x, kq[w].y, kq[w].z, kq[w].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float kf[4];
                        i8x4_f32(w4[i], kf);
#pragma unroll
                        for (int hh = 0; hh < REP; ++hh) {
                            const float4 qv = *reinterpret_cast<const float4 *>(&qs[hh][qp * dims + w * 16 + i * 4]);
                            sc[hh] = fmaf(qv.x, kf[0], sc[hh]);
                            sc[hh] = fmaf(qv.y, kf[1], sc[hh]);
                            sc[hh] = fmaf(qv.z, kf[2], sc[hh]);
                            sc[hh] = fmaf(qv.w, kf[3], sc[hh]);
                        }
                    }
                }
            }
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) {
                // the parts of a token's dot product, then the softmax over the tokens
                float dot = sc[hh];
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                if (lpt == 4) dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                const float s = valid ? dot * kscale_c * a.scale : -INFINITY;
                float cmx = s;
#pragma unroll
                for (int o = 2; o < 32; o <<= 1)
                    if (o >= lpt) cmx = fmaxf(cmx, __shfl_xor_sync(0xffffffffu, cmx, o));
                const float p = valid ? expf(s - cmx) : 0.f;
                float psum = p;
#pragma unroll
                for (int o = 2; o < 32; o <<= 1)
                    if (o >= lpt) psum += __shfl_xor_sync(0xffffffffu, psum, o);
                m_run[hh] = cmx;
                l_run[hh] = psum;
                if (qp == 0) ps[warp][qj][hh] = p * vscale_c;
            }
            __syncwarp();
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                if (t < n) {
                    float vf[4];
                    i8x4_f32(vraw[t], vf);
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        const float p = ps[warp][t][hh];
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[hh][j] = fmaf(p, vf[j], acc[hh][j]);
                    }
                }
            }
        }
        // ---- cached tokens of this warp, 32 at a time
        for (int base = t0; lpt == 1 && base < t1; base += 32) {
            const int n = min(32, t1 - base);
            const bool valid = lane < n;
            if (base != t0) stage_chunk(base, n);
            float sc[REP];
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) sc[hh] = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const uint32_t w4[4] = {kraw[w].x, kraw[w].y, kraw[w].z, kraw[w].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float kf[4];
                    i8x4_f32(w4[i], kf);
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        const float4 qv = *reinterpret_cast<const float4 *>(&qs[hh][w * 16 + i * 4]);
                        sc[hh] = fmaf(qv.x, kf[0], sc[hh]);
                        sc[hh] = fmaf(qv.y, kf[1], sc[hh]);
                        sc[hh] = fmaf(qv.z, kf[2], sc[hh]);
                        sc[hh] = fmaf(qv.w, kf[3], sc[hh]);
                    }
                }
            }
            float pv[REP];
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) {
                const float s = valid ? sc[hh] * kscale_c * a.scale : -INFINITY;
                float cmx = s;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) cmx = fmaxf(cmx, __shfl_xor_sync(0xffffffffu, cmx, o));
                const float m_new = fmaxf(m_run[hh], cmx);
                const float corr = expf(m_run[hh] - m_new);
                const float p = valid ? expf(s - m_new) : 0.f;
                float psum = p;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
                l_run[hh] = l_run[hh] * corr + psum;
                m_run[hh] = m_new;
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[hh][j] *= corr;
                pv[hh] = p * vscale_c;
            }
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) ps[warp][lane][hh] = pv[hh];
            __syncwarp();
            // PV: lanes span head_dim (dims 4l .. 4l+3)
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                if (t < n) {
                    float vf[4];
                    i8x4_f32(vraw[t], vf);
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        const float p = ps[warp][t][hh];
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[hh][j] = fmaf(p, vf[j], acc[hh][j]);
                    }
                }
            }
            __syncwarp();
        }
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) {
            if (lane == 0) { wm[warp][hh] = m_run[hh]; wl[warp][hh] = l_run[hh]; }
#pragma unroll
            for (int j = 0; j < 4; ++j) wacc[warp][hh][lane * 4 + j] = acc[hh][j];
        }
    }
    __syncthreads();

    // ---- merge the eight warps into this CTA's partial
    for (int i = tid; i < REP * HD; i += 256) {
        const int hh = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) M = fmaxf(M, wm[w][hh]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float e = (wm[w][hh] == -INFINITY) ? 0.f : expf(wm[w][hh] - M);
            L += e * wl[w][hh];
            A += e * wacc[w][hh][d];
        }
        cacc[hh][d] = A;
        if (d == 0) { cm[hh] = M; cl[hh] = L; }
    }
    cluster_sync_all();

    // ---- every CTA merges a slice of the output over its peers' partials
    const int total = REP * HD, slice = (total + nsplit - 1) / nsplit;
    for (int j = tid; j < slice; j += 256) {
        const int i = rank * slice + j;
        if (i >= total) break;
        const int hh = i / HD, d = i % HD, head = kvhead * REP + hh;
        // all peer loads in flight at once (a cluster has at most 8 CTAs)
        float mv[8], lv[8], av[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const bool on = s < nsplit;
            mv[s] = on ? ld_peer(&cm[hh], s) : -INFINITY;
            lv[s] = on ? ld_peer(&cl[hh], s) : 0.f;
            av[s] = on ? ld_peer(&cacc[hh][d], s) : 0.f;
        }
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < 8; ++s) M = fmaxf(M, mv[s]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float e = (mv[s] == -INFINITY) ? 0.f : expf(mv[s] - M);
            L += e * lv[s];
            A += e * av[s];
        }
        a.out[(size_t)rrow * a.h * HD + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? A * (1.0f / L) : A);
    }
    // nobody leaves while a peer may still read its shared memory
    cluster_sync_all();
}

template <int REP>
cudaError_t launch_cluster(const ClusterArgs &a, dim3 grid, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = grid.x; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl_launch ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, attn_decode_cluster_kernel<REP>, a);
}

}  // namespace

// True when the cluster kernel serves this configuration.
bool attention_decode_cluster_eligible(const ab2_kv *kv, ab2_dtype dtype, int max_len) {
    static const bool off = getenv("AB2_NO_CLUSTER_ATTN") != nullptr;
    const int rep = kv->h / kv->kvh;
    return !off && kv->dtype == AB2_KV_INT8 && kv->hd == HD && dtype == AB2_BF16 &&
           (rep == 1 || rep == 2 || rep == 4) && max_len <= 8192;
}

int attention_decode_cluster_device(ab2_kv *kv, int layer, const void *qkv, long long stride, void *out,
                                    int row0, int nrows, float scale, const float *cos_t, const float *sin_t,
                                    const int *rope_pos, int max_len, cudaStream_t s) {
    ClusterArgs a;
    a.kv = kv_view(kv, layer);
    a.qkv = (const __nv_bfloat16 *)qkv; a.out = (__nv_bfloat16 *)out; a.stride = stride;
    a.cos_t = cos_t; a.sin_t = sin_t; a.rope_pos = rope_pos;
    a.row0 = row0; a.h = kv->h; a.scale = scale;
    // context splits: one per 128 tokens (rounded up to a power of two, at most 8), but no more
    // than keeps every CTA of the launch resident at once (two CTAs fit an SM): a second wave
    // of clusters costs a whole kernel latency
    const int by_ctx = (max_len + 127) / 128;
    const int want = by_ctx <= 1 ? 1 : (by_ctx <= 2 ? 2 : (by_ctx <= 4 ? 4 : 8));
    const int fit = std::max(1, 2 * device_sm_count() / (nrows * kv->kvh));
    const int cap = fit >= 8 ? 8 : (fit >= 4 ? 4 : (fit >= 2 ? 2 : 1));
    a.nsplit = std::min(want, cap);
    dim3 grid(a.nsplit, kv->kvh, nrows);
    const int rep = kv->h / kv->kvh;
    cudaError_t e;
    if (rep == 1) e = launch_cluster<1>(a, grid, s);
    else if (rep == 2) e = launch_cluster<2>(a, grid, s);
    else e = launch_cluster<4>(a, grid, s);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "cluster attention launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

}  // namespace ab2
