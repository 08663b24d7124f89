// One-kernel decode attention for the decoder step: RoPE on the new token's Q
// and K, quantise + append of its K/V, grouped-query attention over the cache
// and the new token, and the log-sum-exp merge of the context splits.
//
// It produces what the separate operators produce in sequence
// (rope.apply_inference -> KVCache::update -> attention_forward_causal,
// crates/aarambh-studio-nn/src/attention.rs:265-283): Q and K are rounded to the
// activation type after rotation, the new K/V take part in the attention as the
// cache stores them (quantised for INT8), and the softmax is the same online
// form.  Grid (splits, kv heads, rows), 128 threads.  Split 0 owns the new token;
// the CTA that finishes last for a (row, kv head) merges the splits (a counter in
// global memory, reset by that CTA), so no second launch is needed.
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "kv_cache.cuh"
#include "ops.cuh"

using namespace ab2;

namespace ab2 {
int device_sm_count();
namespace {

__device__ __forceinline__ float ld_act(const void *p, int dtype, size_t i) {
    if (dtype == AB2_F32) return ((const float *)p)[i];
    if (dtype == AB2_F16) return __half2float(((const __half *)p)[i]);
    return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
}
__device__ __forceinline__ float round_act(float v, int dtype) {
    if (dtype == AB2_F32) return v;
    if (dtype == AB2_F16) return __half2float(__float2half_rn(v));
    return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void st_act(void *p, int dtype, size_t i, float v) {
    if (dtype == AB2_F32) ((float *)p)[i] = v;
    else if (dtype == AB2_F16) ((__half *)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ void i8x4(uint32_t w, float (&f)[4]) {
    const uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
}
// N consecutive cache elements (N a multiple of 4, or 2) starting at element e.
template <int KVD, int N>
__device__ __forceinline__ void ld_kv(const void *base, size_t e, float (&f)[N]) {
    if constexpr (N == 2) {
        if constexpr (KVD == AB2_KV_F32) {
            float2 v = *reinterpret_cast<const float2 *>((const float *)base + e);
            f[0] = v.x; f[1] = v.y;
        } else if constexpr (KVD == AB2_KV_BF16) {
            uint32_t v = *reinterpret_cast<const uint32_t *>((const __nv_bfloat16 *)base + e);
            f[0] = __uint_as_float(v << 16); f[1] = __uint_as_float(v & 0xffff0000u);
        } else {
            const int8_t *p = (const int8_t *)base + e;
            f[0] = (float)p[0]; f[1] = (float)p[1];
        }
    } else if constexpr (KVD == AB2_KV_F32) {
        const float4 *p = reinterpret_cast<const float4 *>((const float *)base + e);
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            float4 v = p[i];
            f[4 * i] = v.x; f[4 * i + 1] = v.y; f[4 * i + 2] = v.z; f[4 * i + 3] = v.w;
        }
    } else if constexpr (KVD == AB2_KV_BF16) {
        const uint2 *p = reinterpret_cast<const uint2 *>((const __nv_bfloat16 *)base + e);
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            uint2 v = p[i];
            f[4 * i] = __uint_as_float(v.x << 16); f[4 * i + 1] = __uint_as_float(v.x & 0xffff0000u);
            f[4 * i + 2] = __uint_as_float(v.y << 16); f[4 * i + 3] = __uint_as_float(v.y & 0xffff0000u);
        }
    } else {
        const uint32_t *p = reinterpret_cast<const uint32_t *>((const int8_t *)base + e);
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            float t[4];
            i8x4(p[i], t);
            f[4 * i] = t[0]; f[4 * i + 1] = t[1]; f[4 * i + 2] = t[2]; f[4 * i + 3] = t[3];
        }
    }
}

struct FusedArgs {
    KvView kv;
    const void *qkv;      // [rows][stride]: q heads, then k heads, then v heads
    void *out;            // [rows][h * hd]
    long long stride;
    const float *cos_t, *sin_t;
    const int *rope_pos;  // explicit positions per cache row, or nullptr (= cache length)
    int row0, h, rep, nsplit, dtype;
    float scale;
    float *part_acc, *part_ml;
    int *counters;        // [B][kvh], zero between launches
};

template <int KVD, int HD, int REP>
__global__ void __launch_bounds__(128) attn_decode_fused_kernel(FusedArgs a) {
    constexpr int DPL = HD / 32;
    constexpr int VUNROLL = KVD == AB2_KV_F32 ? 8 : (KVD == AB2_KV_BF16 ? 16 : 32);
    __shared__ alignas(16) float qs[REP][HD];
    __shared__ alignas(16) float knew[HD], vnew[HD];
    __shared__ float ps[4][REP][32];
    __shared__ float wm[4][REP], wl[4][REP];
    __shared__ float wacc[4][REP][HD];
    __shared__ float redk[8], redv[8];
    __shared__ int last_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int split = blockIdx.x, kvhead = blockIdx.y, rrow = blockIdx.z, row = kv_row(a.kv, a.row0, rrow);
    const int half = HD / 2;
    const int pos = a.kv.lens[row];                       // cached tokens; the new one lands here
    const int rpos = a.rope_pos ? a.rope_pos[row] : pos;  // RoPE position of the new token
    int per = (pos + a.nsplit - 1) / a.nsplit;
    per = (per + 31) & ~31;
    const int t0 = split * per, t1 = min(pos, t0 + per);
    const size_t tok_base = (size_t)rrow * a.stride;
    const float *cs = a.cos_t + (size_t)rpos * half, *sn = a.sin_t + (size_t)rpos * half;
    const size_t head_base = ((size_t)row * a.kv.kvh + kvhead) * a.kv.cap;

    // The cached K/V of older tokens do not depend on the preceding kernel: the
    // raw bytes of this warp's first chunk are requested before waiting for it,
    // all at once, so the chunk costs one memory round trip instead of a chain.
    constexpr bool STAGED = (KVD != AB2_KV_F32) && HD == 128;
    constexpr int ESZ = KVD == AB2_KV_INT8 ? 1 : 2;
    constexpr int KW = STAGED ? HD * ESZ / 16 : 1;  // 16-byte words of one K row
    constexpr int VW = STAGED ? DPL * ESZ / 4 : 1;  // 4-byte words of one lane's V slice
    uint4 kraw[KW];
    uint32_t vraw[32][VW];
    float kscale_c = 1.f, vscale_c = 1.f;
    auto stage_chunk = [&](int base) {
        const int tok = min(base + lane, t1 - 1);
        const size_t trow = head_base + tok;
        const uint4 *kp = reinterpret_cast<const uint4 *>((const char *)a.kv.k + trow * HD * ESZ);
#pragma unroll
        for (int i = 0; i < KW; ++i) kraw[i] = kp[i];
        if (KVD == AB2_KV_INT8) { kscale_c = a.kv.ks[trow]; vscale_c = a.kv.vs[trow]; }
        const int last = t1 - 1 - base;
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            const uint32_t *vp = reinterpret_cast<const uint32_t *>(
                (const char *)a.kv.v + ((head_base + base + min(t, last)) * HD + lane * DPL) * ESZ);
#pragma unroll
            for (int i = 0; i < VW; ++i) vraw[t][i] = vp[i];
        }
    };
    const int first_base = t0 + warp * 32;
    if (STAGED && first_base < t1) stage_chunk(first_base);
    pdl_wait();  // q, k, v of the new token come from the preceding projection
    pdl_launch_dependents();

    // ---- Q: rotate, round to the activation type
    for (int i = tid; i < REP * half; i += 128) {
        const int hh = i / half, d = i % half;
        float o1 = 0.f, o2 = 0.f;
        if (hh < a.rep) {
            const size_t qb = tok_base + (size_t)(kvhead * a.rep + hh) * HD;
            rope_rotate(ld_act(a.qkv, a.dtype, qb + d), ld_act(a.qkv, a.dtype, qb + half + d), cs[d], sn[d], o1, o2);
            o1 = round_act(o1, a.dtype);
            o2 = round_act(o2, a.dtype);
        }
        qs[hh][d] = o1;
        qs[hh][half + d] = o2;
    }
    // ---- new K / V of this kv head (split 0 stores them; every split 0 CTA also attends to them)
    if (split == 0) {
        const size_t kb = tok_base + (size_t)(a.h + kvhead) * HD;
        const size_t vb = tok_base + (size_t)(a.h + a.kv.kvh + kvhead) * HD;
        if (tid < half) {
            float o1, o2;
            rope_rotate(ld_act(a.qkv, a.dtype, kb + tid), ld_act(a.qkv, a.dtype, kb + half + tid), cs[tid], sn[tid], o1, o2);
            knew[tid] = round_act(o1, a.dtype);
            knew[half + tid] = round_act(o2, a.dtype);
        }
        if (tid < HD) vnew[tid] = ld_act(a.qkv, a.dtype, vb + tid);
    }
    __syncthreads();
    if (split == 0 && pos < a.kv.cap) {
        const size_t trow = ((size_t)row * a.kv.kvh + kvhead) * a.kv.cap + pos;
        if (KVD == AB2_KV_INT8) {
            float ka = tid < HD ? fabsf(knew[tid]) : 0.f, va = tid < HD ? fabsf(vnew[tid]) : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
                va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o));
            }
            if (lane == 0) { redk[warp] = ka; redv[warp] = va; }
            __syncthreads();
            const float kmax = fmaxf(fmaxf(redk[0], redk[1]), fmaxf(redk[2], redk[3]));
            const float vmax = fmaxf(fmaxf(redv[0], redv[1]), fmaxf(redv[2], redv[3]));
            const float kscale = (kmax <= FLT_EPSILON) ? 1.0f : __fdiv_rn(kmax, 127.0f);
            const float vscale = (vmax <= FLT_EPSILON) ? 1.0f : __fdiv_rn(vmax, 127.0f);
            if (tid < HD) {
                auto enc = [](float x, float sc) -> float {
                    float q = roundf(__fdiv_rn(x, sc));
                    q = q < -127.f ? -127.f : (q > 127.f ? 127.f : q);
                    return (q != q) ? 0.f : q;
                };
                const float kq = enc(knew[tid], kscale), vq = enc(vnew[tid], vscale);
                ((int8_t *)a.kv.k)[trow * HD + tid] = (int8_t)kq;
                ((int8_t *)a.kv.v)[trow * HD + tid] = (int8_t)vq;
                knew[tid] = __fmul_rn(kq, kscale);  // what the cache will return
                vnew[tid] = __fmul_rn(vq, vscale);
            }
            if (tid == 0) { a.kv.ks[trow] = kscale; a.kv.vs[trow] = vscale; }
        } else if (tid < HD) {
            if (KVD == AB2_KV_F32) {
                ((float *)a.kv.k)[trow * HD + tid] = knew[tid];
                ((float *)a.kv.v)[trow * HD + tid] = vnew[tid];
            } else {
                const __nv_bfloat16 kb16 = __float2bfloat16_rn(knew[tid]), vb16 = __float2bfloat16_rn(vnew[tid]);
                ((__nv_bfloat16 *)a.kv.k)[trow * HD + tid] = kb16;
                ((__nv_bfloat16 *)a.kv.v)[trow * HD + tid] = vb16;
                knew[tid] = __bfloat162float(kb16);
                vnew[tid] = __bfloat162float(vb16);
            }
        }
        __syncthreads();
    }

    float m_run[REP], l_run[REP], acc[REP][DPL];
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) {
        m_run[hh] = -INFINITY;
        l_run[hh] = 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[hh][j] = 0.f;
    }

    // ---- cached tokens of this split
    for (int base = t0 + warp * 32; base < t1; base += 128) {
        const int tok = base + lane;
        const bool valid = tok < t1;
        const size_t trow = head_base + (valid ? tok : t1 - 1);
        if (STAGED && base != first_base) stage_chunk(base);
        float sc[REP];
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) sc[hh] = 0.f;
#pragma unroll
        for (int d0 = 0; d0 < HD; d0 += 16) {
            float kf[16];
            if constexpr (STAGED) {
                if constexpr (KVD == AB2_KV_INT8) {
                    const uint32_t w4[4] = {kraw[d0 / 16].x, kraw[d0 / 16].y, kraw[d0 / 16].z, kraw[d0 / 16].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float t[4];
                        i8x4(w4[i], t);
                        kf[4 * i] = t[0]; kf[4 * i + 1] = t[1]; kf[4 * i + 2] = t[2]; kf[4 * i + 3] = t[3];
                    }
                } else {
#pragma unroll
                    for (int hv = 0; hv < 2; ++hv) {
                        const uint4 r4 = kraw[d0 / 8 + hv];
                        const uint32_t w4[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            kf[8 * hv + 2 * i] = __uint_as_float(w4[i] << 16);
                            kf[8 * hv + 2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
                        }
                    }
                }
            } else {
                ld_kv<KVD, 16>(a.kv.k, trow * HD + d0, kf);
            }
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) {
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const float4 qv = *reinterpret_cast<const float4 *>(&qs[hh][d0 + i]);
                    sc[hh] = fmaf(qv.x, kf[i], sc[hh]);
                    sc[hh] = fmaf(qv.y, kf[i + 1], sc[hh]);
                    sc[hh] = fmaf(qv.z, kf[i + 2], sc[hh]);
                    sc[hh] = fmaf(qv.w, kf[i + 3], sc[hh]);
                }
            }
        }
        float kscale = kscale_c, vscale = vscale_c;
        if (!STAGED && KVD == AB2_KV_INT8) { kscale = a.kv.ks[trow]; vscale = a.kv.vs[trow]; }
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) {
            const float s = valid ? sc[hh] * kscale * a.scale : -INFINITY;
            float cm = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
            const float m_new = fmaxf(m_run[hh], cm);
            const float corr = expf(m_run[hh] - m_new);
            const float p = valid ? expf(s - m_new) : 0.f;
            float psum = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            l_run[hh] = l_run[hh] * corr + psum;
            m_run[hh] = m_new;
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[hh][j] *= corr;
            ps[warp][hh][lane] = p * vscale;
        }
        __syncwarp();
        // PV: lanes span head_dim; rows past the end were staged from the last valid
        // row and are weighted by p = 0.
        if constexpr (STAGED) {
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                float vf[DPL];
                if constexpr (KVD == AB2_KV_INT8) {
                    i8x4(vraw[t][0], vf);
                } else {
                    vf[0] = __uint_as_float(vraw[t][0] << 16); vf[1] = __uint_as_float(vraw[t][0] & 0xffff0000u);
                    vf[2] = __uint_as_float(vraw[t][1] << 16); vf[3] = __uint_as_float(vraw[t][1] & 0xffff0000u);
                }
#pragma unroll
                for (int hh = 0; hh < REP; ++hh) {
                    const float p = ps[warp][hh][t];
#pragma unroll
                    for (int j = 0; j < DPL; ++j) acc[hh][j] = fmaf(p, vf[j], acc[hh][j]);
                }
            }
        } else {
            const int last = t1 - 1 - base;
#pragma unroll
            for (int tb = 0; tb < 32; tb += VUNROLL) {
                float vf[VUNROLL][DPL];
#pragma unroll
                for (int t = 0; t < VUNROLL; ++t)
                    ld_kv<KVD, DPL>(a.kv.v, (head_base + base + min(tb + t, last)) * HD + lane * DPL, vf[t]);
#pragma unroll
                for (int t = 0; t < VUNROLL; ++t)
#pragma unroll
                    for (int hh = 0; hh < REP; ++hh) {
                        const float p = ps[warp][hh][tb + t];
#pragma unroll
                        for (int j = 0; j < DPL; ++j) acc[hh][j] = fmaf(p, vf[t][j], acc[hh][j]);
                    }
            }
        }
        __syncwarp();
    }

    // ---- the new token (split 0, warp 0): lanes span head_dim
    if (split == 0 && warp == 0) {
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) {
            float dot = 0.f;
#pragma unroll
            for (int j = 0; j < DPL; ++j) dot = fmaf(qs[hh][lane * DPL + j], knew[lane * DPL + j], dot);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float s = dot * a.scale;
            const float m_new = fmaxf(m_run[hh], s);
            const float corr = expf(m_run[hh] - m_new), p = expf(s - m_new);
            l_run[hh] = l_run[hh] * corr + p;
            m_run[hh] = m_new;
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[hh][j] = fmaf(p, vnew[lane * DPL + j], acc[hh][j] * corr);
        }
    }

    // ---- merge the four warps
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) {
        if (lane == 0) { wm[warp][hh] = m_run[hh]; wl[warp][hh] = l_run[hh]; }
#pragma unroll
        for (int j = 0; j < DPL; ++j) wacc[warp][hh][lane * DPL + j] = acc[hh][j];
    }
    __syncthreads();
    const size_t out_base = (size_t)rrow * a.h * HD;
    for (int i = tid; i < a.rep * HD; i += 128) {
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
            st_act(a.out, a.dtype, out_base + (size_t)head * HD + d, L > 0.f ? A * (1.0f / L) : A);
        } else {
            const size_t pi = ((size_t)row * a.h + head) * a.nsplit + split;
            a.part_acc[pi * HD + d] = A;
            if (d == 0) { a.part_ml[pi * 2] = M; a.part_ml[pi * 2 + 1] = L; }
        }
    }
    if (a.nsplit == 1) return;

    // ---- the last CTA of this (row, kv head) merges the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(&a.counters[row * a.kv.kvh + kvhead], 1);
        last_flag = (old == a.nsplit - 1);
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    for (int i = tid; i < a.rep * HD; i += 128) {
        const int hh = i / HD, d = i % HD, head = kvhead * a.rep + hh;
        const size_t p0 = ((size_t)row * a.h + head) * a.nsplit;
        float M = -INFINITY;
        for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, __ldcg(&a.part_ml[(p0 + s) * 2]));
        float L = 0.f, A = 0.f;
        for (int s = 0; s < a.nsplit; ++s) {
            const float m = __ldcg(&a.part_ml[(p0 + s) * 2]);
            const float e = (m == -INFINITY) ? 0.f : expf(m - M);
            L += e * __ldcg(&a.part_ml[(p0 + s) * 2 + 1]);
            A += e * __ldcg(&a.part_acc[(p0 + s) * HD + d]);
        }
        st_act(a.out, a.dtype, out_base + (size_t)head * HD + d, L > 0.f ? A * (1.0f / L) : A);
    }
    if (tid == 0) a.counters[row * a.kv.kvh + kvhead] = 0;
}

template <int KVD, int HD>
void launch_fused(const FusedArgs &a, dim3 grid, cudaStream_t s) {
    if (a.rep == 1) launch_kernel(attn_decode_fused_kernel<KVD, HD, 1>, grid, dim3(128), 0, s, a);
    else if (a.rep == 2) launch_kernel(attn_decode_fused_kernel<KVD, HD, 2>, grid, dim3(128), 0, s, a);
    else if (a.rep <= 4) launch_kernel(attn_decode_fused_kernel<KVD, HD, 4>, grid, dim3(128), 0, s, a);
    else launch_kernel(attn_decode_fused_kernel<KVD, HD, 8>, grid, dim3(128), 0, s, a);
}

template <int KVD>
int launch_fused_hd(const FusedArgs &a, dim3 grid, cudaStream_t s) {
    if (a.kv.hd == 64) launch_fused<KVD, 64>(a, grid, s);
    else if (a.kv.hd == 128) launch_fused<KVD, 128>(a, grid, s);
    else return fail(AB2_ERR_UNSUPPORTED, "attention supports head_dim 64 and 128, got %d", a.kv.hd);
    return AB2_OK;
}

}  // namespace

// qkv: [nrows][stride] activations of one new token per row (q heads, k heads, v
// heads); writes the token's K/V into the cache at each row's current length
// (which the caller advances afterwards) and the attention output [nrows][h*hd].
int attention_decode_fused_device(ab2_kv *kv, int layer, const void *qkv, long long stride, void *out,
                                  int row0, int nrows, float scale, ab2_dtype dtype, const float *cos_t,
                                  const float *sin_t, const int *rope_pos, int len_hint, cudaStream_t s) {
    FusedArgs a;
    a.kv = kv_view(kv, layer);
    a.qkv = qkv; a.out = out; a.stride = stride; a.cos_t = cos_t; a.sin_t = sin_t; a.rope_pos = rope_pos;
    a.row0 = row0; a.h = kv->h; a.rep = kv->h / kv->kvh; a.dtype = (int)dtype; a.scale = scale;
    a.part_acc = kv->part_acc; a.part_ml = kv->part_ml; a.counters = kv->counters;
    int max_len = len_hint;
    if (max_len <= 0)
        for (int i = 0; i < nrows; ++i) max_len = std::max(max_len, kv->lens_host[kv_row_host(kv, row0, i)]);
    const int want = (2 * device_sm_count() + nrows * kv->kvh - 1) / (nrows * kv->kvh);
    a.nsplit = std::max(1, std::min(std::min(want, (max_len + 127) / 128), kv->max_splits));
    dim3 grid(a.nsplit, kv->kvh, nrows);
    int rc;
    if (kv->dtype == AB2_KV_F32) rc = launch_fused_hd<AB2_KV_F32>(a, grid, s);
    else if (kv->dtype == AB2_KV_BF16) rc = launch_fused_hd<AB2_KV_BF16>(a, grid, s);
    else rc = launch_fused_hd<AB2_KV_INT8>(a, grid, s);
    if (rc != AB2_OK) return rc;
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

}  // namespace ab2
