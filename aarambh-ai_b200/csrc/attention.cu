// Grouped-query attention over the KV cache.
//
// One kernel serves decode (one query per sequence, context split across CTAs,
// partial softmax merged with a log-sum-exp reduction) and prefill (S queries
// per sequence, causal).  A CTA owns one (query, kv head, context split) and
// computes all query heads that share the kv head, so K and V are read once
// per group instead of once per query head; the reference first materialises
// the repeated heads (crates/aarambh-studio-nn/src/attention.rs:415-428) and
// runs one row per (b, h, q) (crates/aarambh-studio-kernel/src/cpu/
// parallel_attn.rs:189-234).  Scores are q.k * scale with f32 accumulation and
// an online softmax; causal cut: query qi sees positions <= len - S + qi.
#include <algorithm>
#include <cfloat>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kv_cache.cuh"

using namespace ab2;

namespace ab2 {

__device__ __forceinline__ float load_act(const void *p, int dtype, size_t i) {
    if (dtype == AB2_F32) return ((const float *)p)[i];
    if (dtype == AB2_F16) return __half2float(((const __half *)p)[i]);
    return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
}
__device__ __forceinline__ void store_act(void *p, int dtype, size_t i, float v) {
    if (dtype == AB2_F32) ((float *)p)[i] = v;
    else if (dtype == AB2_F16) ((__half *)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
}

// 4 consecutive int8 codes (one u32) -> f32, via the 2^23 + 128 mantissa trick
// on the sign-flipped bytes (exact).
__device__ __forceinline__ void i8x4_to_f32(uint32_t w, float (&f)[4]) {
    const uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f;
}

// Loads N consecutive cache elements starting at element index `e` as f32.
template <int KVD, int N>
__device__ __forceinline__ void load_kv(const void *base, size_t e, float (&f)[N]) {
    if constexpr (N == 2) {  // head_dim 64: two elements per lane
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
            i8x4_to_f32(p[i], t);
            f[4 * i] = t[0]; f[4 * i + 1] = t[1]; f[4 * i + 2] = t[2]; f[4 * i + 3] = t[3];
        }
    }
}

struct AttnArgs {
    KvView kv;
    const void *q;
    void *out;
    AttnStrides st;
    int S, pending, row0, h, rep, nsplit, dtype;
    float scale;
    float *part_acc, *part_ml;
};

// grid (nsplit, kvh, nrows * S), 128 threads.  REP = compiled head-group width
// (>= rep); HD = head_dim.
template <int KVD, int HD, int REP>
__global__ void __launch_bounds__(128) attn_split_kernel(AttnArgs a) {
    constexpr int DPL = HD / 32;  // output dims per lane in the PV phase
    __shared__ alignas(16) float qs[REP][HD];
    __shared__ float ps[4][REP][32];
    __shared__ float wm[4][REP], wl[4][REP];
    __shared__ float wacc[4][REP][HD];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, kvhead = blockIdx.y;
    const int rrow = blockIdx.z / a.S, qi = blockIdx.z % a.S, row = kv_row(a.kv, a.row0, rrow);
    const int kv_end = a.kv.lens[row] + a.pending - a.S + qi + 1;
    int per = (kv_end + a.nsplit - 1) / a.nsplit;
    per = (per + 31) & ~31;
    const int t0 = split * per, t1 = min(kv_end, t0 + per);

    for (int i = threadIdx.x; i < REP * HD; i += 128) {
        const int hh = i / HD, d = i % HD;
        float v = 0.f;
        if (hh < a.rep)
            v = load_act(a.q, a.dtype,
                         (size_t)((long long)rrow * a.st.q_b + (long long)qi * a.st.q_s +
                                  (long long)(kvhead * a.rep + hh) * a.st.q_h + d));
        qs[hh][d] = v;
    }
    __syncthreads();

    const size_t head_base = ((size_t)row * a.kv.kvh + kvhead) * a.kv.cap;
    float m_run[REP], l_run[REP], acc[REP][DPL];
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) {
        m_run[hh] = -INFINITY;
        l_run[hh] = 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[hh][j] = 0.f;
    }

    for (int base = t0 + warp * 32; base < t1; base += 128) {
        const int tok = base + lane;
        const bool valid = tok < t1;
        const size_t trow = head_base + (valid ? tok : t1 - 1);
        // ---- scores: this lane's token against every query head of the group
        float sc[REP];
#pragma unroll
        for (int hh = 0; hh < REP; ++hh) sc[hh] = 0.f;
#pragma unroll 2
        for (int d0 = 0; d0 < HD; d0 += 16) {
            float kf[16];
            load_kv<KVD, 16>(a.kv.k, trow * HD + d0, kf);
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
        float kscale = 1.f, vscale = 1.f;
        if (KVD == AB2_KV_INT8) { kscale = a.kv.ks[trow]; vscale = a.kv.vs[trow]; }
        // ---- online softmax over the 32 tokens of the chunk
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
        // ---- PV: lanes span head_dim, loop over the chunk's tokens
        const int nt = min(32, t1 - base);
#pragma unroll 4
        for (int t = 0; t < nt; ++t) {
            float vf[DPL];
            load_kv<KVD, DPL>(a.kv.v, (head_base + base + t) * HD + lane * DPL, vf);
#pragma unroll
            for (int hh = 0; hh < REP; ++hh) {
                const float p = ps[warp][hh][t];
#pragma unroll
                for (int j = 0; j < DPL; ++j) acc[hh][j] = fmaf(p, vf[j], acc[hh][j]);
            }
        }
        __syncwarp();
    }

    // ---- merge the four warps
#pragma unroll
    for (int hh = 0; hh < REP; ++hh) {
        if (lane == 0) { wm[warp][hh] = m_run[hh]; wl[warp][hh] = l_run[hh]; }
#pragma unroll
        for (int j = 0; j < DPL; ++j) wacc[warp][hh][lane * DPL + j] = acc[hh][j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.rep * HD; i += 128) {
        const int hh = i / HD, d = i % HD;
        float M = fmaxf(fmaxf(wm[0][hh], wm[1][hh]), fmaxf(wm[2][hh], wm[3][hh]));
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float e = (wm[w][hh] == -INFINITY) ? 0.f : expf(wm[w][hh] - M);
            L += e * wl[w][hh];
            A += e * wacc[w][hh][d];
        }
        const int head = kvhead * a.rep + hh;
        if (a.nsplit == 1) {
            const float o = L > 0.f ? A * (1.0f / L) : A;
            store_act(a.out, a.dtype,
                      (size_t)((long long)rrow * a.st.o_b + (long long)qi * a.st.o_s + (long long)head * a.st.o_h + d), o);
        } else {
            const size_t pi = ((size_t)row * a.h + head) * a.nsplit + split;
            a.part_acc[pi * HD + d] = A;
            if (d == 0) { a.part_ml[pi * 2] = M; a.part_ml[pi * 2 + 1] = L; }
        }
    }
}

// Log-sum-exp merge of the context splits: grid (h, nrows), HD threads.
__global__ void attn_merge_kernel(AttnArgs a, int HD) {
    pdl_wait();  // inputs come from the preceding kernel of the step
    pdl_launch_dependents();
    const int head = blockIdx.x, rrow = blockIdx.y, row = kv_row(a.kv, a.row0, rrow), d = threadIdx.x;
    const size_t p0 = ((size_t)row * a.h + head) * a.nsplit;
    float M = -INFINITY;
    for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, a.part_ml[(p0 + s) * 2]);
    float L = 0.f, A = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
        const float m = a.part_ml[(p0 + s) * 2];
        const float e = (m == -INFINITY) ? 0.f : expf(m - M);
        L += e * a.part_ml[(p0 + s) * 2 + 1];
        A += e * a.part_acc[(p0 + s) * HD + d];
    }
    const float o = L > 0.f ? A * (1.0f / L) : A;
    store_act(a.out, a.dtype, (size_t)((long long)rrow * a.st.o_b + (long long)head * a.st.o_h + d), o);
}

template <int KVD, int HD>
static void launch_split(const AttnArgs &a, dim3 grid, cudaStream_t s) {
    if (a.rep == 1) attn_split_kernel<KVD, HD, 1><<<grid, 128, 0, s>>>(a);
    else if (a.rep == 2) attn_split_kernel<KVD, HD, 2><<<grid, 128, 0, s>>>(a);
    else if (a.rep <= 4) attn_split_kernel<KVD, HD, 4><<<grid, 128, 0, s>>>(a);
    else attn_split_kernel<KVD, HD, 8><<<grid, 128, 0, s>>>(a);
}

template <int KVD>
static int launch_split_hd(const AttnArgs &a, dim3 grid, cudaStream_t s) {
    switch (a.kv.hd) {
    case 64: launch_split<KVD, 64>(a, grid, s); break;
    case 128: launch_split<KVD, 128>(a, grid, s); break;
    default:
        return fail(AB2_ERR_UNSUPPORTED, "attention supports head_dim 64 and 128, got %d", a.kv.hd);
    }
    return AB2_OK;
}

int device_sm_count();

// Whether decode queries over this cache take the tensor-core flash-decode (attention_mma.cu).
static bool decode_on_mma(const ab2_kv *kv) {
    return kv->dtype == AB2_KV_INT8 && kv->hd == 128 && kv->h / kv->kvh <= 8;
}

// Context splits of a decode launch over `nrows` sequences of at most `max_len` tokens: enough
// CTAs to fill the GPU a few times over, never a split shorter than a useful run of tokens.
// One rule for every entry point, so that they return the same bits.
static int decode_split_count(const ab2_kv *kv, int nrows, int max_len, int max_splits, bool mma) {
    const int sms = device_sm_count(), units = nrows * kv->kvh;
    if (mma) {
        // short contexts with at least one (row, KV head) per SM: one CTA each and no merge launch
        // (32 rows x 512 tokens: 4.35 ms per decode step against 4.62 with four splits)
        if (units >= sms && max_len <= 1024) return 1;
        const int want = (sms * 6 + units - 1) / units;
        return std::max(1, std::min(std::min(want, (max_len + 63) / 64), max_splits));
    }
    const int want = (2 * sms + units - 1) / units;
    return std::max(1, std::min(std::min(want, (max_len + 255) / 256), max_splits));
}

int attention_cached_device(const ab2_kv *kv, int layer, const void *q, void *out, int S, int pending,
                            int row0, int nrows, float scale, ab2_dtype dtype, AttnStrides st,
                            int len_hint, cudaStream_t s) {
    AttnArgs a;
    a.kv = kv_view(kv, layer);
    a.q = q; a.out = out; a.st = st; a.S = S; a.pending = pending; a.row0 = row0; a.h = kv->h;
    a.rep = kv->h / kv->kvh;
    a.dtype = (int)dtype; a.scale = scale; a.part_acc = kv->part_acc; a.part_ml = kv->part_ml;
    int max_len = len_hint;
    if (max_len <= 0)
        for (int i = 0; i < nrows; ++i) max_len = std::max(max_len, kv->lens_host[kv_row_host(kv, row0, i)] + pending);
    int nsplit = 1;
    if (S == 1 && decode_on_mma(kv) && st.q_h == kv->hd && st.o_h == st.q_h && st.o_b == (long long)kv->h * kv->hd) {
        // INT8 cache, head_dim 128: tensor-core flash-decode (attention_mma.cu)
        nsplit = decode_split_count(kv, nrows, max_len, kv->max_splits, true);
        a.nsplit = nsplit;
        int rc = attention_decode_mma_device(kv, layer, q, out, row0, nrows, scale, dtype, nsplit, kv->part_acc,
                                             kv->part_ml, pending, st.q_b, s);
        if (rc != AB2_OK) return rc;
        if (nsplit > 1) {
            cudaError_t e = launch_kernel(attn_merge_kernel, dim3(kv->h, nrows), dim3(kv->hd), 0, s, a, (int)kv->hd);
            if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "attention merge launch failed: %s", cudaGetErrorString(e));
        }
        return AB2_OK;
    }
    if (S > 1) {
        // prefill chunk over an INT8 cache: the tensor-core causal kernel (attention_mma.cu)
        static const bool scalar_prefill = getenv("AB2_SCALAR_PREFILL_ATTN") != nullptr;  // measurement switch
        if (!scalar_prefill) {
            int rc = attention_prefill_mma_device(kv, layer, q, out, S, pending, row0, nrows, scale, dtype, st, s);
            if (rc != AB2_ERR_UNSUPPORTED) return rc;
        }
    }
    if (S == 1) nsplit = decode_split_count(kv, nrows, max_len, kv->max_splits, false);
    a.nsplit = nsplit;
    dim3 grid(nsplit, kv->kvh, nrows * S);
    int rc;
    if (kv->dtype == AB2_KV_F32) rc = launch_split_hd<AB2_KV_F32>(a, grid, s);
    else if (kv->dtype == AB2_KV_BF16) rc = launch_split_hd<AB2_KV_BF16>(a, grid, s);
    else rc = launch_split_hd<AB2_KV_INT8>(a, grid, s);
    if (rc != AB2_OK) return rc;
    if (nsplit > 1) attn_merge_kernel<<<dim3(kv->h, nrows), kv->hd, 0, s>>>(a, kv->hd);
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

// Any head_dim (used for shapes outside the streaming kernel's 64 / 128): one
// warp per (b, head, query) row, lanes stride over head_dim, single-pass online
// softmax in the reference's order (one key at a time,
// crates/aarambh-studio-kernel/src/cpu/parallel_attn.rs:196-233).
template <typename T>
__global__ void attn_rowwise_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                                    T *out, int b, int h, int kvh, int q_len, int kv_len, int hd, float scale) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= b * h * q_len) return;
    const int qi = row % q_len, head = (row / q_len) % h, batch = row / (h * q_len);
    const int kvhead = head / (h / kvh), shift = kv_len - q_len;
    const T *qr = q + (size_t)row * hd;
    float acc[8];  // head_dim <= 256
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int t = 0; t <= shift + qi; ++t) {
        const size_t off = (((size_t)batch * kvh + kvhead) * kv_len + t) * hd;
        float dot = 0.f;
        for (int d = lane; d < hd; d += 32) dot = fmaf(to_f32(qr[d]), to_f32(k[off + d]), dot);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = dot * scale;
        const float mn = fmaxf(m, s), os = expf(m - mn), ns = expf(s - mn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = lane + 32 * j;
            if (d < hd) acc[j] = acc[j] * os + ns * to_f32(v[off + d]);
        }
        l = l * os + ns;
        m = mn;
    }
    const float inv = l > 0.f ? 1.0f / l : 1.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) out[(size_t)row * hd + d] = from_f32<T>(acc[j] * inv);
    }
}

}  // namespace ab2

static int check_attention(const ab2_kv *kv, int layer, const void *q, const void *out, int S, int row0,
                           int nrows, ab2_dtype dtype) {
    AB2_REQUIRE(kv && q && out, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(layer >= 0 && layer < kv->L, AB2_ERR_BAD_SHAPE, "layer %d outside the cache's %d layers", layer, kv->L);
    AB2_REQUIRE(S > 0 && nrows > 0 && row0 >= 0 && row0 + nrows <= kv->B, AB2_ERR_BAD_SHAPE,
                "rows %d..%d outside the cache batch %d", row0, row0 + nrows, kv->B);
    AB2_REQUIRE(dtype == AB2_F32 || dtype == AB2_F16 || dtype == AB2_BF16, AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    for (int r = row0; r < row0 + nrows; ++r)
        AB2_REQUIRE(kv->lens_host[r] >= S, AB2_ERR_BAD_SHAPE,
                    "attention head_dim and kv_seq must be non-zero (row %d holds %d tokens for %d queries)", r, kv->lens_host[r], S);
    return AB2_OK;
}

AB2_API int ab2_attention_decode(const ab2_kv *kv, int layer, const void *q_dev, void *out_dev, int row0,
                                 int nrows, float scale, ab2_dtype dtype, ab2_stream stream) {
    int rc = check_attention(kv, layer, q_dev, out_dev, 1, row0, nrows, dtype);
    if (rc != AB2_OK) return rc;
    AttnStrides st;
    st.q_b = (long long)kv->h * kv->hd; st.q_s = 0; st.q_h = kv->hd;
    st.o_b = st.q_b; st.o_s = 0; st.o_h = kv->hd;
    return attention_cached_device(kv, layer, q_dev, out_dev, 1, 0, row0, nrows, scale, dtype, st, 0, (cudaStream_t)stream);
}

AB2_API int ab2_attention_cached(const ab2_kv *kv, int layer, const void *q_dev, void *out_dev, int S,
                                 int row0, int nrows, float scale, ab2_dtype dtype, ab2_stream stream) {
    int rc = check_attention(kv, layer, q_dev, out_dev, S, row0, nrows, dtype);
    if (rc != AB2_OK) return rc;
    AttnStrides st;  // q, out: [nrows][S][h][hd]
    st.q_h = kv->hd; st.q_s = (long long)kv->h * kv->hd; st.q_b = st.q_s * S;
    st.o_h = st.q_h; st.o_s = st.q_s; st.o_b = st.q_b;
    return attention_cached_device(kv, layer, q_dev, out_dev, S, 0, row0, nrows, scale, dtype, st, 0, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Decode attention for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc while they run: a serving
// loop that has handed all free memory to its own pool, a caller holding a
// lock the allocator would also need, or a process confined to a fixed memory
// budget.  For them the partial results of the context splits live in the
// fixed array below instead of in memory allocated with the cache.  Every GPU
// that loads the library reserves the array until the process exits.
// ---------------------------------------------------------------------------
#define AB2_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)  // 8 MiB
static __device__ __align__(256) float g_static_attn_scratch[AB2_STATIC_SCRATCH_FLOATS];
static float *g_static_attn_scratch_ptr[64] = {nullptr};

AB2_API int ab2_attention_decode_static(const ab2_kv *kv, int layer, const void *q_dev, void *out_dev,
                                        int row0, int nrows, float scale, ab2_dtype dtype,
                                        ab2_stream stream) {
    int rc = check_attention(kv, layer, q_dev, out_dev, 1, row0, nrows, dtype);
    if (rc != AB2_OK) return rc;
    AB2_REQUIRE(kv->hd == 64 || kv->hd == 128, AB2_ERR_UNSUPPORTED, "attention supports head_dim 64 and 128, got %d", kv->hd);
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!g_static_attn_scratch_ptr[dev]) {
        // Once per device, with that device current: the array's name is only a
        // host-side stand-in, kernels need the address the runtime reports.
        float *ptr = nullptr;
        AB2_CUDA(cudaGetSymbolAddress((void **)&ptr, g_static_attn_scratch));
        g_static_attn_scratch_ptr[dev] = ptr;
    }
    AttnArgs a;
    a.kv = kv_view(kv, layer);
    a.q = q_dev; a.out = out_dev; a.S = 1; a.pending = 0; a.row0 = row0; a.h = kv->h; a.rep = kv->h / kv->kvh;
    a.dtype = (int)dtype; a.scale = scale;
    a.st.q_b = (long long)kv->h * kv->hd; a.st.q_s = 0; a.st.q_h = kv->hd;
    a.st.o_b = a.st.q_b; a.st.o_s = 0; a.st.o_h = kv->hd;
    int max_len = 0;
    for (int r = row0; r < row0 + nrows; ++r) max_len = std::max(max_len, kv->lens_host[r]);
    // Kernel choice and split count come from the helpers ab2_attention_decode uses (with the
    // cache's own split limit), so both entry points return the same bits.
    const bool mma_path = decode_on_mma(kv);
    a.nsplit = decode_split_count(kv, nrows, max_len, kv->max_splits, mma_path);
    // Partials are indexed by the absolute row, exactly as in the allocated scratch.
    const size_t parts = (size_t)(row0 + nrows) * kv->h * a.nsplit;
    const size_t need = parts * ((size_t)kv->hd + 2);
    AB2_REQUIRE(a.nsplit == 1 || need <= AB2_STATIC_SCRATCH_FLOATS, AB2_ERR_CAPACITY,
                "decode attention needs %zu floats of split scratch (rows %d, heads %d, splits %d) but the "
                "static scratch holds %u; use ab2_attention_decode",
                need, row0 + nrows, kv->h, a.nsplit, (unsigned)AB2_STATIC_SCRATCH_FLOATS);
    a.part_acc = g_static_attn_scratch_ptr[dev];
    a.part_ml = g_static_attn_scratch_ptr[dev] + parts * kv->hd;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(a.nsplit, kv->kvh, nrows);
    if (mma_path) {
        rc = attention_decode_mma_device(kv, layer, q_dev, out_dev, row0, nrows, scale, dtype, a.nsplit, a.part_acc,
                                         a.part_ml, 0, (long long)kv->h * kv->hd, s);
        if (rc != AB2_OK) return rc;
        if (a.nsplit > 1) attn_merge_kernel<<<dim3(kv->h, nrows), kv->hd, 0, s>>>(a, kv->hd);
        AB2_LAUNCH_CHECK();
        return AB2_OK;
    }
    if (kv->dtype == AB2_KV_F32) rc = launch_split_hd<AB2_KV_F32>(a, grid, s);
    else if (kv->dtype == AB2_KV_BF16) rc = launch_split_hd<AB2_KV_BF16>(a, grid, s);
    else rc = launch_split_hd<AB2_KV_INT8>(a, grid, s);
    if (rc != AB2_OK) return rc;
    if (a.nsplit > 1) attn_merge_kernel<<<dim3(kv->h, nrows), kv->hd, 0, s>>>(a, kv->hd);
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

// dispatch::attention_forward_causal on explicit tensors: q [b,h,q_len,hd],
// k,v [b,kv_heads,kv_len,hd] (not repeated), out [b,h,q_len,hd].
AB2_API int ab2_attention_causal(const void *q_dev, const void *k_dev, const void *v_dev, void *out_dev,
                                 int b, int h, int kv_heads, int q_len, int kv_len, int head_dim,
                                 float scale, ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(q_dev && k_dev && v_dev && out_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(b > 0 && h > 0 && kv_heads > 0 && q_len > 0, AB2_ERR_BAD_SHAPE, "attention dimensions must be positive");
    AB2_REQUIRE(head_dim > 0 && kv_len > 0, AB2_ERR_BAD_SHAPE, "attention head_dim and kv_seq must be non-zero");
    AB2_REQUIRE(h % kv_heads == 0 && h / kv_heads <= 8, AB2_ERR_BAD_SHAPE, "query heads (%d) must be 1..8 times the kv heads (%d)", h, kv_heads);
    AB2_REQUIRE(kv_len >= q_len, AB2_ERR_BAD_SHAPE, "kv_len %d shorter than q_len %d", kv_len, q_len);
    AB2_REQUIRE(dtype == AB2_F32 || dtype == AB2_BF16, AB2_ERR_BAD_DTYPE, "attention on explicit tensors takes f32 or bf16, got %d", (int)dtype);
    if ((head_dim != 64 && head_dim != 128) || ((uintptr_t)k_dev & 15) || ((uintptr_t)v_dev & 15)) {
        AB2_REQUIRE(head_dim <= 256, AB2_ERR_UNSUPPORTED, "head_dim %d exceeds 256", head_dim);
        const int rows = b * h * q_len;
        cudaStream_t s = (cudaStream_t)stream;
        if (dtype == AB2_F32)
            attn_rowwise_kernel<float><<<(rows + 3) / 4, 128, 0, s>>>((const float *)q_dev, (const float *)k_dev, (const float *)v_dev,
                                                                      (float *)out_dev, b, h, kv_heads, q_len, kv_len, head_dim, scale);
        else
            attn_rowwise_kernel<__nv_bfloat16><<<(rows + 3) / 4, 128, 0, s>>>((const __nv_bfloat16 *)q_dev, (const __nv_bfloat16 *)k_dev,
                                                                              (const __nv_bfloat16 *)v_dev, (__nv_bfloat16 *)out_dev, b, h,
                                                                              kv_heads, q_len, kv_len, head_dim, scale);
        AB2_LAUNCH_CHECK();
        return AB2_OK;
    }
    // A borrowed view over the caller's tensors: [b][kv_heads][kv_len][hd] is the cache layout.
    ab2_kv view;
    memset(&view, 0, sizeof(view));
    view.L = 1; view.B = b; view.cap = kv_len; view.kvh = kv_heads; view.hd = head_dim; view.h = h;
    view.dtype = dtype == AB2_F32 ? AB2_KV_F32 : AB2_KV_BF16;
    view.k = const_cast<void *>(k_dev); view.v = const_cast<void *>(v_dev);
    int *lens_dev = nullptr;
    std::vector<int> lens(b, kv_len);
    AB2_CUDA(cudaMalloc((void **)&lens_dev, (size_t)b * 4));
    cudaError_t e = cudaMemcpy(lens_dev, lens.data(), (size_t)b * 4, cudaMemcpyHostToDevice);
    view.lens_dev = lens_dev; view.lens_host = lens.data(); view.max_splits = 1;
    int rc = AB2_OK;
    if (e != cudaSuccess) rc = fail(AB2_ERR_CUDA, "copy failed: %s", cudaGetErrorString(e));
    if (rc == AB2_OK) {
        AttnStrides st;  // [b][h][q_len][hd]
        st.q_s = head_dim; st.q_h = (long long)q_len * head_dim; st.q_b = st.q_h * h;
        st.o_s = st.q_s; st.o_h = st.q_h; st.o_b = st.q_b;
        // q_len queries over a context whose last q_len positions are theirs
        rc = attention_cached_device(&view, 0, q_dev, out_dev, q_len, 0, 0, b, scale, dtype, st, 0, (cudaStream_t)stream);
    }
    if (rc == AB2_OK && cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess)
        rc = fail(AB2_ERR_CUDA, "attention kernel failed");
    cudaFree(lens_dev);
    return rc;
}
