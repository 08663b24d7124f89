// Dense-GQA decoder over packed weights: the device-side counterpart of
// AarambhModel::{forward_with_cache, forward_decode_batch}
// (crates/aarambh-studio-model/src/model.rs:508-641), TransformerBlock::forward
// (crates/aarambh-studio-nn/src/block.rs:331-371), GroupedQueryAttention
// (crates/aarambh-studio-nn/src/attention.rs:170-288) and SwiGluFfn
// (crates/aarambh-studio-nn/src/ffn.rs:29-37).  Q/K/V and gate/up share one
// packed weight each; the one-token step is captured in a CUDA graph.
#include <cmath>
#include <cstring>
#include <map>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "kv_cache.cuh"
#include "ops.cuh"
#include "tp.cuh"
#include "decode_step_persistent.cuh"

using namespace ab2;

namespace ab2 {
int qlinear_dispatch(const ab2_qweight *w, const void *x, int M, ab2_dtype dtype, void *y, cudaStream_t s);
int device_status_word(int **out);
int w4a16_prepare_stream(cudaStream_t s);
bool qlinear_w4a16_norm_fusable(const ab2_qweight *w, ab2_dtype dtype, int M);
int qlinear_w4a16_norm(const ab2_qweight *w, const void *x, const float *norm_w, float eps, void *y, int epi, cudaStream_t s);
int qlinear_w4a16_norm_peer(const ab2_qweight *w, const void *x, const float *norm_w, float eps, void *y, int epi,
                            ab2_tp *tp, void *x_out, cudaStream_t s);
bool qlinear_w4a16_mma_eligible(const ab2_qweight *w, ab2_dtype dtype);
int qlinear_w4a16_mma_add(const ab2_qweight *w, const void *x, int M, void *y, const void *resid, cudaStream_t s);
int qlinear_w4a16_mma_swiglu(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s);
int qlinear_w4a16_mma_f32(const ab2_qweight *w, const void *x, int M, float *y, cudaStream_t s);
int qlinear_w4a16_mma_f32_peer(const ab2_qweight *w, const void *x, int M, ab2_tp *tp, cudaStream_t s);
}
extern "C" int ab2_qweight_interleave_gate_up(ab2_qweight **out, const ab2_qweight *gate, const ab2_qweight *up);

struct LayerWeights {
    const ab2_qweight *part[7];  // wq wk wv wo gate up down (borrowed)
    ab2_qweight *wqkv, *wgu;     // fused (owned)
    float *norm1, *norm2;        // owned, device
};

struct StepGraph {
    cudaGraphExec_t exec;
};

struct ab2_model {
    ab2_model_config cfg;
    ab2_dtype dtype;
    int max_tokens;
    std::vector<LayerWeights> layers;
    const ab2_qweight *embedding, *lm_head;
    float *final_norm;
    float *cos_t, *sin_t;  // [max_seq][head_dim/2]
    bool finalized;
    bool fused_epilogues;  // W4A16 + bf16: residual add and SwiGLU ride the GEMV epilogues
    ab2_tp *tp;            // tensor-parallel context (borrowed), or null
    float *proj32;            // tensor-parallel: f32 partial sums of the row-parallel projections
    void *lg_local, *lg_all;  // tensor-parallel logits: this rank's vocabulary shard / all shards
    // workspace, sized for max_tokens
    void *x, *xn, *qkv, *attn, *proj, *gu, *hid;
    int *positions;        // [max rows] explicit RoPE offsets
    int *positions_host;   // pinned
    std::map<std::tuple<const void *, const void *, int, int, const void *, const void *, int>, StepGraph> graphs;
    // one sequence, one token: the whole step as one persistent kernel (null when not eligible)
    ab2::PersistentStep *persistent;
    std::vector<ab2::PsLayerDesc> ps_layers;
    // device copies of the token ids and greedy tokens of ab2_model_decode_step_host
    uint32_t *host_step_ids, *host_step_out;
    int host_step_rows;
};

namespace ab2 {

// Copies the last token's row of every sequence: in [nrows][S][d] -> out [nrows][d].
template <typename T>
__global__ void gather_last_kernel(const T *in, T *out, int S, int d) {
    const T *src = in + ((size_t)blockIdx.x * S + (S - 1)) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)blockIdx.x * d + i] = src[i];
}

// x = x + round(p), p the all-reduced f32 projection: the residual add of
// TransformerBlock::forward with the projection rounded to bf16 once, after the sum.
__global__ void add_f32_projection_kernel(__nv_bfloat16 *x, const float *p, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + __bfloat162float(__float2bfloat16_rn(p[i])));
}

// SwiGLU over the output of the interleaved gate|up weight: columns come in
// blocks of 16 = 8 gate values followed by the 8 matching up values.
__global__ void swiglu_interleaved8_kernel(const __nv_bfloat16 *gu, __nv_bfloat16 *out, int ffn, size_t n8) {
    pdl_wait();  // inputs come from the preceding kernel of the step
    pdl_launch_dependents();
    // one thread per block of 16 columns: 16 bytes of gate, 16 bytes of up, 16 bytes out
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const int per_row = ffn >> 3;
    const size_t tok = i / per_row;
    const int jb = (int)(i % per_row);
    const uint4 *src = reinterpret_cast<const uint4 *>(gu + tok * 2 * (size_t)ffn + (size_t)jb * 16);
    const uint4 g = src[0], u = src[1];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
        const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xffff0000u);
        o[k] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(swiglu_value(g0, u0))) |
               ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(swiglu_value(g1, u1))) << 16);
    }
    *reinterpret_cast<uint4 *>(out + tok * (size_t)ffn + (size_t)jb * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

// [world][rows][vn] (all-gathered vocabulary shards) -> [rows][world * vn]
template <typename T>
__global__ void reorder_shards_kernel(const T *in, T *out, int rows, int vn, int world) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t n = (size_t)rows * vn * world;
    if (i >= n) return;
    int j = (int)(i % vn);
    int r = (int)((i / vn) % world);
    int b = (int)(i / ((size_t)vn * world));
    out[i] = in[((size_t)r * rows + b) * vn + j];
}

// Decode attention as rotation + append + tensor-core flash-decode (+ merge) instead of the
// one-launch CUDA-core kernels.  The one-launch kernels win while the launch count is what
// matters; they are bound by the int8 -> float conversion once a step reads many cached tokens.
static bool decode_attention_on_tensor_cores(const ab2_kv *kv, int nrows, int max_len) {
    if (kv->dtype != AB2_KV_INT8 || kv->hd != 128 || kv->h / kv->kvh > 8) return false;
    static const char *force = getenv("AB2_DECODE_ATTN");
    if (force) return strcmp(force, "mma") == 0;
    return nrows >= 2 ? nrows * (long long)max_len > 1024 : max_len > 6144;
}

#define STEP(expr)                     \
    do {                               \
        int _rc = (expr);              \
        if (_rc != AB2_OK) return _rc; \
    } while (0)

// out = epilogue(RMSNorm(x; norm_w) . W^T).  One decode token on the W4A16 fast path
// normalises inside the GEMV; otherwise the norm is its own launch into m->xn.
// epi: 0 plain projection (any format), 2 SwiGLU over an interleaved gate|up weight.
static int norm_linear(ab2_model *m, const ab2_qweight *w, const void *x, const float *norm_w, int T, void *out,
                       int epi, cudaStream_t s, bool normed = false) {
    const ab2_model_config &c = m->cfg;
    if (normed) return qlinear_dispatch(w, m->xn, T, m->dtype, out, s);  // m->xn already holds RMSNorm(x; norm_w)
    if (m->fused_epilogues && qlinear_w4a16_norm_fusable(w, m->dtype, T))
        return qlinear_w4a16_norm(w, x, norm_w, c.rms_eps, out, epi, s);
    STEP(launch_rms_norm(x, norm_w, m->xn, T, c.d_model, c.rms_eps, m->dtype, s));
    if (epi == 2) return qlinear_w4a16_mma_swiglu(w, m->xn, T, out, s);
    return qlinear_dispatch(w, m->xn, T, m->dtype, out, s);
}

// The forward pass proper; every launch goes to `s`, nothing synchronises.
static int forward_launches(ab2_model *m, ab2_kv *kv, const uint32_t *ids, int S, int row0, int nrows,
                            const int *rope_base, int logits_mode, void *logits, uint32_t *argmax_out,
                            int len_hint, cudaStream_t s) {
    const ab2_model_config &c = m->cfg;
    const int T = nrows * S, d = c.d_model, hd = c.head_dim;
    const size_t esz = dtype_size(m->dtype);
    const long long qkv_stride = (long long)(c.n_heads + 2 * c.n_kv_heads) * hd;
    const float scale = (float)(1.0 / std::sqrt((double)hd));
    STEP(launch_embedding(m->embedding, ids, T, m->x, m->dtype, s));
    // Tensor parallel, one token: the partial sums of a row-parallel projection stay in the
    // ranks' inboxes ("pending") and the next normalising GEMV adds them to the residual
    // stream in its prologue, writing the new stream to the other of two buffers.
    void *xcur = m->x;
    bool pending = false;
    const bool fuse_exchange = m->tp && m->tp->world > 1 && m->fused_epilogues && T == 1 &&
                               tp_peer_ready(m->tp, (size_t)d) && qlinear_w4a16_norm_fusable(m->layers[0].wqkv, m->dtype, T) &&
                               qlinear_w4a16_norm_fusable(m->lm_head, m->dtype, T) &&  // it consumes the last exchange
                               getenv("AB2_TP_SEPARATE_REDUCE") == nullptr;
    auto consume = [&](const ab2_qweight *w, const float *norm_w, void *out, int epi) -> int {
        void *xnext = xcur == m->x ? m->xn : m->x;
        int rc2 = qlinear_w4a16_norm_peer(w, xcur, norm_w, c.rms_eps, out, epi, m->tp, xnext, s);
        xcur = xnext;
        pending = false;
        return rc2;
    };
    bool xn_ready = false;  // the preceding layer's last residual add also wrote RMSNorm(x; norm1) of this layer
    for (int l = 0; l < c.n_layers; ++l) {
        LayerWeights &L = m->layers[l];
        if (pending) STEP(consume(L.wqkv, L.norm1, m->qkv, 0));
        else STEP(norm_linear(m, L.wqkv, xcur, L.norm1, T, m->qkv, 0, s, xn_ready));
        xn_ready = false;
        int max_len = len_hint;
        if (S == 1 && max_len <= 0)
            for (int i = 0; i < nrows; ++i) max_len = std::max(max_len, kv->lens_host[kv_row_host(kv, row0, i)] + 1);
        if (S == 1 && !decode_attention_on_tensor_cores(kv, nrows, max_len)) {
            // decode: RoPE, KV append, attention and split merge in one launch
            if (attention_decode_cluster_eligible(kv, m->dtype, max_len))
                STEP(attention_decode_cluster_device(kv, l, m->qkv, qkv_stride, m->attn, row0, nrows, scale, m->cos_t,
                                                     m->sin_t, rope_base == kv->lens_dev ? nullptr : rope_base,
                                                     max_len, s));
            else
                STEP(attention_decode_fused_device(kv, l, m->qkv, qkv_stride, m->attn, row0, nrows, scale, m->dtype,
                                                   m->cos_t, m->sin_t, rope_base == kv->lens_dev ? nullptr : rope_base,
                                                   len_hint, s));
        } else {
            // one launch: RoPE on the query heads in place, RoPE + quantise + append of K / V
            const char *kptr = (const char *)m->qkv + (size_t)c.n_heads * hd * esz;
            const char *vptr = kptr + (size_t)c.n_kv_heads * hd * esz;
            STEP(kv_append_device(kv, l, kptr, vptr, qkv_stride, S, row0, nrows, m->dtype, m->cos_t, m->sin_t,
                                  rope_base == kv->lens_dev ? nullptr : rope_base, s, m->qkv, c.n_heads));
            AttnStrides st;
            st.q_h = hd; st.q_s = qkv_stride; st.q_b = qkv_stride * S;
            st.o_h = hd; st.o_s = (long long)c.n_heads * hd; st.o_b = st.o_s * S;
            STEP(attention_cached_device(kv, l, m->qkv, m->attn, S, S, row0, nrows, scale, m->dtype, st, len_hint, s));
        }
        const bool tp = m->tp && m->tp->world > 1;
        if (tp) {
            // row-parallel O and down produce partial sums: all-reduce, then the residual add
            const size_t nd = (size_t)T * d;
            if (m->fused_epilogues) {
                // f32 partial sums meet either in the ranks' inboxes over NVLink (the projection
                // stores them there; one small kernel per exchange) or through NCCL
                const bool peer = T <= 16 && tp_peer_ready(m->tp, nd);
                if (fuse_exchange) {
                    STEP(qlinear_w4a16_mma_f32_peer(L.part[3], m->attn, T, m->tp, s));
                    STEP(consume(L.wgu, L.norm2, m->hid, 2));
                    STEP(qlinear_w4a16_mma_f32_peer(L.part[6], m->hid, T, m->tp, s));
                    pending = true;
                    continue;
                }
                if (peer) {
                    STEP(qlinear_w4a16_mma_f32_peer(L.part[3], m->attn, T, m->tp, s));
                    STEP(tp_peer_reduce_add(m->tp, m->x, nd, s));
                } else {
                    STEP(qlinear_w4a16_mma_f32(L.part[3], m->attn, T, m->proj32, s));
                    STEP(tp_all_reduce(m->tp, m->proj32, nd, AB2_F32, s));
                    add_f32_projection_kernel<<<(unsigned)ceil_div(nd, 256), 256, 0, s>>>((__nv_bfloat16 *)m->x, m->proj32, nd);
                }
                STEP(norm_linear(m, L.wgu, m->x, L.norm2, T, m->hid, 2, s));
                if (peer) {
                    STEP(qlinear_w4a16_mma_f32_peer(L.part[6], m->hid, T, m->tp, s));
                    STEP(tp_peer_reduce_add(m->tp, m->x, nd, s));
                } else {
                    STEP(qlinear_w4a16_mma_f32(L.part[6], m->hid, T, m->proj32, s));
                    STEP(tp_all_reduce(m->tp, m->proj32, nd, AB2_F32, s));
                    add_f32_projection_kernel<<<(unsigned)ceil_div(nd, 256), 256, 0, s>>>((__nv_bfloat16 *)m->x, m->proj32, nd);
                }
                AB2_LAUNCH_CHECK();
            } else {
                STEP(qlinear_dispatch(L.part[3], m->attn, T, m->dtype, m->proj, s));
                STEP(tp_all_reduce(m->tp, m->proj, nd, m->dtype, s));
                STEP(launch_add(m->x, m->proj, m->x, nd, m->dtype, s));
                STEP(launch_rms_norm(m->x, L.norm2, m->xn, T, d, c.rms_eps, m->dtype, s));
                STEP(qlinear_dispatch(L.wgu, m->xn, T, m->dtype, m->gu, s));
                STEP(launch_swiglu_fused(m->gu, m->hid, T, c.ffn_hidden, m->dtype, s));
                STEP(qlinear_dispatch(L.part[6], m->hid, T, m->dtype, m->proj, s));
                STEP(tp_all_reduce(m->tp, m->proj, nd, m->dtype, s));
                STEP(launch_add(m->x, m->proj, m->x, nd, m->dtype, s));
            }
        } else if (m->fused_epilogues && T > 16) {
            // many tokens: tensor-core GEMMs, then the element-wise steps as their own launches (from 17
            // tokens on this measured faster than the residual / SwiGLU epilogues of the decode GEMM:
            // 6330 against 6120 tok/s at 32 rows, 7360 against 6740 at 64; with the strip kernel on the
            // gate|up weight, 7980 against 7850 at 32 rows)
            STEP(qlinear_dispatch(L.part[3], m->attn, T, m->dtype, m->proj, s));
            STEP(launch_add_rms_norm(m->x, m->proj, L.norm2, m->xn, T, d, c.rms_eps, m->dtype, s));
            STEP(qlinear_dispatch(L.wgu, m->xn, T, m->dtype, m->gu, s));
            {
                size_t n8 = (size_t)T * (c.ffn_hidden / 8);
                cudaError_t e = launch_kernel(swiglu_interleaved8_kernel, dim3((unsigned)ceil_div(n8, 256)), dim3(256), 0, s,
                                              (const __nv_bfloat16 *)m->gu, (__nv_bfloat16 *)m->hid, (int)c.ffn_hidden, n8);
                if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "SwiGLU launch failed: %s", cudaGetErrorString(e));
            }
            STEP(qlinear_dispatch(L.part[6], m->hid, T, m->dtype, m->proj, s));
            if (l + 1 < c.n_layers) {  // the add and the next layer's first normalisation in one launch
                STEP(launch_add_rms_norm(m->x, m->proj, m->layers[l + 1].norm1, m->xn, T, d, c.rms_eps, m->dtype, s));
                xn_ready = true;
            } else {
                STEP(launch_add(m->x, m->proj, m->x, (size_t)T * d, m->dtype, s));
            }
        } else if (m->fused_epilogues) {
            STEP(qlinear_w4a16_mma_add(L.part[3], m->attn, T, m->x, m->x, s));
            STEP(norm_linear(m, L.wgu, m->x, L.norm2, T, m->hid, 2, s));
            STEP(qlinear_w4a16_mma_add(L.part[6], m->hid, T, m->x, m->x, s));
        } else {
            STEP(qlinear_dispatch(L.part[3], m->attn, T, m->dtype, m->proj, s));
            STEP(launch_add(m->x, m->proj, m->x, (size_t)T * d, m->dtype, s));
            STEP(launch_rms_norm(m->x, L.norm2, m->xn, T, d, c.rms_eps, m->dtype, s));
            STEP(qlinear_dispatch(L.wgu, m->xn, T, m->dtype, m->gu, s));
            STEP(launch_swiglu_fused(m->gu, m->hid, T, c.ffn_hidden, m->dtype, s));
            STEP(qlinear_dispatch(L.part[6], m->hid, T, m->dtype, m->proj, s));
            STEP(launch_add(m->x, m->proj, m->x, (size_t)T * d, m->dtype, s));
        }
    }
    if (logits_mode == 0 && argmax_out == nullptr) return AB2_OK;
    const void *hidden = xcur;
    int rows = T;
    if (logits_mode != 2 && S > 1) {  // only the last token of each row is needed
        switch (m->dtype) {
        case AB2_F32: gather_last_kernel<float><<<nrows, 128, 0, s>>>((const float *)m->x, (float *)m->proj, S, d); break;
        case AB2_F16: gather_last_kernel<__half><<<nrows, 128, 0, s>>>((const __half *)m->x, (__half *)m->proj, S, d); break;
        default: gather_last_kernel<__nv_bfloat16><<<nrows, 128, 0, s>>>((const __nv_bfloat16 *)m->x, (__nv_bfloat16 *)m->proj, S, d); break;
        }
        hidden = m->proj;
        rows = nrows;
    }
    void *lg = logits ? logits : m->gu;  // scratch when only the argmax is wanted
    if (m->tp && m->tp->world > 1) {
        // vocabulary-parallel LM head: local shard, all-gather, reorder to [rows][vocab]
        const int vn = c.vocab / m->tp->world;
        if (pending) STEP(consume(m->lm_head, m->final_norm, m->lg_local, 0));
        else STEP(norm_linear(m, m->lm_head, hidden, m->final_norm, rows, m->lg_local, 0, s));
        if (!logits && argmax_out && rows == nrows && rows <= AB2_TP_ARGMAX_ROWS && m->tp->attached) {
            // only the sampled token is wanted: local argmax, one (value, index) pair per rank over NVLink
            return tp_peer_argmax(m->tp, m->lg_local, rows, vn, m->dtype, argmax_out, s);
        }
        void *gathered = rows == 1 ? lg : m->lg_all;
        STEP(tp_all_gather(m->tp, m->lg_local, gathered, (size_t)rows * vn, m->dtype, s));
        if (rows > 1) {
            size_t n = (size_t)rows * c.vocab;
            unsigned blocks = (unsigned)ceil_div(n, 256);
            if (esz == 4) reorder_shards_kernel<float><<<blocks, 256, 0, s>>>((const float *)m->lg_all, (float *)lg, rows, vn, m->tp->world);
            else reorder_shards_kernel<uint16_t><<<blocks, 256, 0, s>>>((const uint16_t *)m->lg_all, (uint16_t *)lg, rows, vn, m->tp->world);
            AB2_LAUNCH_CHECK();
        }
    } else {
        STEP(norm_linear(m, m->lm_head, hidden, m->final_norm, rows, lg, 0, s));
    }
    if (argmax_out) {
        // last token of each row
        const char *src = (const char *)lg;
        if (rows == T && S > 1) {
            return fail(AB2_ERR_UNSUPPORTED, "argmax with all-token logits needs S == 1");
        }
        STEP(launch_argmax(src, nrows, c.vocab, m->dtype, argmax_out, s));
    }
    return AB2_OK;
}

static int check_forward(ab2_model *m, ab2_kv *kv, const void *ids, int S, int row0, int nrows,
                         const int *offsets_host, int logits_mode, const void *logits) {
    AB2_REQUIRE(m && kv && ids, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(m->finalized, AB2_ERR_BAD_ARG, "model is not finalised");
    const ab2_model_config &c = m->cfg;
    AB2_REQUIRE(kv->L == c.n_layers, AB2_ERR_BAD_SHAPE, "expected %d cache layers, got %d", c.n_layers, kv->L);
    AB2_REQUIRE(kv->kvh == c.n_kv_heads && kv->hd == c.head_dim && kv->h == c.n_heads, AB2_ERR_BAD_SHAPE,
                "KV cache head layout does not match the model");
    AB2_REQUIRE(S > 0 && nrows > 0 && row0 >= 0 && row0 + nrows <= kv->B, AB2_ERR_BAD_SHAPE,
                "rows %d..%d outside the cache batch %d", row0, row0 + nrows, kv->B);
    for (int r = 0; r < nrows; ++r) {
        const int row = kv_row_host(kv, row0, r);
        AB2_REQUIRE(row >= 0 && row < kv->B, AB2_ERR_BAD_SHAPE, "selected row %d outside the cache batch %d", row, kv->B);
        for (int q = 0; q < r; ++q)
            AB2_REQUIRE(kv_row_host(kv, row0, q) != row, AB2_ERR_BAD_ARG, "cache row %d is selected twice", row);
    }
    AB2_REQUIRE(nrows * S <= m->max_tokens, AB2_ERR_CAPACITY, "%d tokens exceed the model workspace of %d", nrows * S, m->max_tokens);
    AB2_REQUIRE(logits_mode >= 0 && logits_mode <= 2, AB2_ERR_BAD_ARG, "logits_mode must be 0, 1 or 2");
    AB2_REQUIRE(logits_mode == 0 || logits != nullptr, AB2_ERR_BAD_ARG, "logits buffer is null");
    for (int r = 0; r < nrows; ++r) {
        const int crow = kv_row_host(kv, row0, r);
        int off = offsets_host ? offsets_host[r] : kv->lens_host[crow];
        AB2_REQUIRE(off >= 0 && off + S <= c.max_seq, AB2_ERR_BAD_SHAPE,
                    "batch row %d offset %d exceeds max_seq_len %d", r, off, c.max_seq);
        AB2_REQUIRE(kv->lens_host[crow] + S <= kv->cap, AB2_ERR_CAPACITY, "KV cache length %d exceeds capacity %d",
                    kv->lens_host[crow] + S, kv->cap);
    }
    return AB2_OK;
}

}  // namespace ab2

AB2_API int ab2_model_create(ab2_model **out, const ab2_model_config *cfg, ab2_dtype dtype, int max_tokens) {
    AB2_REQUIRE(out && cfg, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(cfg->n_layers > 0 && cfg->d_model > 0 && cfg->n_heads > 0 && cfg->n_kv_heads > 0 &&
                    cfg->head_dim > 0 && cfg->ffn_hidden > 0 && cfg->vocab > 0 && cfg->max_seq > 0,
                AB2_ERR_BAD_SHAPE, "model dimensions must be positive");
    AB2_REQUIRE(cfg->n_heads % cfg->n_kv_heads == 0, AB2_ERR_BAD_SHAPE, "n_heads must be a multiple of n_kv_heads");
    AB2_REQUIRE(cfg->head_dim % 2 == 0, AB2_ERR_BAD_SHAPE, "head_dim must be even");
    AB2_REQUIRE(dtype == AB2_F32 || dtype == AB2_F16 || dtype == AB2_BF16, AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    AB2_REQUIRE(max_tokens > 0, AB2_ERR_BAD_SHAPE, "max_tokens must be positive");
    ab2_model *m = new ab2_model();
    m->cfg = *cfg; m->dtype = dtype; m->max_tokens = max_tokens;
    m->layers.resize(cfg->n_layers);
    for (auto &L : m->layers) memset(&L, 0, sizeof(L));
    m->embedding = m->lm_head = nullptr;
    m->final_norm = m->cos_t = m->sin_t = nullptr;
    m->finalized = false;
    m->x = m->xn = m->qkv = m->attn = m->proj = m->gu = m->hid = nullptr;
    m->positions = nullptr; m->positions_host = nullptr;
    m->tp = nullptr; m->lg_local = m->lg_all = nullptr; m->proj32 = nullptr; m->fused_epilogues = false;
    m->persistent = nullptr;
    *out = m;
    return AB2_OK;
}

AB2_API int ab2_model_destroy(ab2_model *m) {
    if (!m) return AB2_OK;
    for (auto &g : m->graphs) cudaGraphExecDestroy(g.second.exec);
    persistent_step_destroy(m->persistent);
    for (auto &L : m->layers) {
        ab2_qweight_destroy(L.wqkv); ab2_qweight_destroy(L.wgu);
        cudaFree(L.norm1); cudaFree(L.norm2);
    }
    cudaFree(m->final_norm); cudaFree(m->cos_t); cudaFree(m->sin_t);
    cudaFree(m->x); cudaFree(m->xn); cudaFree(m->qkv); cudaFree(m->attn); cudaFree(m->proj);
    cudaFree(m->gu); cudaFree(m->hid); cudaFree(m->positions); cudaFree(m->lg_local); cudaFree(m->lg_all); cudaFree(m->proj32);
    if (m->positions_host) cudaFreeHost(m->positions_host);
    cudaFree(m->host_step_ids); cudaFree(m->host_step_out);
    delete m;
    return AB2_OK;
}

AB2_API int ab2_model_set_linear(ab2_model *m, int layer, int which, const ab2_qweight *w) {
    AB2_REQUIRE(m && w, AB2_ERR_BAD_ARG, "null argument");
    const ab2_model_config &c = m->cfg;
    int N = 0, K = 0;
    if (layer < 0) {
        AB2_REQUIRE(which == 0 || which == 1, AB2_ERR_BAD_ARG, "model-level weight index must be 0 (embedding) or 1 (lm_head)");
        N = (which == 1 && m->tp) ? c.vocab / m->tp->world : c.vocab;
        K = c.d_model;
    } else {
        AB2_REQUIRE(layer < c.n_layers && which >= 0 && which < 7, AB2_ERR_BAD_ARG, "layer %d / weight %d out of range", layer, which);
        const int qd = c.n_heads * c.head_dim, kd = c.n_kv_heads * c.head_dim;
        const int Ns[7] = {qd, kd, kd, c.d_model, c.ffn_hidden, c.ffn_hidden, c.d_model};
        const int Ks[7] = {c.d_model, c.d_model, c.d_model, qd, c.d_model, c.d_model, c.ffn_hidden};
        N = Ns[which]; K = Ks[which];
    }
    AB2_REQUIRE(w->N == N && w->K == K, AB2_ERR_BAD_SHAPE, "weight is [%d,%d], expected [%d,%d]", w->N, w->K, N, K);
    if (layer < 0) (which == 0 ? m->embedding : m->lm_head) = w;
    else m->layers[layer].part[which] = w;
    m->finalized = false;
    return AB2_OK;
}

AB2_API int ab2_model_set_norm(ab2_model *m, int layer, int which, const float *weight) {
    AB2_REQUIRE(m && weight, AB2_ERR_BAD_ARG, "null argument");
    const int d = m->cfg.d_model;
    float **slot;
    if (layer < 0) slot = &m->final_norm;
    else {
        AB2_REQUIRE(layer < m->cfg.n_layers && (which == 0 || which == 1), AB2_ERR_BAD_ARG, "layer %d / norm %d out of range", layer, which);
        slot = which == 0 ? &m->layers[layer].norm1 : &m->layers[layer].norm2;
    }
    if (!*slot) AB2_CUDA(cudaMalloc((void **)slot, (size_t)d * 4));
    AB2_CUDA(cudaMemcpy(*slot, weight, (size_t)d * 4, cudaMemcpyDefault));
    return AB2_OK;
}

AB2_API int ab2_model_finalize(ab2_model *m) {
    AB2_REQUIRE(m != nullptr, AB2_ERR_BAD_ARG, "null argument");
    const ab2_model_config &c = m->cfg;
    AB2_REQUIRE(m->embedding && m->final_norm, AB2_ERR_BAD_ARG, "embedding or final norm not set");
    if (!m->lm_head) {
        AB2_REQUIRE(c.tied, AB2_ERR_BAD_ARG, "lm_head not set and embeddings are not tied");
        // the tied head is the whole embedding table; a rank needs its own vocabulary shard
        AB2_REQUIRE(!(m->tp && m->tp->world > 1), AB2_ERR_BAD_ARG,
                    "tensor parallel needs an explicit lm_head shard of %d rows (tied embeddings are not sharded)",
                    c.vocab / (m->tp ? m->tp->world : 1));
        m->lm_head = m->embedding;  // LmHead::tied_with_qat (crates/aarambh-studio-model/src/head.rs:59-64)
    }
    if (m->tp && m->tp->world > 1)  // the context may have been set after the head
        AB2_REQUIRE(m->lm_head->N == c.vocab / m->tp->world, AB2_ERR_BAD_SHAPE,
                    "lm_head shard has %d rows, expected vocab / world = %d", m->lm_head->N, c.vocab / m->tp->world);
    bool fast = true;
    for (int l = 0; l < c.n_layers && fast; ++l)
        for (int i = 0; i < 7; ++i)
            fast = fast && m->layers[l].part[i] && qlinear_w4a16_mma_eligible(m->layers[l].part[i], m->dtype);
    m->fused_epilogues = fast && c.ffn_hidden % 8 == 0;
    for (int l = 0; l < c.n_layers; ++l) {
        LayerWeights &L = m->layers[l];
        for (int i = 0; i < 7; ++i) AB2_REQUIRE(L.part[i] != nullptr, AB2_ERR_BAD_ARG, "layer %d weight %d not set", l, i);
        AB2_REQUIRE(L.norm1 && L.norm2, AB2_ERR_BAD_ARG, "layer %d norms not set", l);
        ab2_qweight_destroy(L.wqkv); L.wqkv = nullptr;
        ab2_qweight_destroy(L.wgu); L.wgu = nullptr;
        const ab2_qweight *qkv[3] = {L.part[0], L.part[1], L.part[2]};
        const ab2_qweight *gu[2] = {L.part[4], L.part[5]};
        int rc = ab2_qweight_concat_rows(&L.wqkv, qkv, 3);
        if (rc != AB2_OK) return rc;
        rc = m->fused_epilogues ? ab2_qweight_interleave_gate_up(&L.wgu, gu[0], gu[1])
                                : ab2_qweight_concat_rows(&L.wgu, gu, 2);
        if (rc != AB2_OK) return rc;
    }
    // RoPE tables: inverse frequencies from an f64 pow cast to f32, angle in f32
    // (crates/aarambh-studio-nn/src/rope_scaling.rs:6-11, rope.rs:54-64).
    const int half = c.head_dim / 2;
    std::vector<float> cosv((size_t)c.max_seq * half), sinv((size_t)c.max_seq * half);
    for (int pos = 0; pos < c.max_seq; ++pos)
        for (int i = 0; i < half; ++i) {
            float inv = (float)(1.0 / std::pow(c.rope_theta, 2.0 * (double)i / (double)c.head_dim));
            float val = (float)pos * inv;
            cosv[(size_t)pos * half + i] = cosf(val);
            sinv[(size_t)pos * half + i] = sinf(val);
        }
    if (!m->cos_t) {
        AB2_CUDA(cudaMalloc((void **)&m->cos_t, cosv.size() * 4));
        AB2_CUDA(cudaMalloc((void **)&m->sin_t, sinv.size() * 4));
    }
    AB2_CUDA(cudaMemcpy(m->cos_t, cosv.data(), cosv.size() * 4, cudaMemcpyHostToDevice));
    AB2_CUDA(cudaMemcpy(m->sin_t, sinv.data(), sinv.size() * 4, cudaMemcpyHostToDevice));
    if (!m->x) {
        const size_t T = m->max_tokens, esz = dtype_size(m->dtype);
        const size_t qkvw = (size_t)(c.n_heads + 2 * c.n_kv_heads) * c.head_dim;
        const size_t guw = std::max((size_t)2 * c.ffn_hidden, (size_t)c.vocab);
        AB2_CUDA(cudaMalloc(&m->x, T * c.d_model * esz));
        AB2_CUDA(cudaMalloc(&m->xn, T * c.d_model * esz));
        AB2_CUDA(cudaMalloc(&m->qkv, T * qkvw * esz));
        AB2_CUDA(cudaMalloc(&m->attn, T * c.n_heads * c.head_dim * esz));
        AB2_CUDA(cudaMalloc(&m->proj, T * c.d_model * esz));
        AB2_CUDA(cudaMalloc(&m->gu, T * guw * esz));
        AB2_CUDA(cudaMalloc(&m->hid, T * c.ffn_hidden * esz));
        if (m->tp && m->tp->world > 1) {
            AB2_CUDA(cudaMalloc(&m->lg_local, T * (c.vocab / m->tp->world) * esz));
            AB2_CUDA(cudaMalloc(&m->lg_all, T * c.vocab * esz));
            AB2_CUDA(cudaMalloc((void **)&m->proj32, T * c.d_model * 4));
        }
        AB2_CUDA(cudaMalloc((void **)&m->positions, (size_t)m->max_tokens * 4));
        AB2_CUDA(cudaMallocHost((void **)&m->positions_host, (size_t)m->max_tokens * 4));
    }
    for (auto &g : m->graphs) cudaGraphExecDestroy(g.second.exec);
    m->graphs.clear();
    int *status_word = nullptr;  // allocate the device status word outside any capture
    int rc = device_status_word(&status_word);
    if (rc != AB2_OK) return rc;
    persistent_step_destroy(m->persistent);
    m->persistent = nullptr;
    if (m->fused_epilogues && !(m->tp && m->tp->world > 1)) {
        m->ps_layers.resize(c.n_layers);
        for (int l = 0; l < c.n_layers; ++l) {
            const LayerWeights &L = m->layers[l];
            m->ps_layers[l] = PsLayerDesc{L.wqkv, L.part[3], L.wgu, L.part[6], L.norm1, L.norm2};
        }
        PsModelDesc d;
        d.n_layers = c.n_layers; d.d_model = c.d_model; d.n_heads = c.n_heads; d.n_kv_heads = c.n_kv_heads;
        d.head_dim = c.head_dim; d.ffn_hidden = c.ffn_hidden; d.vocab = c.vocab; d.eps = c.rms_eps;
        d.embedding = m->embedding; d.lm_head = m->lm_head; d.final_norm = m->final_norm;
        d.layers = m->ps_layers.data();
        d.x = m->x; d.qkv = m->qkv; d.attn = m->attn; d.hid = m->hid;
        d.cos_t = m->cos_t; d.sin_t = m->sin_t;
        rc = persistent_step_create(&m->persistent, d);
        if (rc != AB2_OK) return rc;
    }
    m->finalized = true;
    return AB2_OK;
}

AB2_API int ab2_model_set_tp(ab2_model *m, ab2_tp *tp) {
    AB2_REQUIRE(m != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(m->x == nullptr, AB2_ERR_BAD_ARG, "set the tensor-parallel context before the model is finalised");
    if (tp) AB2_REQUIRE(m->cfg.vocab % tp->world == 0, AB2_ERR_BAD_SHAPE, "vocab %d is not divisible by the world size %d", m->cfg.vocab, tp->world);
    m->tp = tp;
    return AB2_OK;
}

AB2_API int ab2_model_rope_tables(const ab2_model *m, const float **cos_dev, const float **sin_dev) {
    AB2_REQUIRE(m && m->finalized, AB2_ERR_BAD_ARG, "model is not finalised");
    if (cos_dev) *cos_dev = m->cos_t;
    if (sin_dev) *sin_dev = m->sin_t;
    return AB2_OK;
}

AB2_API int ab2_model_forward(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, int S, int row0, int nrows,
                              const int *offsets_host, int logits_mode, void *logits_dev,
                              uint32_t *argmax_dev, ab2_stream stream) {
    int rc = check_forward(m, kv, ids_dev, S, row0, nrows, offsets_host, logits_mode, logits_dev);
    if (rc != AB2_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const int *rope_base = kv->lens_dev;
    if (offsets_host) {
        bool same = true;
        for (int r = 0; r < nrows; ++r) same = same && offsets_host[r] == kv->lens_host[kv_row_host(kv, row0, r)];
        if (!same) {
            AB2_REQUIRE(!kv->rows_on, AB2_ERR_UNSUPPORTED, "a forward over selected rows takes the cache lengths as offsets");
            // explicit seqlen offsets that differ from the cache lengths
            AB2_CUDA(cudaStreamSynchronize(s));
            // the buffers hold max_tokens entries and nrows <= max_tokens: they are filled from
            // entry 0, and the kernels, which index by the absolute cache row, get the base moved back
            for (int r = 0; r < nrows; ++r) m->positions_host[r] = offsets_host[r];
            AB2_CUDA(cudaMemcpyAsync(m->positions, m->positions_host, (size_t)nrows * 4, cudaMemcpyHostToDevice, s));
            rope_base = m->positions - row0;
        }
    }
    rc = forward_launches(m, kv, ids_dev, S, row0, nrows, rope_base, logits_mode, logits_dev, argmax_dev, 0, s);
    if (rc != AB2_OK) return rc;
    return kv_commit_device(kv, S, row0, nrows, s);
}

// Selects `nrows` cache rows for the call that follows: the list goes to the cache's pinned
// mirror and, in stream order, to the device copy the kernels read.
static int select_rows(ab2_kv *kv, const int *rows_host, int nrows, cudaStream_t s) {
    AB2_REQUIRE(kv && rows_host, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(nrows > 0 && nrows <= kv->B, AB2_ERR_BAD_SHAPE, "%d rows selected, the cache holds %d", nrows, kv->B);
    // the pinned list may still be in flight to the device from the previous call on this stream
    AB2_CUDA(cudaStreamSynchronize(s));
    for (int i = 0; i < nrows; ++i) kv->rows_host[i] = rows_host[i];
    AB2_CUDA(cudaMemcpyAsync(kv->rows_dev, kv->rows_host, (size_t)nrows * 4, cudaMemcpyHostToDevice, s));
    kv->rows_on = true;
    return AB2_OK;
}

AB2_API int ab2_model_forward_rows(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, int S, const int *rows_host,
                                   int nrows, int logits_mode, void *logits_dev, uint32_t *argmax_dev,
                                   ab2_stream stream) {
    int rc = select_rows(kv, rows_host, nrows, (cudaStream_t)stream);
    if (rc != AB2_OK) return rc;
    rc = ab2_model_forward(m, kv, ids_dev, S, 0, nrows, nullptr, logits_mode, logits_dev, argmax_dev, stream);
    kv->rows_on = false;
    return rc;
}

AB2_API int ab2_model_decode_step_rows(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, const int *rows_host,
                                       int nrows, void *logits_dev, uint32_t *argmax_dev, ab2_stream stream) {
    int rc = select_rows(kv, rows_host, nrows, (cudaStream_t)stream);
    if (rc != AB2_OK) return rc;
    rc = ab2_model_decode_step(m, kv, ids_dev, 0, nrows, logits_dev, argmax_dev, stream);
    kv->rows_on = false;
    return rc;
}

AB2_API int ab2_model_step_trace(const ab2_model *m, unsigned long long *values_host, int capacity, int *nphases) {
    AB2_REQUIRE(m && values_host && nphases, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(m->persistent != nullptr, AB2_ERR_UNSUPPORTED, "this model does not run its decode step as one persistent kernel");
    return persistent_step_trace(m->persistent, values_host, capacity, nphases);
}

AB2_API int ab2_model_decode_step(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, int row0, int nrows,
                                  void *logits_dev, uint32_t *argmax_dev, ab2_stream stream) {
    int rc = check_forward(m, kv, ids_dev, 1, row0, nrows, nullptr, logits_dev ? 1 : 0, logits_dev);
    if (rc != AB2_OK) return rc;
    AB2_REQUIRE(logits_dev || argmax_dev, AB2_ERR_BAD_ARG, "decode step needs a logits or an argmax output");
    cudaStream_t s = (cudaStream_t)stream;
    if (s == nullptr || s == cudaStreamLegacy) {
        // the legacy default stream cannot be captured: run the step as plain launches
        rc = forward_launches(m, kv, ids_dev, 1, row0, nrows, kv->lens_dev, logits_dev ? 1 : 0, logits_dev, argmax_dev, 0, s);
        if (rc != AB2_OK) return rc;
        return kv_commit_device(kv, 1, row0, nrows, s);
    }
    // The attention launch is shaped by the context length (splits, kernel choice), which a captured
    // launch cannot read: graphs are kept per power-of-two bound of the longest row.
    int longest = 1;
    for (int i = 0; i < nrows; ++i) longest = std::max(longest, kv->lens_host[kv_row_host(kv, row0, i)] + 1);
    if (nrows == 1 && !kv->rows_on && m->persistent && persistent_step_serves(m->persistent, kv, longest)) {
        // one sequence: the whole step is one persistent kernel (no graph needed)
        void *lg = logits_dev ? logits_dev : m->gu;
        rc = persistent_step_launch(m->persistent, kv, ids_dev, row0, lg, argmax_dev, s);
        if (rc == AB2_OK) {
            kv->lens_host[row0] += 1;
            return AB2_OK;
        }
        // the launch was refused (for instance, not every CTA can be resident): use the graph path from now on
        persistent_step_destroy(m->persistent);
        m->persistent = nullptr;
    }
    int len_bound = 512;
    while (len_bound < longest) len_bound <<= 1;
    len_bound = std::min(len_bound, kv->cap);
    auto key = std::make_tuple((const void *)kv, (const void *)ids_dev, kv->rows_on ? -1 : row0, nrows, (const void *)logits_dev,
                               (const void *)argmax_dev, len_bound);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        cudaGraph_t graph = nullptr;
        rc = w4a16_prepare_stream(s);  // scratch of the GEMV is allocated outside the capture
        if (rc != AB2_OK) return rc;
        AB2_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        g_pdl_launch = m->fused_epilogues;  // every kernel of the fast path takes part in the chain
        rc = forward_launches(m, kv, ids_dev, 1, row0, nrows, kv->lens_dev, logits_dev ? 1 : 0, logits_dev, argmax_dev, len_bound, s);
        if (rc == AB2_OK) {
            // lengths advance inside the graph; the host mirror is advanced per replay
            std::vector<int> keep(kv->lens_host, kv->lens_host + kv->B);
            rc = kv_commit_device(kv, 1, row0, nrows, s);
            memcpy(kv->lens_host, keep.data(), (size_t)kv->B * 4);
        }
        g_pdl_launch = false;
        cudaError_t e = cudaStreamEndCapture(s, &graph);
        if (rc != AB2_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        StepGraph sg;
        e = cudaGraphInstantiate(&sg.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "graph instantiation failed: %s", cudaGetErrorString(e));
        it = m->graphs.emplace(key, sg).first;
    }
    AB2_CUDA(cudaGraphLaunch(it->second.exec, s));
    for (int i = 0; i < nrows; ++i) kv->lens_host[kv_row_host(kv, row0, i)] += 1;
    return AB2_OK;
}

// The same step for a caller that holds its tokens on the host (the serving loop of the
// reference does: InferenceEngine::decode_sessions takes and returns host tokens,
// crates/aarambh-studio-inference/src/engine.rs:323-355): ids in, greedy tokens out, one call,
// one wait.  The device copies live in the model, so every call replays the same graph.
AB2_API int ab2_model_decode_step_host(ab2_model *m, ab2_kv *kv, const uint32_t *ids_host, int row0, int nrows,
                                       uint32_t *argmax_host, ab2_stream stream) {
    AB2_REQUIRE(m && kv && ids_host && argmax_host, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(nrows >= 1, AB2_ERR_BAD_ARG, "nrows must be at least 1, got %d", nrows);
    cudaStream_t s = (cudaStream_t)stream;
    if (m->host_step_rows < nrows) {
        AB2_CUDA(cudaStreamSynchronize(s));  // a step in flight may still use the old buffers
        cudaFree(m->host_step_ids);
        cudaFree(m->host_step_out);
        m->host_step_ids = m->host_step_out = nullptr;
        m->host_step_rows = 0;
        const int cap = std::max(nrows, 8);
        AB2_CUDA(cudaMalloc((void **)&m->host_step_ids, (size_t)cap * sizeof(uint32_t)));
        AB2_CUDA(cudaMalloc((void **)&m->host_step_out, (size_t)cap * sizeof(uint32_t)));
        m->host_step_rows = cap;
    }
    AB2_CUDA(cudaMemcpyAsync(m->host_step_ids, ids_host, (size_t)nrows * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
    int rc = ab2_model_decode_step(m, kv, m->host_step_ids, row0, nrows, nullptr, m->host_step_out, stream);
    if (rc != AB2_OK) return rc;
    AB2_CUDA(cudaMemcpyAsync(argmax_host, m->host_step_out, (size_t)nrows * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    AB2_CUDA(cudaStreamSynchronize(s));
    return AB2_OK;
}
