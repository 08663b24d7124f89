// KV cache: storage, append (with optional fused RoPE and per-token-per-head
// INT8 quantisation), truncate / clear / clone, and read-back.
//
// Storage layout is head-major, [batch][kv_head][capacity][head_dim] (INT8
// caches add f32 scales [batch][kv_head][capacity]), so that the decode
// attention of one (sequence, kv head) streams one contiguous region.  The
// reference keeps [batch, capacity, kv_heads, head_dim]
// (crates/aarambh-studio-nn/src/kvcache.rs:349-368) and transposes on every
// step (crates/aarambh-studio-nn/src/attention.rs:272-276).
#include <cfloat>
#include <cstring>

#include "common.cuh"
#include "kv_cache.cuh"
#include "ops.cuh"

using namespace ab2;

namespace ab2 {

static size_t kv_elem_size(int dtype) { return dtype == AB2_KV_F32 ? 4 : dtype == AB2_KV_BF16 ? 2 : 1; }

// One block per (s, kv head, row); blockDim.x == head_dim.
// k_in / v_in: [nrows][S][kvh][hd].  The vector of one (token, head) is rotated
// (K only, when tables are given), then stored as f32 / bf16, or quantised with
// the absmax arithmetic of crates/aarambh-studio-quant/src/absmax.rs:7-24
// applied to the head_dim vector.
template <typename T, int KVD>
__global__ void kv_append_kernel(KvView kv, const T *__restrict__ k_in, const T *__restrict__ v_in,
                                 long long in_stride, int S, int row0, const float *__restrict__ cos_t,
                                 const float *__restrict__ sin_t, const int *__restrict__ rope_pos,
                                 T *q_rot, int q_heads, int tpb) {
    extern __shared__ float sh[];  // [2][hd] values, then 2 * 8 reduction slots
    pdl_wait();  // inputs come from the preceding kernel of the step
    pdl_launch_dependents();
    const int hd = kv.hd, half = hd >> 1;
    const int head = blockIdx.y, rrow = blockIdx.z, row = kv_row(kv, row0, rrow);
    const int d = threadIdx.x;
    // a block serves `tpb` consecutive tokens of its (row, head): one block per token leaves a long
    // prefill bound by block launches (every branch below is uniform over the block)
    for (int s = blockIdx.x * tpb; s < min(S, (int)(blockIdx.x + 1) * tpb); ++s) {
    if (s != blockIdx.x * tpb) __syncthreads();  // the previous token's values in shared memory have been read
    if (head >= kv.kvh) {
        // blocks past the KV heads rotate one query head in place (same row stride as k / v)
        T *q = q_rot + ((size_t)rrow * S + s) * (size_t)in_stride + (size_t)(head - kv.kvh) * hd;
        sh[d] = to_f32(q[d]);
        __syncthreads();
        const int p = (rope_pos ? rope_pos[row] : kv.lens[row]) + s;
        const int i = d < half ? d : d - half;
        float o1, o2;
        rope_rotate(sh[i], sh[half + i], cos_t[(size_t)p * half + i], sin_t[(size_t)p * half + i], o1, o2);
        q[d] = from_f32<T>(d < half ? o1 : o2);
        continue;
    }
    const int pos = kv.lens[row] + s;
    if (pos >= kv.cap) continue;  // capacity is checked on the host; never write out of range
    const size_t in_off = ((size_t)rrow * S + s) * (size_t)in_stride + (size_t)head * hd;
    float kval = to_f32(k_in[in_off + d]);
    const float vval = to_f32(v_in[in_off + d]);
    if (cos_t != nullptr) {
        sh[d] = kval;
        __syncthreads();
        const int p = (rope_pos ? rope_pos[row] : kv.lens[row]) + s;
        const int i = d < half ? d : d - half;
        const float c = cos_t[(size_t)p * half + i], sn = sin_t[(size_t)p * half + i];
        float o1, o2;
        rope_rotate(sh[i], sh[half + i], c, sn, o1, o2);
        kval = d < half ? o1 : o2;
        // value as the activation dtype would hold it
        kval = to_f32(from_f32<T>(kval));
        __syncthreads();
    }
    const size_t out_off = (((size_t)row * kv.kvh + head) * kv.cap + pos) * hd + d;
    if (KVD == AB2_KV_F32) {
        ((float *)kv.k)[out_off] = kval;
        ((float *)kv.v)[out_off] = vval;
    } else if (KVD == AB2_KV_BF16) {
        ((__nv_bfloat16 *)kv.k)[out_off] = __float2bfloat16_rn(kval);
        ((__nv_bfloat16 *)kv.v)[out_off] = __float2bfloat16_rn(vval);
    } else {
        float ka = fabsf(kval), va = fabsf(vval);
        float *red = sh + 2 * hd;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
            va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o));
        }
        if ((d & 31) == 0) { red[d >> 5] = ka; red[8 + (d >> 5)] = va; }
        __syncthreads();
        float kmax = 0.f, vmax = 0.f;
        for (int w = 0; w < (hd >> 5); ++w) { kmax = fmaxf(kmax, red[w]); vmax = fmaxf(vmax, red[8 + w]); }
        const float kscale = (kmax <= FLT_EPSILON) ? 1.0f : __fdiv_rn(kmax, 127.0f);
        const float vscale = (vmax <= FLT_EPSILON) ? 1.0f : __fdiv_rn(vmax, 127.0f);
        auto enc = [](float x, float sc) -> int8_t {
            float q = roundf(__fdiv_rn(x, sc));
            q = q < -127.f ? -127.f : (q > 127.f ? 127.f : q);
            return (q != q) ? (int8_t)0 : (int8_t)q;
        };
        ((int8_t *)kv.k)[out_off] = enc(kval, kscale);
        ((int8_t *)kv.v)[out_off] = enc(vval, vscale);
        if (d == 0) {
            const size_t soff = ((size_t)row * kv.kvh + head) * kv.cap + pos;
            kv.ks[soff] = kscale;
            kv.vs[soff] = vscale;
        }
    }
    }
}

__global__ void kv_advance_kernel(int *lens, const int *rows, int row0, int nrows, int S) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nrows) lens[rows ? rows[row0 + i] : row0 + i] += S;
}

// Dequantised contents of one sequence in the reference layout [len][kvh][hd].
template <int KVD>
__global__ void kv_read_kernel(KvView kv, int row, int len, float *k_out, float *v_out) {
    size_t n = (size_t)len * kv.kvh * kv.hd;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        int d = (int)(i % kv.hd);
        int head = (int)((i / kv.hd) % kv.kvh);
        int pos = (int)(i / ((size_t)kv.hd * kv.kvh));
        size_t tok = ((size_t)row * kv.kvh + head) * kv.cap + pos;
        size_t off = tok * kv.hd + d;
        if (KVD == AB2_KV_F32) {
            k_out[i] = ((const float *)kv.k)[off];
            v_out[i] = ((const float *)kv.v)[off];
        } else if (KVD == AB2_KV_BF16) {
            k_out[i] = __bfloat162float(((const __nv_bfloat16 *)kv.k)[off]);
            v_out[i] = __bfloat162float(((const __nv_bfloat16 *)kv.v)[off]);
        } else {  // dequantise_i8: code as f32 * scale
            k_out[i] = __fmul_rn((float)((const int8_t *)kv.k)[off], kv.ks[tok]);
            v_out[i] = __fmul_rn((float)((const int8_t *)kv.v)[off], kv.vs[tok]);
        }
    }
}

KvView kv_view(const ab2_kv *kv, int layer) {
    KvView v;
    v.B = kv->B; v.cap = kv->cap; v.kvh = kv->kvh; v.hd = kv->hd; v.dtype = kv->dtype;
    const size_t tokens = (size_t)kv->B * kv->kvh * kv->cap;
    const size_t bytes = tokens * kv->hd * kv_elem_size(kv->dtype);
    v.k = (char *)kv->k + (size_t)layer * bytes;
    v.v = (char *)kv->v + (size_t)layer * bytes;
    v.ks = kv->ks ? kv->ks + (size_t)layer * tokens : nullptr;
    v.vs = kv->vs ? kv->vs + (size_t)layer * tokens : nullptr;
    v.lens = kv->lens_dev;
    v.rows = kv->rows_on ? kv->rows_dev : nullptr;
    return v;
}

template <typename T>
static int launch_append(ab2_kv *kv, int layer, const T *k, const T *v, long long in_stride, int S,
                         int row0, int nrows, const float *cos_t, const float *sin_t,
                         const int *rope_pos, T *q_rot, int q_heads, cudaStream_t s) {
    KvView view = kv_view(kv, layer);
    if (q_rot == nullptr || cos_t == nullptr) q_heads = 0;
    const int tpb = S >= 64 ? 8 : 1;  // tokens per block
    dim3 grid((S + tpb - 1) / tpb, kv->kvh + q_heads, nrows);
    size_t smem = (2 * (size_t)kv->hd + 16) * sizeof(float);
    cudaError_t e;
    if (kv->dtype == AB2_KV_F32)
        e = launch_kernel(kv_append_kernel<T, AB2_KV_F32>, grid, dim3(kv->hd), smem, s, view, k, v, in_stride, S, row0, cos_t, sin_t, rope_pos, q_rot, q_heads, tpb);
    else if (kv->dtype == AB2_KV_BF16)
        e = launch_kernel(kv_append_kernel<T, AB2_KV_BF16>, grid, dim3(kv->hd), smem, s, view, k, v, in_stride, S, row0, cos_t, sin_t, rope_pos, q_rot, q_heads, tpb);
    else
        e = launch_kernel(kv_append_kernel<T, AB2_KV_INT8>, grid, dim3(kv->hd), smem, s, view, k, v, in_stride, S, row0, cos_t, sin_t, rope_pos, q_rot, q_heads, tpb);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "KV append launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

int kv_append_device(ab2_kv *kv, int layer, const void *k, const void *v, long long in_stride, int S,
                     int row0, int nrows, ab2_dtype dtype, const float *cos_t, const float *sin_t,
                     const int *rope_pos, cudaStream_t s, void *q_rot, int q_heads) {
    switch (dtype) {
    case AB2_F32: return launch_append<float>(kv, layer, (const float *)k, (const float *)v, in_stride, S, row0, nrows, cos_t, sin_t, rope_pos, (float *)q_rot, q_heads, s);
    case AB2_F16: return launch_append<__half>(kv, layer, (const __half *)k, (const __half *)v, in_stride, S, row0, nrows, cos_t, sin_t, rope_pos, (__half *)q_rot, q_heads, s);
    default: return launch_append<__nv_bfloat16>(kv, layer, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v, in_stride, S, row0, nrows, cos_t, sin_t, rope_pos, (__nv_bfloat16 *)q_rot, q_heads, s);
    }
}

int kv_commit_device(ab2_kv *kv, int S, int row0, int nrows, cudaStream_t s) {
    kv_advance_kernel<<<(nrows + 127) / 128, 128, 0, s>>>(kv->lens_dev, kv->rows_on ? kv->rows_dev : nullptr, row0, nrows, S);
    AB2_LAUNCH_CHECK();
    for (int i = 0; i < nrows; ++i) kv->lens_host[kv_row_host(kv, row0, i)] += S;
    return AB2_OK;
}

}  // namespace ab2

AB2_API int ab2_kv_create(ab2_kv **out, int n_layers, int batch, int capacity, int kv_heads,
                          int head_dim, int n_heads, ab2_kv_dtype dtype) {
    AB2_REQUIRE(out != nullptr, AB2_ERR_BAD_ARG, "output handle pointer is null");
    AB2_REQUIRE(n_layers > 0 && batch > 0 && capacity > 0 && kv_heads > 0, AB2_ERR_BAD_SHAPE, "KV cache dimensions must be positive");
    AB2_REQUIRE(head_dim >= 32 && head_dim <= 256 && head_dim % 32 == 0, AB2_ERR_BAD_SHAPE,
                "head_dim must be a multiple of 32 in 32..256, got %d", head_dim);
    AB2_REQUIRE(n_heads >= kv_heads && n_heads % kv_heads == 0 && n_heads / kv_heads <= 8, AB2_ERR_BAD_SHAPE,
                "query heads (%d) must be 1..8 times the kv heads (%d)", n_heads, kv_heads);
    AB2_REQUIRE(dtype == AB2_KV_F32 || dtype == AB2_KV_BF16 || dtype == AB2_KV_INT8, AB2_ERR_BAD_DTYPE,
                "unsupported KV dtype %d", (int)dtype);
    ab2_kv *kv = new ab2_kv();
    memset(kv, 0, sizeof(*kv));
    kv->L = n_layers; kv->B = batch; kv->cap = capacity; kv->kvh = kv_heads; kv->hd = head_dim; kv->h = n_heads;
    kv->dtype = dtype;
    size_t elems = (size_t)n_layers * batch * kv_heads * capacity * head_dim;
    size_t esz = kv_elem_size(dtype);
    cudaError_t e = cudaMalloc(&kv->k, elems * esz);
    if (e == cudaSuccess) e = cudaMalloc(&kv->v, elems * esz);
    if (e == cudaSuccess) e = cudaMemset(kv->k, 0, elems * esz);
    if (e == cudaSuccess) e = cudaMemset(kv->v, 0, elems * esz);
    if (e == cudaSuccess && dtype == AB2_KV_INT8) {
        size_t ns = (size_t)n_layers * batch * kv_heads * capacity;
        e = cudaMalloc((void **)&kv->ks, ns * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&kv->vs, ns * 4);
    }
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->lens_dev, (size_t)batch * 4);
    if (e == cudaSuccess) e = cudaMemset(kv->lens_dev, 0, (size_t)batch * 4);
    if (e == cudaSuccess) e = cudaMallocHost((void **)&kv->lens_host, (size_t)batch * 4);
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->rows_dev, (size_t)batch * 4);
    if (e == cudaSuccess) e = cudaMallocHost((void **)&kv->rows_host, (size_t)batch * 4);
    // split-context scratch: partial accumulators and (max, sum) pairs
    kv->max_splits = AB2_KV_MAX_SPLITS;
    size_t nparts = (size_t)batch * n_heads * kv->max_splits;
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->part_acc, nparts * head_dim * 4);
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->part_ml, nparts * 2 * 4);
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->counters, (size_t)batch * kv_heads * 4);
    if (e == cudaSuccess) e = cudaMemset(kv->counters, 0, (size_t)batch * kv_heads * 4);
    if (e != cudaSuccess) {
        ab2_kv_destroy(kv);
        return fail(AB2_ERR_CUDA, "KV cache allocation failed: %s", cudaGetErrorString(e));
    }
    memset(kv->lens_host, 0, (size_t)batch * 4);
    *out = kv;
    return AB2_OK;
}

AB2_API int ab2_kv_destroy(ab2_kv *kv) {
    if (!kv) return AB2_OK;
    cudaFree(kv->k); cudaFree(kv->v); cudaFree(kv->ks); cudaFree(kv->vs); cudaFree(kv->lens_dev);
    cudaFree(kv->part_acc); cudaFree(kv->part_ml); cudaFree(kv->counters);
    if (kv->lens_host) cudaFreeHost(kv->lens_host);
    cudaFree(kv->rows_dev);
    if (kv->rows_host) cudaFreeHost(kv->rows_host);
    delete kv;
    return AB2_OK;
}

static int check_append(const ab2_kv *kv, int layer, const void *k, const void *v, int S, int row0,
                        int nrows, ab2_dtype dtype) {
    AB2_REQUIRE(kv && k && v, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(layer >= 0 && layer < kv->L, AB2_ERR_BAD_SHAPE, "layer %d outside the cache's %d layers", layer, kv->L);
    AB2_REQUIRE(S > 0 && nrows > 0 && row0 >= 0 && row0 + nrows <= kv->B, AB2_ERR_BAD_SHAPE,
                "rows %d..%d outside the cache batch %d", row0, row0 + nrows, kv->B);
    AB2_REQUIRE(dtype == AB2_F32 || dtype == AB2_F16 || dtype == AB2_BF16, AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    for (int r = row0; r < row0 + nrows; ++r)
        AB2_REQUIRE(kv->lens_host[r] + S <= kv->cap, AB2_ERR_CAPACITY, "KV cache length %d exceeds capacity %d",
                    kv->lens_host[r] + S, kv->cap);
    return AB2_OK;
}

AB2_API int ab2_kv_append(ab2_kv *kv, int layer, const void *k_dev, const void *v_dev, int S, int row0,
                          int nrows, ab2_dtype dtype, const float *cos_dev, const float *sin_dev,
                          const int *positions_dev, int max_seq, ab2_stream stream) {
    int rc = check_append(kv, layer, k_dev, v_dev, S, row0, nrows, dtype);
    if (rc != AB2_OK) return rc;
    AB2_REQUIRE((cos_dev == nullptr) == (sin_dev == nullptr), AB2_ERR_BAD_ARG, "cos and sin tables must be given together");
    if (cos_dev && !positions_dev)
        for (int r = row0; r < row0 + nrows; ++r)
            AB2_REQUIRE(kv->lens_host[r] + S <= max_seq, AB2_ERR_BAD_SHAPE, "RoPE positions exceed the table length %d", max_seq);
    return kv_append_device(kv, layer, k_dev, v_dev, (long long)kv->kvh * kv->hd, S, row0, nrows, dtype,
                            cos_dev, sin_dev, positions_dev, (cudaStream_t)stream);
}

AB2_API int ab2_kv_commit(ab2_kv *kv, int S, int row0, int nrows, ab2_stream stream) {
    AB2_REQUIRE(kv != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(S > 0 && nrows > 0 && row0 >= 0 && row0 + nrows <= kv->B, AB2_ERR_BAD_SHAPE,
                "rows %d..%d outside the cache batch %d", row0, row0 + nrows, kv->B);
    for (int r = row0; r < row0 + nrows; ++r)
        AB2_REQUIRE(kv->lens_host[r] + S <= kv->cap, AB2_ERR_CAPACITY, "KV cache length %d exceeds capacity %d",
                    kv->lens_host[r] + S, kv->cap);
    return kv_commit_device(kv, S, row0, nrows, (cudaStream_t)stream);
}

AB2_API int ab2_kv_update(ab2_kv *kv, const void *k_dev, const void *v_dev, int S, int row0, int nrows,
                          ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(kv != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(kv->L == 1, AB2_ERR_UNSUPPORTED, "update is the single-layer KVCache operation; this cache has %d layers", kv->L);
    int rc = check_append(kv, 0, k_dev, v_dev, S, row0, nrows, dtype);
    if (rc != AB2_OK) return rc;
    rc = kv_append_device(kv, 0, k_dev, v_dev, (long long)kv->kvh * kv->hd, S, row0, nrows, dtype, nullptr,
                          nullptr, nullptr, (cudaStream_t)stream);
    if (rc != AB2_OK) return rc;
    return kv_commit_device(kv, S, row0, nrows, (cudaStream_t)stream);
}

AB2_API int ab2_kv_truncate(ab2_kv *kv, int row, int new_len, ab2_stream stream) {
    AB2_REQUIRE(kv != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(row >= 0 && row < kv->B, AB2_ERR_BAD_SHAPE, "row %d outside the cache batch %d", row, kv->B);
    AB2_REQUIRE(new_len >= 0 && new_len <= kv->lens_host[row], AB2_ERR_CAPACITY,
                "cannot grow KV cache from %d to %d with truncate", kv->lens_host[row], new_len);
    kv->lens_host[row] = new_len;
    AB2_CUDA(cudaMemcpyAsync(kv->lens_dev + row, kv->lens_host + row, 4, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    AB2_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return AB2_OK;
}

AB2_API int ab2_kv_clear(ab2_kv *kv, ab2_stream stream) {
    AB2_REQUIRE(kv != nullptr, AB2_ERR_BAD_ARG, "null argument");
    memset(kv->lens_host, 0, (size_t)kv->B * 4);
    AB2_CUDA(cudaMemsetAsync(kv->lens_dev, 0, (size_t)kv->B * 4, (cudaStream_t)stream));
    return AB2_OK;
}

AB2_API int ab2_kv_seq_len(const ab2_kv *kv, int row, int *len) {
    AB2_REQUIRE(kv != nullptr && len != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(row >= 0 && row < kv->B, AB2_ERR_BAD_SHAPE, "row %d outside the cache batch %d", row, kv->B);
    *len = kv->lens_host[row];
    return AB2_OK;
}

AB2_API int ab2_kv_capacity(const ab2_kv *kv, int *capacity) {
    AB2_REQUIRE(kv != nullptr && capacity != nullptr, AB2_ERR_BAD_ARG, "null argument");
    *capacity = kv->cap;
    return AB2_OK;
}

AB2_API int ab2_kv_clone(ab2_kv **out, const ab2_kv *src, ab2_stream stream) {
    AB2_REQUIRE(out != nullptr && src != nullptr, AB2_ERR_BAD_ARG, "null argument");
    int rc = ab2_kv_create(out, src->L, src->B, src->cap, src->kvh, src->hd, src->h, (ab2_kv_dtype)src->dtype);
    if (rc != AB2_OK) return rc;
    ab2_kv *dst = *out;
    cudaStream_t s = (cudaStream_t)stream;
    size_t elems = (size_t)src->L * src->B * src->kvh * src->cap * src->hd, esz = kv_elem_size(src->dtype);
    cudaError_t e = cudaMemcpyAsync(dst->k, src->k, elems * esz, cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst->v, src->v, elems * esz, cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess && src->dtype == AB2_KV_INT8) {
        size_t ns = (size_t)src->L * src->B * src->kvh * src->cap * 4;
        e = cudaMemcpyAsync(dst->ks, src->ks, ns, cudaMemcpyDeviceToDevice, s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dst->vs, src->vs, ns, cudaMemcpyDeviceToDevice, s);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst->lens_dev, src->lens_dev, (size_t)src->B * 4, cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        ab2_kv_destroy(dst);
        *out = nullptr;
        return fail(AB2_ERR_CUDA, "KV cache clone failed: %s", cudaGetErrorString(e));
    }
    memcpy(dst->lens_host, src->lens_host, (size_t)src->B * 4);
    return AB2_OK;
}

AB2_API int ab2_kv_read(const ab2_kv *kv, int layer, int row, float *k_out_dev, float *v_out_dev,
                        ab2_stream stream) {
    AB2_REQUIRE(kv && k_out_dev && v_out_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(layer >= 0 && layer < kv->L, AB2_ERR_BAD_SHAPE, "layer %d outside the cache's %d layers", layer, kv->L);
    AB2_REQUIRE(row >= 0 && row < kv->B, AB2_ERR_BAD_SHAPE, "row %d outside the cache batch %d", row, kv->B);
    int len = kv->lens_host[row];
    if (len == 0) return AB2_OK;
    KvView view = kv_view(kv, layer);
    cudaStream_t s = (cudaStream_t)stream;
    unsigned blocks = (unsigned)std::min<size_t>(ceil_div((size_t)len * kv->kvh * kv->hd, 256), 2048);
    if (kv->dtype == AB2_KV_F32) kv_read_kernel<AB2_KV_F32><<<blocks, 256, 0, s>>>(view, row, len, k_out_dev, v_out_dev);
    else if (kv->dtype == AB2_KV_BF16) kv_read_kernel<AB2_KV_BF16><<<blocks, 256, 0, s>>>(view, row, len, k_out_dev, v_out_dev);
    else kv_read_kernel<AB2_KV_INT8><<<blocks, 256, 0, s>>>(view, row, len, k_out_dev, v_out_dev);
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}
