// Element-wise operators of the decoder block: RMSNorm, RoPE, SwiGLU, residual
// add, embedding gather and greedy argmax.  These are the unfused forms behind
// the C ABI; the decoder step uses the same device functions.
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "ops.cuh"
#include "w4a16_layout.cuh"

using namespace ab2;

namespace ab2 {

// ---- RMSNorm ---------------------------------------------------------------
// x * rsqrt(mean(x^2) + eps) * w, evaluated as the reference's scalar kernel:
// inv = 1 / sqrt(sum / d + eps); out = x * inv * w (two roundings, in that order).
template <typename T>
__global__ void rms_norm_kernel(const T *__restrict__ x, const float *__restrict__ w, T *out, int d,
                                float eps) {
    __shared__ float warp_sums[32];
    __shared__ float inv_shared;
    const T *row = x + (size_t)blockIdx.x * d;
    float sum = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = to_f32(row[i]);
        sum = fmaf(v, v, sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) inv_shared = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(v, (float)d), eps)));
    }
    __syncthreads();
    const float inv = inv_shared;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[(size_t)blockIdx.x * d + i] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(row[i]), inv), w[i]));
}

// bf16 rows with d % 8 == 0: every thread owns 8-element vectors, all loads of a
// row are in flight at once (decode rows are latency-bound, not bandwidth-bound).
// ADD: the row is first replaced by x + p (the residual add of the decoder, rounded to bf16 as the
// stand-alone add does) and the normalisation reads the new row: one launch for the pair.
template <bool ADD>
__global__ void rms_norm_bf16_vec_kernel(__nv_bfloat16 *x, const __nv_bfloat16 *p, const float *__restrict__ w,
                                         __nv_bfloat16 *out, int d, float eps) {
    __shared__ float warp_sums[32];
    __shared__ float inv_shared;
    pdl_wait();
    pdl_launch_dependents();
    uint4 *row = reinterpret_cast<uint4 *>(x + (size_t)blockIdx.x * d);
    const int nvec = d >> 3;
    uint4 v[2];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        v[it] = i < nvec ? row[i] : make_uint4(0, 0, 0, 0);
        if (ADD && i < nvec) {
            const uint4 q = reinterpret_cast<const uint4 *>(p + (size_t)blockIdx.x * d)[i];
            const uint32_t a4[4] = {v[it].x, v[it].y, v[it].z, v[it].w}, b4[4] = {q.x, q.y, q.z, q.w};
            uint32_t s4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = __fadd_rn(__uint_as_float(a4[j] << 16), __uint_as_float(b4[j] << 16));
                const float hi = __fadd_rn(__uint_as_float(a4[j] & 0xffff0000u), __uint_as_float(b4[j] & 0xffff0000u));
                s4[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
            }
            v[it] = make_uint4(s4[0], s4[1], s4[2], s4[3]);
            row[i] = v[it];
        }
        const uint32_t r[4] = {v[it].x, v[it].y, v[it].z, v[it].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = __uint_as_float(r[j] << 16), b = __uint_as_float(r[j] & 0xffff0000u);
            sum = fmaf(a, a, sum);
            sum = fmaf(b, b, sum);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) inv_shared = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)d), eps)));
    }
    __syncthreads();
    const float inv = inv_shared;
    uint4 *orow = reinterpret_cast<uint4 *>(out + (size_t)blockIdx.x * d);
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i >= nvec) continue;
        const float4 w0 = reinterpret_cast<const float4 *>(w)[2 * i], w1 = reinterpret_cast<const float4 *>(w)[2 * i + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const uint32_t r[4] = {v[it].x, v[it].y, v[it].z, v[it].w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = __uint_as_float(r[j] << 16), b = __uint_as_float(r[j] & 0xffff0000u);
            const __nv_bfloat16 oa = __float2bfloat16_rn(__fmul_rn(__fmul_rn(a, inv), ww[2 * j]));
            const __nv_bfloat16 ob = __float2bfloat16_rn(__fmul_rn(__fmul_rn(b, inv), ww[2 * j + 1]));
            o[j] = (uint32_t)__bfloat16_as_ushort(oa) | ((uint32_t)__bfloat16_as_ushort(ob) << 16);
        }
        orow[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

int launch_rms_norm(const void *x, const float *w, void *out, int rows, int d, float eps,
                    ab2_dtype dtype, cudaStream_t s) {
    if (dtype == AB2_BF16 && d % 8 == 0 && d / 8 <= 2048 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w) & 15) == 0) {
        int threads = std::min(1024, ((d / 8 + 1) / 2 + 31) / 32 * 32);
        cudaError_t e = launch_kernel(rms_norm_bf16_vec_kernel<false>, dim3(rows), dim3(threads), 0, s,
                                      (__nv_bfloat16 *)const_cast<void *>(x), (const __nv_bfloat16 *)nullptr, w,
                                      (__nv_bfloat16 *)out, d, eps);
        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "RMSNorm launch failed: %s", cudaGetErrorString(e));
        return AB2_OK;
    }
    int threads = d >= 1024 ? 256 : 128;
    switch (dtype) {
    case AB2_F32: rms_norm_kernel<float><<<rows, threads, 0, s>>>((const float *)x, w, (float *)out, d, eps); break;
    case AB2_F16: rms_norm_kernel<__half><<<rows, threads, 0, s>>>((const __half *)x, w, (__half *)out, d, eps); break;
    default: rms_norm_kernel<__nv_bfloat16><<<rows, threads, 0, s>>>((const __nv_bfloat16 *)x, w, (__nv_bfloat16 *)out, d, eps); break;
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

// x += p (row-wise, rounded to the activation type), then out = RMSNorm(x; w): one launch where the
// vector kernel applies, else the two launches it replaces.
int launch_add_rms_norm(void *x, const void *p, const float *w, void *out, int rows, int d, float eps,
                        ab2_dtype dtype, cudaStream_t s) {
    if (dtype == AB2_BF16 && d % 8 == 0 && d / 8 <= 2048 &&
        (((uintptr_t)x | (uintptr_t)p | (uintptr_t)out | (uintptr_t)w) & 15) == 0) {
        int threads = std::min(1024, ((d / 8 + 1) / 2 + 31) / 32 * 32);
        cudaError_t e = launch_kernel(rms_norm_bf16_vec_kernel<true>, dim3(rows), dim3(threads), 0, s, (__nv_bfloat16 *)x,
                                      (const __nv_bfloat16 *)p, w, (__nv_bfloat16 *)out, d, eps);
        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "add + RMSNorm launch failed: %s", cudaGetErrorString(e));
        return AB2_OK;
    }
    int rc = launch_add(x, p, x, (size_t)rows * d, dtype, s);
    if (rc != AB2_OK) return rc;
    return launch_rms_norm(x, w, out, rows, d, eps, dtype, s);
}

// ---- RoPE ------------------------------------------------------------------
// x [rows, heads, hd]; row i uses table row positions[i] (or offset + i % seq).
template <typename T>
__global__ void rope_kernel(const T *__restrict__ x, T *out, const float *__restrict__ cos_t,
                            const float *__restrict__ sin_t, const int *__restrict__ positions,
                            int offset, int seq, int heads, int hd, size_t total_pairs) {
    const int half = hd >> 1;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_pairs) return;
    int i = (int)(idx % half);
    size_t rh = idx / half;  // row * heads + head
    size_t row = rh / heads;
    int pos = positions ? positions[row] : offset + (int)(row % seq);
    size_t base = rh * hd;
    float x1 = to_f32(x[base + i]), x2 = to_f32(x[base + half + i]);
    float o1, o2;
    rope_rotate(x1, x2, cos_t[(size_t)pos * half + i], sin_t[(size_t)pos * half + i], o1, o2);
    out[base + i] = from_f32<T>(o1);
    out[base + half + i] = from_f32<T>(o2);
}

// ---- SwiGLU ----------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T *__restrict__ gate, const T *__restrict__ up, T *out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(swiglu_value(to_f32(gate[i]), to_f32(up[i])));
}

// gate and up interleaved per token as [tokens][2*ffn] (gate first): the layout
// the fused gate|up projection produces.
template <typename T>
__global__ void swiglu_fused_kernel(const T *__restrict__ gu, T *out, int ffn, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t tok = i / ffn, j = i % ffn;
    const T *row = gu + tok * 2 * (size_t)ffn;
    out[i] = from_f32<T>(swiglu_value(to_f32(row[j]), to_f32(row[ffn + j])));
}

template <typename T>
__global__ void add_kernel(const T *__restrict__ a, const T *__restrict__ b, T *out, size_t n) {
    pdl_wait();  // inputs come from the preceding kernel of the step
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(__fadd_rn(to_f32(a[i]), to_f32(b[i])));
}
// The same sums, 16 bytes per thread (n a multiple of the vector width, pointers 16-byte aligned).
template <typename T>
__global__ void add_vec_kernel(const T *a, const T *b, T *out, size_t nvec) {
    constexpr int V = 16 / sizeof(T);
    pdl_wait();  // inputs come from the preceding kernel of the step
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    union { uint4 q; T e[V]; } va, vb, vo;
    va.q = reinterpret_cast<const uint4 *>(a)[i];
    vb.q = reinterpret_cast<const uint4 *>(b)[i];
#pragma unroll
    for (int k = 0; k < V; ++k) vo.e[k] = from_f32<T>(__fadd_rn(to_f32(va.e[k]), to_f32(vb.e[k])));
    reinterpret_cast<uint4 *>(out)[i] = vo.q;
}

int launch_swiglu_fused(const void *gu, void *out, int tokens, int ffn, ab2_dtype dtype, cudaStream_t s) {
    size_t n = (size_t)tokens * ffn;
    unsigned blocks = (unsigned)ceil_div(n, 256);
    switch (dtype) {
    case AB2_F32: swiglu_fused_kernel<float><<<blocks, 256, 0, s>>>((const float *)gu, (float *)out, ffn, n); break;
    case AB2_F16: swiglu_fused_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)gu, (__half *)out, ffn, n); break;
    default: swiglu_fused_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)gu, (__nv_bfloat16 *)out, ffn, n); break;
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

int launch_add(const void *a, const void *b, void *out, size_t n, ab2_dtype dtype, cudaStream_t s) {
    cudaError_t e;
    const size_t esz = dtype == AB2_F32 ? 4 : 2;
    const bool vec = n % (16 / esz) == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
    if (vec) {
        const size_t nvec = n / (16 / esz);
        unsigned blocks = (unsigned)ceil_div(nvec, 256);
        switch (dtype) {
        case AB2_F32: e = launch_kernel(add_vec_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float *)a, (const float *)b, (float *)out, nvec); break;
        case AB2_F16: e = launch_kernel(add_vec_kernel<__half>, dim3(blocks), dim3(256), 0, s, (const __half *)a, (const __half *)b, (__half *)out, nvec); break;
        default: e = launch_kernel(add_vec_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (__nv_bfloat16 *)out, nvec); break;
        }
    } else {
        unsigned blocks = (unsigned)ceil_div(n, 256);
        switch (dtype) {
        case AB2_F32: e = launch_kernel(add_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float *)a, (const float *)b, (float *)out, n); break;
        case AB2_F16: e = launch_kernel(add_kernel<__half>, dim3(blocks), dim3(256), 0, s, (const __half *)a, (const __half *)b, (__half *)out, n); break;
        default: e = launch_kernel(add_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (__nv_bfloat16 *)out, n); break;
        }
    }
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "add launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

// ---- argmax ----------------------------------------------------------------
// Last index among equal maxima under the f32 total order (-NaN < -inf < ... <
// -0 < +0 < ... < +inf < +NaN): the key is monotone in that order, and ties on
// the key go to the larger index.
__device__ __forceinline__ long long argmax_key(float v, int idx) {
    int b = __float_as_int(v);
    b ^= (int)(((unsigned)(b >> 31)) >> 1);
    return ((long long)b << 32) | (unsigned)idx;
}

template <typename T>
__global__ void argmax_kernel(const T *__restrict__ logits, int vocab, uint32_t *out) {
    __shared__ long long warp_best[32];
    const T *row = logits + (size_t)blockIdx.x * vocab;
    long long best = LLONG_MIN;
    if (sizeof(T) == 2 && ((uintptr_t)row & 15) == 0) {
        // 16-bit logits: eight per load, every load of a thread in flight at once
        const int nvec = vocab >> 3;
        const uint4 *row4 = reinterpret_cast<const uint4 *>(row);
        for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * blockDim.x;
                v[u] = i < nvec ? row4[i] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i >= nvec) continue;
                const T *e = reinterpret_cast<const T *>(&v[u]);
#pragma unroll
                for (int j = 0; j < 8; ++j) best = max(best, argmax_key(to_f32(e[j]), i * 8 + j));
            }
        }
        for (int i = (nvec << 3) + threadIdx.x; i < vocab; i += blockDim.x) best = max(best, argmax_key(to_f32(row[i]), i));
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = max(best, argmax_key(to_f32(row[i]), i));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        long long v = threadIdx.x < (blockDim.x >> 5) ? warp_best[threadIdx.x] : LLONG_MIN;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
        if (threadIdx.x == 0) out[blockIdx.x] = (uint32_t)(v & 0xffffffffll);
    }
}

int launch_argmax(const void *logits, int rows, int vocab, ab2_dtype dtype, uint32_t *out, cudaStream_t s) {
    switch (dtype) {
    case AB2_F32: argmax_kernel<float><<<rows, 1024, 0, s>>>((const float *)logits, vocab, out); break;
    case AB2_F16: argmax_kernel<__half><<<rows, 1024, 0, s>>>((const __half *)logits, vocab, out); break;
    default: argmax_kernel<__nv_bfloat16><<<rows, 1024, 0, s>>>((const __nv_bfloat16 *)logits, vocab, out); break;
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

// ---- embedding gather --------------------------------------------------------
// TokenEmbedding::forward over a packed table: out[t, :] = dequant(table[ids[t], :]).
template <typename T>
__global__ void embedding_kernel(const uint32_t *__restrict__ ids, int vocab, int fmt, const void *codes,
                                 const float *scales, const float *zeros, const uint32_t *block_params,
                                 int N, int K, int group, T *out) {
    uint32_t id = ids[blockIdx.x];
    if (id >= (uint32_t)vocab) id = vocab - 1;  // ids are validated on the host; keep reads in range
    // grid (tokens, slices of the row): one element per thread, so a row costs one
    // round trip to memory instead of a chain of them
    for (int k = blockIdx.y * blockDim.x + threadIdx.x; k < K; k += gridDim.y * blockDim.x) {
        size_t idx = (size_t)id * K + k;
        float v;
        if (fmt == FMT_I8) {
            v = __fmul_rn((float)((const int8_t *)codes)[idx], scales[id]);
        } else if (fmt == FMT_I4_AFFINE) {
            uint8_t byte = ((const uint8_t *)codes)[idx >> 1];
            float q = (float)((idx & 1) ? (byte >> 4) : (byte & 0x0f));
            size_t g = idx / (size_t)group;
            v = __fmul_rn(__fsub_rn(q, zeros[g]), scales[g]);
        } else if (fmt == FMT_Q4KM) {
            uint8_t byte = ((const uint8_t *)codes)[idx >> 1];
            float q = (float)((idx & 1) ? (byte >> 4) : (byte & 0x0f));
            uint32_t p = block_params[idx >> 8];
            v = __fadd_rn(__fmul_rn(q, f16_bits_to_f32((uint16_t)(p & 0xffffu))), f16_bits_to_f32((uint16_t)(p >> 16)));
        } else {
            W4Layout L{N, K, group};
            const uint32_t *t = (const uint32_t *)codes;
            uint32_t word = t[L.code_index((int)id, k >> 3)];
            int e = k & 7, slot = (e >> 1) + 4 * (e & 1);
            uint32_t p = t[L.param_index((int)id, k / group)];
            v = __fmul_rn(__fsub_rn((float)((word >> (4 * slot)) & 0xFu), (float)((p >> 16) & 0xFu)),
                          bf16_bits_to_f32((uint16_t)(p & 0xffffu)));
        }
        out[(size_t)blockIdx.x * K + k] = from_f32<T>(v);
    }
}

int launch_embedding(const ab2_qweight *table, const uint32_t *ids, int tokens, void *out, ab2_dtype dtype,
                     cudaStream_t s) {
    const dim3 grid(tokens, tokens <= 64 ? std::min(32, std::max(1, (table->K + 127) / 128)) : 1);
#define AB2_EMB(T) embedding_kernel<T><<<grid, 128, 0, s>>>(ids, table->N, table->fmt, table->codes, table->scales, table->zeros, table->block_params, table->N, table->K, table->group, (T *)out)
    switch (dtype) {
    case AB2_F32: AB2_EMB(float); break;
    case AB2_F16: AB2_EMB(__half); break;
    default: AB2_EMB(__nv_bfloat16); break;
    }
#undef AB2_EMB
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

}  // namespace ab2

static bool dtype_ok(ab2_dtype d) { return d == AB2_F32 || d == AB2_F16 || d == AB2_BF16; }

AB2_API int ab2_rms_norm(const void *x_dev, const float *weight_dev, void *out_dev, int rows, int d,
                         float eps, ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(x_dev && weight_dev && out_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(rows > 0 && d > 0, AB2_ERR_BAD_SHAPE, "rms_norm hidden dimension must be non-zero");
    AB2_REQUIRE(dtype_ok(dtype), AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    return launch_rms_norm(x_dev, weight_dev, out_dev, rows, d, eps, dtype, (cudaStream_t)stream);
}

AB2_API int ab2_rope_apply(const void *x_dev, void *out_dev, const float *cos_dev, const float *sin_dev,
                           int batch, int seq, int heads, int head_dim, int offset, int max_seq,
                           ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(x_dev && out_dev && cos_dev && sin_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(batch > 0 && seq > 0 && heads > 0 && head_dim > 0 && head_dim % 2 == 0, AB2_ERR_BAD_SHAPE,
                "RoPE needs positive dimensions and an even head_dim, got head_dim=%d", head_dim);
    AB2_REQUIRE(offset >= 0 && offset + seq <= max_seq, AB2_ERR_BAD_SHAPE,
                "RoPE positions %d..%d exceed the table length %d", offset, offset + seq, max_seq);
    AB2_REQUIRE(dtype_ok(dtype), AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    size_t pairs = (size_t)batch * seq * heads * (head_dim / 2);
    unsigned blocks = (unsigned)ceil_div(pairs, 256);
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case AB2_F32: rope_kernel<float><<<blocks, 256, 0, s>>>((const float *)x_dev, (float *)out_dev, cos_dev, sin_dev, nullptr, offset, seq, heads, head_dim, pairs); break;
    case AB2_F16: rope_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)x_dev, (__half *)out_dev, cos_dev, sin_dev, nullptr, offset, seq, heads, head_dim, pairs); break;
    default: rope_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)x_dev, (__nv_bfloat16 *)out_dev, cos_dev, sin_dev, nullptr, offset, seq, heads, head_dim, pairs); break;
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

AB2_API int ab2_swiglu(const void *gate_dev, const void *up_dev, void *out_dev, size_t n, ab2_dtype dtype,
                       ab2_stream stream) {
    AB2_REQUIRE(gate_dev && up_dev && out_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(dtype_ok(dtype), AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    if (n == 0) return AB2_OK;
    unsigned blocks = (unsigned)ceil_div(n, 256);
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case AB2_F32: swiglu_kernel<float><<<blocks, 256, 0, s>>>((const float *)gate_dev, (const float *)up_dev, (float *)out_dev, n); break;
    case AB2_F16: swiglu_kernel<__half><<<blocks, 256, 0, s>>>((const __half *)gate_dev, (const __half *)up_dev, (__half *)out_dev, n); break;
    default: swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16 *)gate_dev, (const __nv_bfloat16 *)up_dev, (__nv_bfloat16 *)out_dev, n); break;
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

AB2_API int ab2_argmax(const void *logits_dev, int rows, int vocab, ab2_dtype dtype, uint32_t *out_dev,
                       ab2_stream stream) {
    AB2_REQUIRE(logits_dev && out_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(rows > 0 && vocab > 0, AB2_ERR_BAD_SHAPE, "argmax needs a non-empty logits matrix");
    AB2_REQUIRE(dtype_ok(dtype), AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    return launch_argmax(logits_dev, rows, vocab, dtype, out_dev, (cudaStream_t)stream);
}

AB2_API int ab2_embedding_forward(const ab2_qweight *table, const uint32_t *ids_dev, int tokens,
                                  void *out_dev, ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(table && ids_dev && out_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tokens > 0, AB2_ERR_BAD_SHAPE, "token count must be positive");
    AB2_REQUIRE(dtype_ok(dtype), AB2_ERR_BAD_DTYPE, "unsupported dtype %d", (int)dtype);
    return launch_embedding(table, ids_dev, tokens, out_dev, dtype, (cudaStream_t)stream);
}
