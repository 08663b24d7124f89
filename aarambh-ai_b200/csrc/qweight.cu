// Packed-weight handles: constructors from the reference layouts, device-side
// quantisers, export and the bit-exact dequantisation entry point.
#include <cfloat>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "w4a16_layout.cuh"

namespace ab2 {

static thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

}  // namespace ab2

AB2_API int ab2_version(void) { return 100; }
AB2_API const char *ab2_last_error(void) { return ab2::g_last_error.c_str(); }

using namespace ab2;

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------
static int alloc_handle(ab2_qweight **out, int fmt, int N, int K, int group) {
    AB2_REQUIRE(out != nullptr, AB2_ERR_BAD_ARG, "output handle pointer is null");
    AB2_REQUIRE(N > 0 && K > 0, AB2_ERR_BAD_SHAPE, "weight shape must be positive, got [%d,%d]", N, K);
    ab2_qweight *w = new ab2_qweight();
    memset(w, 0, sizeof(*w));
    w->fmt = fmt; w->N = N; w->K = K; w->group = group;
    cudaGetDevice(&w->device);
    *out = w;
    return AB2_OK;
}

static int dev_alloc(void **p, size_t bytes) {
    AB2_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    return AB2_OK;
}

#define TRY(expr)                         \
    do {                                  \
        int _rc = (expr);                 \
        if (_rc != AB2_OK) return _rc;    \
    } while (0)

#define TRY_OR_FREE(w, expr)              \
    do {                                  \
        int _rc = (expr);                 \
        if (_rc != AB2_OK) {              \
            ab2_qweight_destroy(w);       \
            return _rc;                   \
        }                                 \
    } while (0)

AB2_API int ab2_qweight_destroy(ab2_qweight *w) {
    if (!w) return AB2_OK;
    cudaFree(w->codes); cudaFree(w->scales); cudaFree(w->zeros);
    cudaFree(w->block_params);
    delete w;
    return AB2_OK;
}

AB2_API int ab2_qweight_shape(const ab2_qweight *w, int *N, int *K, int *group, int *format) {
    AB2_REQUIRE(w != nullptr, AB2_ERR_BAD_ARG, "weight handle is null");
    if (N) *N = w->N;
    if (K) *K = w->K;
    if (group) *group = w->group;
    if (format) *format = w->fmt;
    return AB2_OK;
}

AB2_API int ab2_qweight_nbytes(const ab2_qweight *w, size_t *nbytes) {
    AB2_REQUIRE(w != nullptr && nbytes != nullptr, AB2_ERR_BAD_ARG, "null argument");
    *nbytes = w->codes_bytes + w->param_bytes;
    return AB2_OK;
}

// ---------------------------------------------------------------------------
// constructors from reference layouts
// ---------------------------------------------------------------------------
__global__ void fill_f32_kernel(float *p, float v, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

static int make_i8(ab2_qweight **out, int N, int K, bool per_tensor) {
    TRY(alloc_handle(out, FMT_I8, N, K, K));
    ab2_qweight *w = *out;
    w->per_tensor = per_tensor;
    w->codes_bytes = (size_t)N * K;
    w->param_bytes = per_tensor ? 4 : (size_t)N * 4;
    TRY_OR_FREE(w, dev_alloc(&w->codes, (w->codes_bytes + 15) / 16 * 16));
    TRY_OR_FREE(w, dev_alloc((void **)&w->scales, (size_t)N * 4));
    return AB2_OK;
}

static int upload_i8(ab2_qweight **out, const int8_t *codes, const float *scales_N, float scale,
                     int N, int K) {
    TRY(make_i8(out, N, K, scales_N == nullptr));
    ab2_qweight *w = *out;
    cudaError_t e = cudaMemcpy(w->codes, codes, w->codes_bytes, cudaMemcpyDefault);
    if (e == cudaSuccess && scales_N) e = cudaMemcpy(w->scales, scales_N, (size_t)N * 4, cudaMemcpyDefault);
    if (e == cudaSuccess && !scales_N) fill_f32_kernel<<<(N + 255) / 256, 256>>>(w->scales, scale, N);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        ab2_qweight_destroy(w);
        *out = nullptr;
        return fail(AB2_ERR_CUDA, "int8 weight upload failed: %s", cudaGetErrorString(e));
    }
    return AB2_OK;
}

AB2_API int ab2_qweight_from_i8_tensor(ab2_qweight **out, const int8_t *codes, float scale, int N,
                                       int K) {
    AB2_REQUIRE(codes != nullptr, AB2_ERR_BAD_ARG, "codes pointer is null");
    return upload_i8(out, codes, nullptr, scale, N, K);
}

AB2_API int ab2_qweight_from_i8_channel(ab2_qweight **out, const int8_t *codes,
                                        const float *scales_N, int N, int K) {
    AB2_REQUIRE(codes != nullptr && scales_N != nullptr, AB2_ERR_BAD_ARG, "null input pointer");
    return upload_i8(out, codes, scales_N, 0.f, N, K);
}

static int make_i4_affine(ab2_qweight **out, int N, int K, int group) {
    AB2_REQUIRE(group > 0, AB2_ERR_BAD_SHAPE, "group_size must be non-zero");
    TRY(alloc_handle(out, FMT_I4_AFFINE, N, K, group));
    ab2_qweight *w = *out;
    size_t n = (size_t)N * K, ng = ceil_div(n, (size_t)group);
    w->codes_bytes = ceil_div(n, 2);
    w->param_bytes = ng * 8;
    // codes are padded to a multiple of 16 bytes so vector loads may over-read.
    TRY_OR_FREE(w, dev_alloc(&w->codes, (w->codes_bytes + 15) / 16 * 16));
    TRY_OR_FREE(w, dev_alloc((void **)&w->scales, ng * 4));
    TRY_OR_FREE(w, dev_alloc((void **)&w->zeros, ng * 4));
    return AB2_OK;
}

AB2_API int ab2_qweight_from_i4_affine(ab2_qweight **out, const uint8_t *packed,
                                       const float *scales, const float *zeros, int N, int K,
                                       int group) {
    AB2_REQUIRE(packed && scales && zeros, AB2_ERR_BAD_ARG, "null input pointer");
    TRY(make_i4_affine(out, N, K, group));
    ab2_qweight *w = *out;
    size_t ng = ceil_div((size_t)N * K, (size_t)group);
    cudaError_t e = cudaMemcpy(w->codes, packed, w->codes_bytes, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMemcpy(w->scales, scales, ng * 4, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMemcpy(w->zeros, zeros, ng * 4, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { ab2_qweight_destroy(w); *out = nullptr; return fail(AB2_ERR_CUDA, "int4 weight upload failed: %s", cudaGetErrorString(e)); }
    return AB2_OK;
}

static int make_q4km(ab2_qweight **out, int N, int K) {
    TRY(alloc_handle(out, FMT_Q4KM, N, K, 256));
    ab2_qweight *w = *out;
    size_t nb = ceil_div((size_t)N * K, 256);
    w->codes_bytes = nb * 128;
    w->param_bytes = nb * 4;
    TRY_OR_FREE(w, dev_alloc(&w->codes, w->codes_bytes));
    TRY_OR_FREE(w, dev_alloc((void **)&w->block_params, nb * 4));
    return AB2_OK;
}

// Splits 132-byte blocks into a code plane (128 B per block) and a parameter
// plane (one u32 per block: f16 scale in the low half, f16 min in the high half).
__global__ void q4km_split_kernel(const uint8_t *blocks, uint8_t *codes, uint32_t *params,
                                  size_t nblocks) {
    size_t b = blockIdx.x;
    if (b >= nblocks) return;
    const uint8_t *src = blocks + b * 132;
    int t = threadIdx.x;  // 128 threads
    codes[b * 128 + t] = src[4 + t];
    if (t == 0)
        params[b] = (uint32_t)src[0] | ((uint32_t)src[1] << 8) | ((uint32_t)src[2] << 16) |
                    ((uint32_t)src[3] << 24);
}

__global__ void q4km_join_kernel(const uint8_t *codes, const uint32_t *params, uint8_t *blocks,
                                 size_t nblocks) {
    size_t b = blockIdx.x;
    if (b >= nblocks) return;
    uint8_t *dst = blocks + b * 132;
    int t = threadIdx.x;
    dst[4 + t] = codes[b * 128 + t];
    if (t < 4) dst[t] = (uint8_t)(params[b] >> (8 * t));
}

AB2_API int ab2_qweight_from_q4km_blocks(ab2_qweight **out, const uint8_t *blocks132, int N, int K) {
    AB2_REQUIRE(blocks132 != nullptr, AB2_ERR_BAD_ARG, "null input pointer");
    TRY(make_q4km(out, N, K));
    ab2_qweight *w = *out;
    size_t nb = ceil_div((size_t)N * K, 256);
    uint8_t *staging = nullptr;
    cudaError_t e = cudaMalloc((void **)&staging, nb * 132);
    if (e == cudaSuccess) e = cudaMemcpy(staging, blocks132, nb * 132, cudaMemcpyDefault);
    if (e == cudaSuccess) {
        q4km_split_kernel<<<(unsigned)nb, 128>>>(staging, (uint8_t *)w->codes, w->block_params, nb);
        e = cudaDeviceSynchronize();
    }
    cudaFree(staging);
    if (e != cudaSuccess) { ab2_qweight_destroy(w); *out = nullptr; return fail(AB2_ERR_CUDA, "Q4 block upload failed: %s", cudaGetErrorString(e)); }
    return AB2_OK;
}

static int make_w4a16(ab2_qweight **out, int N, int K, int group) {
    AB2_REQUIRE(group > 0 && group % 8 == 0, AB2_ERR_BAD_SHAPE, "group size must be a positive multiple of 8, got %d", group);
    AB2_REQUIRE(K % group == 0, AB2_ERR_BAD_SHAPE, "K=%d is not a multiple of the group size %d", K, group);
    TRY(alloc_handle(out, FMT_W4A16, N, K, group));
    ab2_qweight *w = *out;
    W4Layout L{N, K, group};
    w->codes_bytes = (size_t)L.tiles() * 16 * K / 2;
    w->param_bytes = (size_t)L.tiles() * 16 * L.G() * 4;
    TRY_OR_FREE(w, dev_alloc(&w->codes, L.total_words() * 4));
    cudaError_t e = cudaMemset(w->codes, 0, L.total_words() * 4);
    if (e != cudaSuccess) { ab2_qweight_destroy(w); *out = nullptr; return fail(AB2_ERR_CUDA, "cudaMemset failed: %s", cudaGetErrorString(e)); }
    return AB2_OK;
}

// Input layout [N][K/8] code words (natural or interleaved nibble order),
// scales [N][G] bf16, zero points [N][ceil(G/8)] -> tile-major blocks.
__device__ __forceinline__ uint32_t w4_to_interleaved(uint32_t v) {
    const int slot_of[8] = {0, 4, 1, 5, 2, 6, 3, 7};
    uint32_t o = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) o |= ((v >> (4 * e)) & 0xFu) << (4 * slot_of[e]);
    return o;
}
__device__ __forceinline__ uint32_t w4_to_natural(uint32_t v) {
    const int slot_of[8] = {0, 4, 1, 5, 2, 6, 3, 7};
    uint32_t o = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) o |= ((v >> (4 * slot_of[e])) & 0xFu) << (4 * e);
    return o;
}

__global__ void w4a16_tile_codes_kernel(const uint32_t *qweight, W4Layout L, bool awq,
                                        uint32_t *tiles) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t wpr = (size_t)L.K >> 3;
    if (i >= (size_t)L.N * wpr) return;
    int n = (int)(i / wpr), word = (int)(i % wpr);
    uint32_t v = qweight[i];
    tiles[L.code_index(n, word)] = awq ? v : w4_to_interleaved(v);
}

__global__ void w4a16_tile_params_kernel(const uint16_t *scales16, const uint32_t *qzeros,
                                         W4Layout L, bool awq, uint32_t *tiles) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int G = L.G();
    if (i >= (size_t)L.N * G) return;
    int n = (int)(i / G), g = (int)(i % G);
    int e = g & 7, slot = awq ? (e >> 1) + 4 * (e & 1) : e;
    uint32_t z = (qzeros[(size_t)n * ((G + 7) >> 3) + (g >> 3)] >> (4 * slot)) & 0xFu;
    tiles[L.param_index(n, g)] = (uint32_t)scales16[i] | ((0xC300u | z) << 16);
}

// tile-major blocks -> natural-order [N][K/8] words, scales, zero points
__global__ void w4a16_untile_codes_kernel(const uint32_t *tiles, W4Layout L, uint32_t *qweight) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t wpr = (size_t)L.K >> 3;
    if (i >= (size_t)L.N * wpr) return;
    qweight[i] = w4_to_natural(tiles[L.code_index((int)(i / wpr), (int)(i % wpr))]);
}

__global__ void w4a16_untile_params_kernel(const uint32_t *tiles, W4Layout L, uint16_t *scales16,
                                           uint32_t *qzeros) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int G = L.G();
    if (i >= (size_t)L.N * G) return;
    int n = (int)(i / G), g = (int)(i % G);
    uint32_t p = tiles[L.param_index(n, g)];
    scales16[i] = (uint16_t)(p & 0xffffu);
    atomicOr(&qzeros[(size_t)n * ((G + 7) >> 3) + (g >> 3)], ((p >> 16) & 0xFu) << (4 * (g & 7)));
}

static int from_w4a16(ab2_qweight **out, const uint32_t *qweight, const uint16_t *scales_bf16,
                      const uint32_t *qzeros, int N, int K, int group, bool awq) {
    AB2_REQUIRE(qweight && scales_bf16 && qzeros, AB2_ERR_BAD_ARG, "null input pointer");
    TRY(make_w4a16(out, N, K, group));
    ab2_qweight *w = *out;
    W4Layout L{N, K, group};
    size_t G = (size_t)L.G(), ZW = ceil_div(G, 8), nw = (size_t)N * K / 8;
    uint32_t *c_dev = nullptr, *z_dev = nullptr;
    uint16_t *s_dev = nullptr;
    cudaError_t e = cudaMalloc((void **)&c_dev, nw * 4);
    if (e == cudaSuccess) e = cudaMalloc((void **)&s_dev, (size_t)N * G * 2);
    if (e == cudaSuccess) e = cudaMalloc((void **)&z_dev, (size_t)N * ZW * 4);
    if (e == cudaSuccess) e = cudaMemcpy(c_dev, qweight, nw * 4, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMemcpy(s_dev, scales_bf16, (size_t)N * G * 2, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMemcpy(z_dev, qzeros, (size_t)N * ZW * 4, cudaMemcpyDefault);
    if (e == cudaSuccess) {
        w4a16_tile_codes_kernel<<<(unsigned)ceil_div(nw, 256), 256>>>(c_dev, L, awq, (uint32_t *)w->codes);
        w4a16_tile_params_kernel<<<(unsigned)ceil_div((size_t)N * G, 256), 256>>>(s_dev, z_dev, L, awq, (uint32_t *)w->codes);
        e = cudaDeviceSynchronize();
    }
    cudaFree(c_dev); cudaFree(s_dev); cudaFree(z_dev);
    if (e != cudaSuccess) { ab2_qweight_destroy(w); *out = nullptr; return fail(AB2_ERR_CUDA, "W4A16 weight upload failed: %s", cudaGetErrorString(e)); }
    return AB2_OK;
}

AB2_API int ab2_qweight_from_w4a16_gptq(ab2_qweight **out, const uint32_t *qweight,
                                        const uint16_t *scales_bf16, const uint32_t *qzeros, int N,
                                        int K, int group) {
    return from_w4a16(out, qweight, scales_bf16, qzeros, N, K, group, false);
}

AB2_API int ab2_qweight_from_w4a16_awq(ab2_qweight **out, const uint32_t *qweight,
                                       const uint16_t *scales_bf16, const uint32_t *qzeros, int N,
                                       int K, int group) {
    return from_w4a16(out, qweight, scales_bf16, qzeros, N, K, group, true);
}

AB2_API int ab2_qweight_export(const ab2_qweight *w, void *codes, void *scales, void *zeros) {
    AB2_REQUIRE(w != nullptr, AB2_ERR_BAD_ARG, "weight handle is null");
    size_t n = (size_t)w->N * w->K;
    switch (w->fmt) {
    case FMT_I8:
        if (codes) AB2_CUDA(cudaMemcpy(codes, w->codes, n, cudaMemcpyDefault));
        if (scales) AB2_CUDA(cudaMemcpy(scales, w->scales, w->per_tensor ? 4 : (size_t)w->N * 4, cudaMemcpyDefault));
        break;
    case FMT_I4_AFFINE: {
        size_t ng = ceil_div(n, (size_t)w->group);
        if (codes) AB2_CUDA(cudaMemcpy(codes, w->codes, w->codes_bytes, cudaMemcpyDefault));
        if (scales) AB2_CUDA(cudaMemcpy(scales, w->scales, ng * 4, cudaMemcpyDefault));
        if (zeros) AB2_CUDA(cudaMemcpy(zeros, w->zeros, ng * 4, cudaMemcpyDefault));
        break;
    }
    case FMT_Q4KM: {
        if (codes) {
            size_t nb = ceil_div(n, 256);
            uint8_t *staging = nullptr;
            AB2_CUDA(cudaMalloc((void **)&staging, nb * 132));
            q4km_join_kernel<<<(unsigned)nb, 128>>>((const uint8_t *)w->codes, w->block_params, staging, nb);
            cudaError_t e = cudaMemcpy(codes, staging, nb * 132, cudaMemcpyDefault);
            cudaFree(staging);
            if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "Q4 block export failed: %s", cudaGetErrorString(e));
        }
        break;
    }
    case FMT_W4A16: {  // exported in the natural (GPTQ) nibble order
        W4Layout L{w->N, w->K, w->group};
        size_t G = (size_t)L.G(), ZW = ceil_div(G, 8), nw = (size_t)w->N * w->K / 8, NG = (size_t)w->N * G;
        uint32_t *c_dev = nullptr, *z_dev = nullptr;
        uint16_t *s_dev = nullptr;
        cudaError_t e = cudaMalloc((void **)&c_dev, nw * 4);
        if (e == cudaSuccess) e = cudaMalloc((void **)&s_dev, NG * 2);
        if (e == cudaSuccess) e = cudaMalloc((void **)&z_dev, (size_t)w->N * ZW * 4);
        if (e == cudaSuccess) e = cudaMemset(z_dev, 0, (size_t)w->N * ZW * 4);
        if (e == cudaSuccess) {
            w4a16_untile_codes_kernel<<<(unsigned)ceil_div(nw, 256), 256>>>((const uint32_t *)w->codes, L, c_dev);
            w4a16_untile_params_kernel<<<(unsigned)ceil_div(NG, 256), 256>>>((const uint32_t *)w->codes, L, s_dev, z_dev);
            if (codes) e = cudaMemcpy(codes, c_dev, nw * 4, cudaMemcpyDefault);
            if (e == cudaSuccess && scales) e = cudaMemcpy(scales, s_dev, NG * 2, cudaMemcpyDefault);
            if (e == cudaSuccess && zeros) e = cudaMemcpy(zeros, z_dev, (size_t)w->N * ZW * 4, cudaMemcpyDefault);
        }
        cudaFree(c_dev); cudaFree(s_dev); cudaFree(z_dev);
        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "W4A16 export failed: %s", cudaGetErrorString(e));
        break;
    }
    default:
        return fail(AB2_ERR_BAD_ARG, "unknown weight format %d", w->fmt);
    }
    return AB2_OK;
}

// ---------------------------------------------------------------------------
// dequantisation (bit-exact with the reference arithmetic for f32 output)
// ---------------------------------------------------------------------------
struct QView {
    int fmt, N, K, group;
    const void *codes;
    const float *scales, *zeros;
    const uint32_t *block_params;
};

static QView view_of(const ab2_qweight *w) {
    QView v;
    v.fmt = w->fmt; v.N = w->N; v.K = w->K; v.group = w->group;
    v.codes = w->codes; v.scales = w->scales; v.zeros = w->zeros;
    v.block_params = w->block_params;
    return v;
}

// One dequantised element, evaluated with exactly the reference's operations:
// no fused multiply-add, same operand order.
__device__ __forceinline__ float dequant_element(const QView &v, size_t idx) {
    switch (v.fmt) {
    case FMT_I8: {  // dequant.rs:8-16: code as f32 * scale
        float c = (float)((const int8_t *)v.codes)[idx];
        return __fmul_rn(c, v.scales[idx / v.K]);
    }
    case FMT_I4_AFFINE: {  // int4.rs:88: (q as f32 - zero) * scale
        uint8_t byte = ((const uint8_t *)v.codes)[idx >> 1];
        float q = (float)((idx & 1) ? (byte >> 4) : (byte & 0x0f));
        size_t g = idx / (size_t)v.group;
        return __fmul_rn(__fsub_rn(q, v.zeros[g]), v.scales[g]);
    }
    case FMT_Q4KM: {  // gguf_quant.rs:45-46: q as f32 * scale + min
        uint8_t byte = ((const uint8_t *)v.codes)[idx >> 1];
        float q = (float)((idx & 1) ? (byte >> 4) : (byte & 0x0f));
        uint32_t p = v.block_params[idx >> 8];
        float s = f16_bits_to_f32((uint16_t)(p & 0xffffu)), m = f16_bits_to_f32((uint16_t)(p >> 16));
        return __fadd_rn(__fmul_rn(q, s), m);
    }
    default: {  // FMT_W4A16: (q - z) * s with bf16 s, u4 z widened to f32
        int n = (int)(idx / v.K), k = (int)(idx % v.K);
        int g = k / v.group;
        W4Layout L{v.N, v.K, v.group};
        uint32_t word = ((const uint32_t *)v.codes)[L.code_index(n, k >> 3)];
        int e = k & 7, slot = (e >> 1) + 4 * (e & 1);
        float q = (float)((word >> (4 * slot)) & 0xFu);
        uint32_t p = ((const uint32_t *)v.codes)[L.param_index(n, g)];
        float z = (float)((p >> 16) & 0xFu);
        float s = bf16_bits_to_f32((uint16_t)(p & 0xffffu));
        return __fmul_rn(__fsub_rn(q, z), s);
    }
    }
}

template <typename T>
__global__ void dequant_kernel(QView v, T *out, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(dequant_element(v, i));
}

AB2_API int ab2_qweight_dequant(const ab2_qweight *w, void *out_dev, ab2_dtype dtype,
                                ab2_stream stream) {
    AB2_REQUIRE(w != nullptr && out_dev != nullptr, AB2_ERR_BAD_ARG, "null argument");
    size_t n = (size_t)w->N * w->K;
    QView v = view_of(w);
    cudaStream_t s = (cudaStream_t)stream;
    unsigned blocks = (unsigned)std::min<size_t>(ceil_div(n, 256), 148 * 32);
    switch (dtype) {
    case AB2_F32: dequant_kernel<float><<<blocks, 256, 0, s>>>(v, (float *)out_dev, n); break;
    case AB2_F16: dequant_kernel<__half><<<blocks, 256, 0, s>>>(v, (__half *)out_dev, n); break;
    case AB2_BF16: dequant_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(v, (__nv_bfloat16 *)out_dev, n); break;
    default: return fail(AB2_ERR_BAD_DTYPE, "unsupported output dtype %d", (int)dtype);
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

// ---------------------------------------------------------------------------
// device-side quantisers (reference arithmetic; IEEE division, roundf = half
// away from zero, saturating casts)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float clamp_f(float v, float lo, float hi) {
    // f32::clamp keeps NaN; the saturating cast that follows maps NaN to 0.
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}
__device__ __forceinline__ int8_t sat_i8(float v) {
    if (v != v) return 0;
    return (int8_t)fminf(fmaxf(v, -128.f), 127.f);
}
__device__ __forceinline__ uint8_t sat_u8(float v) {
    if (v != v) return 0;
    return (uint8_t)fminf(fmaxf(v, 0.f), 255.f);
}

// max |w| over a range per block -> atomicMax on the bit pattern (non-negative
// floats order like unsigned integers; NaN is skipped as f32::max does).
__global__ void absmax_partial_kernel(const float *w, size_t n, unsigned *out_bits) {
    float m = 0.f;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        m = fmaxf(m, fabsf(w[i]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));
}

__global__ void i8_tensor_scale_kernel(const unsigned *max_bits, float *scales, int N) {
    float max_abs = __uint_as_float(*max_bits);
    float scale = (max_abs <= FLT_EPSILON) ? 1.0f : __fdiv_rn(max_abs, 127.0f);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x)
        scales[i] = scale;
}

__global__ void i8_row_scale_kernel(const float *w, int N, int K, float *scales) {
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const float *r = w + (size_t)row * K;
    float m = 0.f;
    for (int k = threadIdx.x & 31; k < K; k += 32) m = fmaxf(m, fabsf(r[k]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) scales[row] = (m <= FLT_EPSILON) ? 1.0f : __fdiv_rn(m, 127.0f);
}

__global__ void i8_encode_kernel(const float *w, const float *scales, int K, size_t n,
                                 int8_t *codes) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float s = scales[i / K];
        codes[i] = sat_i8(clamp_f(roundf(__fdiv_rn(w[i], s)), -127.f, 127.f));
    }
}

AB2_API int ab2_qweight_quantise_i8(ab2_qweight **out, const float *w_dev, int N, int K,
                                    int per_channel, ab2_stream stream) {
    AB2_REQUIRE(w_dev != nullptr, AB2_ERR_BAD_ARG, "null input pointer");
    TRY(make_i8(out, N, K, !per_channel));
    ab2_qweight *w = *out;
    cudaStream_t s = (cudaStream_t)stream;
    size_t n = (size_t)N * K;
    unsigned blocks = (unsigned)std::min<size_t>(ceil_div(n, 256), 148 * 16);
    if (per_channel) {
        i8_row_scale_kernel<<<(N + 7) / 8, 256, 0, s>>>(w_dev, N, K, w->scales);
    } else {
        unsigned *bits = nullptr;
        AB2_CUDA(cudaMalloc((void **)&bits, 4));
        AB2_CUDA(cudaMemsetAsync(bits, 0, 4, s));
        absmax_partial_kernel<<<blocks, 256, 0, s>>>(w_dev, n, bits);
        i8_tensor_scale_kernel<<<(N + 255) / 256, 256, 0, s>>>(bits, w->scales, N);
        AB2_CUDA(cudaStreamSynchronize(s));
        cudaFree(bits);
    }
    i8_encode_kernel<<<blocks, 256, 0, s>>>(w_dev, w->scales, K, n, (int8_t *)w->codes);
    AB2_LAUNCH_CHECK();
    AB2_CUDA(cudaStreamSynchronize(s));
    return AB2_OK;
}

// One warp per flat group (int4.rs:16-35).  `group` is even, so every group
// starts on a byte boundary and a lane owns whole bytes.
__global__ void i4_affine_quantise_kernel(const float *w, size_t n, int group, uint8_t *packed,
                                          float *scales, float *zeros, size_t ngroups) {
    size_t g = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (g >= ngroups) return;
    int lane = threadIdx.x & 31;
    size_t start = g * (size_t)group;
    int len = (int)min((size_t)group, n - start);
    float mn = INFINITY, mx = -INFINITY;
    for (int i = lane; i < len; i += 32) {
        float v = w[start + i];
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    float range = __fsub_rn(mx, mn);
    float scale = (fabsf(range) <= FLT_EPSILON) ? 1.0f : __fdiv_rn(range, 15.0f);
    float zero = roundf(__fdiv_rn(-mn, scale));
    if (lane == 0) { scales[g] = scale; zeros[g] = zero; }
    for (int p = lane; 2 * p < len; p += 32) {
        float a = w[start + 2 * p];
        uint8_t lo = sat_u8(clamp_f(roundf(__fadd_rn(__fdiv_rn(a, scale), zero)), 0.f, 15.f));
        uint8_t hi = 0;
        if (2 * p + 1 < len) {
            float b = w[start + 2 * p + 1];
            hi = sat_u8(clamp_f(roundf(__fadd_rn(__fdiv_rn(b, scale), zero)), 0.f, 15.f));
        }
        packed[(start >> 1) + p] = (uint8_t)((lo & 0x0f) | (hi << 4));
    }
}

AB2_API int ab2_qweight_quantise_i4_affine(ab2_qweight **out, const float *w_dev, int N, int K,
                                           int group, ab2_stream stream) {
    AB2_REQUIRE(w_dev != nullptr, AB2_ERR_BAD_ARG, "null input pointer");
    AB2_REQUIRE(group > 0 && group % 2 == 0, AB2_ERR_BAD_SHAPE, "device quantiser needs an even group size, got %d", group);
    TRY(make_i4_affine(out, N, K, group));
    ab2_qweight *w = *out;
    size_t n = (size_t)N * K, ng = ceil_div(n, (size_t)group);
    cudaStream_t s = (cudaStream_t)stream;
    i4_affine_quantise_kernel<<<(unsigned)ceil_div(ng, 8), 256, 0, s>>>(w_dev, n, group, (uint8_t *)w->codes, w->scales, w->zeros, ng);
    AB2_LAUNCH_CHECK();
    AB2_CUDA(cudaStreamSynchronize(s));
    return AB2_OK;
}

// One warp per 256-value block (gguf_quant.rs:7-36); the tail block is padded
// with zeros before min/max are taken (gguf.rs:218-221).
__global__ void q4km_quantise_kernel(const float *w, size_t n, uint8_t *codes, uint32_t *params,
                                     size_t nblocks) {
    size_t b = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= nblocks) return;
    int lane = threadIdx.x & 31;
    size_t start = b * 256;
    float vals[8];
    float mn = INFINITY, mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // lane owns pairs p = lane + 32*j  -> elements 2p, 2p+1
        size_t i0 = start + 2 * (size_t)(lane + 32 * j);
        vals[2 * j] = i0 < n ? w[i0] : 0.f;
        vals[2 * j + 1] = i0 + 1 < n ? w[i0 + 1] : 0.f;
        mn = fminf(mn, fminf(vals[2 * j], vals[2 * j + 1]));
        mx = fmaxf(mx, fmaxf(vals[2 * j], vals[2 * j + 1]));
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    float range = __fsub_rn(mx, mn);
    float scale = (fabsf(range) <= FLT_EPSILON) ? 1.0f : __fdiv_rn(range, 15.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint8_t qa = sat_u8(clamp_f(roundf(__fdiv_rn(__fsub_rn(vals[2 * j], mn), scale)), 0.f, 15.f));
        uint8_t qb = sat_u8(clamp_f(roundf(__fdiv_rn(__fsub_rn(vals[2 * j + 1], mn), scale)), 0.f, 15.f));
        codes[b * 128 + lane + 32 * j] = (uint8_t)(qa | (qb << 4));
    }
    if (lane == 0) {
        // Custom f32 -> f16 of gguf_quant.rs:52-83: round half up on bit 12,
        // flush half_exp < -10 to signed zero.
        auto enc = [](float value) -> uint32_t {
            uint32_t bits = __float_as_uint(value);
            uint32_t sign = (bits >> 16) & 0x8000u;
            int exp = (int)((bits >> 23) & 0xffu);
            uint32_t mant = bits & 0x7fffffu;
            if (exp == 255) return sign | (mant == 0 ? 0x7c00u : 0x7e00u);
            int half_exp = exp - 127 + 15;
            if (half_exp >= 31) return sign | 0x7c00u;
            if (half_exp <= 0) {
                if (half_exp < -10) return sign;
                mant |= 0x800000u;
                int shift = 14 - half_exp;
                uint32_t hm = (mant >> shift) & 0xffffu;
                if ((mant >> (shift - 1)) & 1u) hm = (hm + 1u) & 0xffffu;
                return sign | hm;
            }
            uint32_t half = sign | ((uint32_t)half_exp << 10) | (mant >> 13);
            if (mant & 0x1000u) half = (half + 1u) & 0xffffu;
            return half;
        };
        params[b] = enc(scale) | (enc(mn) << 16);
    }
}

AB2_API int ab2_qweight_quantise_q4km(ab2_qweight **out, const float *w_dev, int N, int K,
                                      ab2_stream stream) {
    AB2_REQUIRE(w_dev != nullptr, AB2_ERR_BAD_ARG, "null input pointer");
    TRY(make_q4km(out, N, K));
    ab2_qweight *w = *out;
    size_t n = (size_t)N * K, nb = ceil_div(n, 256);
    cudaStream_t s = (cudaStream_t)stream;
    q4km_quantise_kernel<<<(unsigned)ceil_div(nb, 8), 256, 0, s>>>(w_dev, n, (uint8_t *)w->codes, w->block_params, nb);
    AB2_LAUNCH_CHECK();
    AB2_CUDA(cudaStreamSynchronize(s));
    return AB2_OK;
}

// One warp per (row, group).  The stored scale is the bf16 rounding of the
// int4.rs scale; zero point and codes are derived from the stored scale.
__global__ void w4a16_quantise_kernel(const float *w, int N, int K, int group, uint32_t *tiles) {
    W4Layout L{N, K, group};
    int G = K / group;
    size_t wg = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wg >= (size_t)N * G) return;
    int lane = threadIdx.x & 31;
    int n = (int)(wg / G), g = (int)(wg % G);
    const float *src = w + (size_t)n * K + (size_t)g * group;
    float mn = INFINITY, mx = -INFINITY;
    for (int i = lane; i < group; i += 32) {
        mn = fminf(mn, src[i]);
        mx = fmaxf(mx, src[i]);
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    float range = __fsub_rn(mx, mn);
    float scale = (fabsf(range) <= FLT_EPSILON) ? 1.0f : __fdiv_rn(range, 15.0f);
    __nv_bfloat16 sb = __float2bfloat16_rn(scale);
    float s = __bfloat162float(sb);
    float zero = clamp_f(roundf(__fdiv_rn(-mn, s)), 0.f, 15.f);
    if (lane == 0)
        tiles[L.param_index(n, g)] =
            (uint32_t)__bfloat16_as_ushort(sb) | ((0xC300u | (uint32_t)sat_u8(zero)) << 16);
    for (int word = lane; word < group / 8; word += 32) {
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v = src[word * 8 + j];
            uint32_t q = sat_u8(clamp_f(roundf(__fadd_rn(__fdiv_rn(v, s), zero)), 0.f, 15.f));
            packed |= (q & 0xFu) << (4 * ((j >> 1) + 4 * (j & 1)));
        }
        tiles[L.code_index(n, g * (group / 8) + word)] = packed;
    }
}

AB2_API int ab2_qweight_quantise_w4a16(ab2_qweight **out, const float *w_dev, int N, int K,
                                       int group, ab2_stream stream) {
    AB2_REQUIRE(w_dev != nullptr, AB2_ERR_BAD_ARG, "null input pointer");
    TRY(make_w4a16(out, N, K, group));
    ab2_qweight *w = *out;
    size_t G = (size_t)K / group;
    cudaStream_t s = (cudaStream_t)stream;
    w4a16_quantise_kernel<<<(unsigned)ceil_div((size_t)N * G, 8), 256, 0, s>>>(
        w_dev, N, K, group, (uint32_t *)w->codes);
    AB2_LAUNCH_CHECK();
    AB2_CUDA(cudaStreamSynchronize(s));
    return AB2_OK;
}
