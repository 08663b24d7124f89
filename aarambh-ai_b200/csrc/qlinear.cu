// QatLinear::forward over packed weights: shape checks and kernel selection.
#include <algorithm>

#include "common.cuh"
#include "gemv_generic.cuh"
#include "gemv_w4a16_mma.cuh"

using namespace ab2;

namespace ab2 {

GemvArgs gemv_args_of(const ab2_qweight *w) {
    GemvArgs a;
    a.codes = w->codes; a.scales = w->scales; a.zeros = w->zeros;
    a.block_params = w->block_params;
    a.N = w->N; a.K = w->K; a.group = w->group;
    return a;
}

template <int FMT, typename T>
static int launch_generic(const ab2_qweight *w, const T *x, int M, T *y, cudaStream_t s) {
    GemvArgs a = gemv_args_of(w);
    dim3 grid((w->N + 7) / 8), block(256);
    for (int m0 = 0; m0 < M; m0 += 4) {
        int mv = M - m0 < 4 ? M - m0 : 4;
        if (mv == 1) gemv_generic_kernel<FMT, T, 1><<<grid, block, 0, s>>>(a, x, y, m0, 1);
        else if (mv == 2) gemv_generic_kernel<FMT, T, 2><<<grid, block, 0, s>>>(a, x, y, m0, 2);
        else gemv_generic_kernel<FMT, T, 4><<<grid, block, 0, s>>>(a, x, y, m0, mv);
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

template <typename T>
static int launch_generic_fmt(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    switch (w->fmt) {
    case FMT_I8: return launch_generic<FMT_I8, T>(w, (const T *)x, M, (T *)y, s);
    case FMT_I4_AFFINE: return launch_generic<FMT_I4_AFFINE, T>(w, (const T *)x, M, (T *)y, s);
    case FMT_Q4KM: return launch_generic<FMT_Q4KM, T>(w, (const T *)x, M, (T *)y, s);
    case FMT_W4A16: return launch_generic<FMT_W4A16, T>(w, (const T *)x, M, (T *)y, s);
    default: return fail(AB2_ERR_BAD_ARG, "unknown weight format %d", w->fmt);
    }
}

// Checks shared by every linear path.
int qlinear_validate(const ab2_qweight *w, const void *x, int M, ab2_dtype dtype, const void *y) {
    AB2_REQUIRE(w != nullptr, AB2_ERR_BAD_ARG, "weight handle is null");
    AB2_REQUIRE(x != nullptr && y != nullptr, AB2_ERR_BAD_ARG, "null activation pointer");
    AB2_REQUIRE(M > 0, AB2_ERR_BAD_SHAPE, "token count must be positive, got %d", M);
    AB2_REQUIRE(dtype == AB2_F32 || dtype == AB2_F16 || dtype == AB2_BF16, AB2_ERR_BAD_DTYPE,
                "unsupported activation dtype %d", (int)dtype);
    AB2_REQUIRE(w->K % 8 == 0, AB2_ERR_BAD_SHAPE, "in_features=%d must be a multiple of 8", w->K);
    AB2_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)y & (dtype_size(dtype) - 1)) == 0,
                AB2_ERR_BAD_ALIGN, "activations must be 16-byte aligned");
    if (w->fmt == FMT_I4_AFFINE)
        AB2_REQUIRE(w->group % 8 == 0, AB2_ERR_UNSUPPORTED,
                    "fused linear needs a group size that is a multiple of 8, got %d", w->group);
    return AB2_OK;
}

int qlinear_generic(const ab2_qweight *w, const void *x, int M, ab2_dtype dtype, void *y,
                    cudaStream_t s) {
    switch (dtype) {
    case AB2_F32: return launch_generic_fmt<float>(w, x, M, y, s);
    case AB2_F16: return launch_generic_fmt<__half>(w, x, M, y, s);
    default: return launch_generic_fmt<__nv_bfloat16>(w, x, M, y, s);
    }
}

thread_local bool g_pdl_launch = false;

// Per-device status word written by kernels whose bounded waits ran out.
static int *g_status_word[64] = {nullptr};
static int g_sm_count[64] = {0};

int device_status_word(int **out) {
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!g_status_word[dev]) {
        AB2_CUDA(cudaMalloc((void **)&g_status_word[dev], sizeof(int)));
        AB2_CUDA(cudaMemset(g_status_word[dev], 0, sizeof(int)));
        AB2_CUDA(cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
    }
    *out = g_status_word[dev];
    return AB2_OK;
}

int device_sm_count() {
    int dev = 0;
    cudaGetDevice(&dev);
    return (dev >= 0 && dev < 64 && g_sm_count[dev] > 0) ? g_sm_count[dev] : 148;
}

// Tensor-core decode GEMV: W4A16, group 128, bf16 activations.
bool qlinear_w4a16_mma_eligible(const ab2_qweight *w, ab2_dtype dtype) {
    return w->fmt == FMT_W4A16 && w->group == 128 && dtype == AB2_BF16;
}

template <int EPI>
static int launch_w4a16_stream(const ab2_qweight *w, const void *x, int M, void *y, const void *resid,
                               cudaStream_t s) {
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    const int tiles = (w->N + 15) / 16;
    const int grid = std::min(tiles, device_sm_count() * 4);
    const uint32_t *wt = (const uint32_t *)w->codes;
    const int out_n = EPI == W4_EPI_SWIGLU ? w->N / 2 : w->N;
    for (int m0 = 0; m0 < M; m0 += 16) {
        const __nv_bfloat16 *xp = (const __nv_bfloat16 *)x + (size_t)m0 * w->K;
        __nv_bfloat16 *yp = EPI == W4_EPI_F32 ? (__nv_bfloat16 *)((float *)y + (size_t)m0 * out_n)
                                              : (__nv_bfloat16 *)y + (size_t)m0 * out_n;
        const __nv_bfloat16 *rp = resid ? (const __nv_bfloat16 *)resid + (size_t)m0 * out_n : nullptr;
        int mv = M - m0 < 16 ? M - m0 : 16;
        cudaError_t e;
        if (mv <= 8) e = launch_kernel(gemv_w4a16_stream_kernel<1, EPI>, dim3(grid), dim3(256), 0, s, wt, xp, yp, rp, w->N, w->K, mv, status);
        else e = launch_kernel(gemv_w4a16_stream_kernel<2, EPI>, dim3(grid), dim3(256), 0, s, wt, xp, yp, rp, w->N, w->K, mv, status);
        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "GEMV launch failed: %s", cudaGetErrorString(e));
    }
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

int qlinear_w4a16_mma(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    return launch_w4a16_stream<W4_EPI_STORE>(w, x, M, y, nullptr, s);
}
// y = resid + x . W^T (resid may be y)
int qlinear_w4a16_mma_add(const ab2_qweight *w, const void *x, int M, void *y, const void *resid, cudaStream_t s) {
    return launch_w4a16_stream<W4_EPI_ADD>(w, x, M, y, resid, s);
}
// y[M][N] f32 = x . W^T, unrounded (partial sums of a row-parallel shard)
int qlinear_w4a16_mma_f32(const ab2_qweight *w, const void *x, int M, float *y, cudaStream_t s) {
    return launch_w4a16_stream<W4_EPI_F32>(w, x, M, y, nullptr, s);
}
// y[M][N/2] = silu(gate) * up for a gate|up weight interleaved in 8-row halves
int qlinear_w4a16_mma_swiglu(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    return launch_w4a16_stream<W4_EPI_SWIGLU>(w, x, M, y, nullptr, s);
}

int qlinear_w4a16_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s);

int qlinear_dispatch(const ab2_qweight *w, const void *x, int M, ab2_dtype dtype, void *y, cudaStream_t s) {
    if (qlinear_w4a16_mma_eligible(w, dtype)) {
        // Few tokens: HBM-bound GEMV on the warp MMA (16 tokens per pass).  The
        // tcgen05 GEMM tiles 128 output channels per CTA, which leaves most SMs
        // idle until the token count supplies the parallelism.
        if (M <= 64) return qlinear_w4a16_mma(w, x, M, y, s);
        return qlinear_w4a16_tc(w, x, M, y, s);
    }
    return qlinear_generic(w, x, M, dtype, y, s);
}

}  // namespace ab2

AB2_API int ab2_qlinear_forward(const ab2_qweight *w, const void *x_dev, int M, ab2_dtype dtype,
                                void *y_dev, ab2_stream stream) {
    int rc = qlinear_validate(w, x_dev, M, dtype, y_dev);
    if (rc != AB2_OK) return rc;
    return qlinear_dispatch(w, x_dev, M, dtype, y_dev, (cudaStream_t)stream);
}

AB2_API int ab2_device_status(int *status_host) {
    AB2_REQUIRE(status_host != nullptr, AB2_ERR_BAD_ARG, "null argument");
    int *word = nullptr;
    int rc = device_status_word(&word);
    if (rc != AB2_OK) return rc;
    AB2_CUDA(cudaDeviceSynchronize());
    AB2_CUDA(cudaMemcpy(status_host, word, sizeof(int), cudaMemcpyDeviceToHost));
    AB2_CUDA(cudaMemset(word, 0, sizeof(int)));
    return AB2_OK;
}
