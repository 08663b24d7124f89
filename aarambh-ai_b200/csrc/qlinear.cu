// QatLinear::forward over packed weights: shape checks and kernel selection.
#include "common.cuh"
#include "gemv_generic.cuh"

using namespace ab2;

namespace ab2 {

GemvArgs gemv_args_of(const ab2_qweight *w) {
    GemvArgs a;
    a.codes = w->codes; a.scales = w->scales; a.zeros = w->zeros;
    a.block_params = w->block_params; a.qzeros = w->qzeros; a.scales16 = w->scales16;
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

}  // namespace ab2

AB2_API int ab2_qlinear_forward(const ab2_qweight *w, const void *x_dev, int M, ab2_dtype dtype,
                                void *y_dev, ab2_stream stream) {
    int rc = qlinear_validate(w, x_dev, M, dtype, y_dev);
    if (rc != AB2_OK) return rc;
    return qlinear_generic(w, x_dev, M, dtype, y_dev, (cudaStream_t)stream);
}
