// QatLinear::forward over packed weights: shape checks and kernel selection.
#include <algorithm>
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "gemv_generic.cuh"
#include "tp.cuh"
#include "gemv_w4a16_mma.cuh"
#include "gemv_w4a16_warp.cuh"
#include "gemv_w4a16_m1.cuh"
#include "gemv_w4a16_strip.cuh"

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
    // one launch whatever the token count: the kernel walks the tokens in groups of MT
    if (M == 1) gemv_generic_kernel<FMT, T, 1><<<grid, block, 0, s>>>(a, x, y, M);
    else if (M == 2) gemv_generic_kernel<FMT, T, 2><<<grid, block, 0, s>>>(a, x, y, M);
    else gemv_generic_kernel<FMT, T, 4><<<grid, block, 0, s>>>(a, x, y, M);
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

// Counts the times ab2_device_status found a wait that had run out.  Objects that keep
// counters in device memory compare it with the value they saw last and put their
// counters back to rest when it moved (a kernel that gave up may have left them part-way).
static int g_recovery_epoch = 0;
int device_recovery_epoch() { return g_recovery_epoch; }

int device_sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (g_sm_count[dev] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

// Tensor-core decode GEMV: W4A16, group 128, bf16 activations.
bool qlinear_w4a16_mma_eligible(const ab2_qweight *w, ab2_dtype dtype) {
    return w->fmt == FMT_W4A16 && w->group == 128 && dtype == AB2_BF16;
}

// Scratch of the warp-streaming GEMV (partial sums of tiles cut by a range
// boundary, and one counter per tile), one set per (device, stream): launches
// on one stream run in order and may share it, launches on different streams
// may overlap and must not.  A set is allocated the first time its stream is
// seen, which must not be while that stream is being captured: a caller that
// captures graphs calls w4a16_prepare_stream() (or runs one eager launch) first.
constexpr int W4W_MAX_TILES = 1 << 18;
struct GemvScratch {
    float *partials = nullptr;
    int *counters = nullptr;
    int max_ctas = 0;
};
static std::mutex g_scratch_mutex;
static std::map<std::pair<int, cudaStream_t>, GemvScratch> g_scratch;

static int gemv_scratch_for(cudaStream_t s, GemvScratch *out) {
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    auto key = std::make_pair(dev, s);
    auto it = g_scratch.find(key);
    if (it == g_scratch.end()) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(s, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return fail(AB2_ERR_UNSUPPORTED,
                        "first quantised linear on this stream is inside a graph capture: run one launch "
                        "on the stream before capturing (its scratch buffers are allocated then)");
        GemvScratch sc;
        sc.max_ctas = device_sm_count() * 3;
        // two partial tiles per warp of the warp kernels, or two partial tile sets per CTA of the strip kernel
        const size_t pbytes = std::max((size_t)sc.max_ctas * W4W_WARPS * 2 * W4W_SLOT_FLOATS,
                                       (size_t)device_sm_count() * 2 * W4S_MAX_SLOT_FLOATS) * sizeof(float);
        AB2_CUDA(cudaMalloc((void **)&sc.partials, pbytes));
        AB2_CUDA(cudaMalloc((void **)&sc.counters, W4W_MAX_TILES * sizeof(int)));
        AB2_CUDA(cudaMemset(sc.counters, 0, W4W_MAX_TILES * sizeof(int)));
        AB2_CUDA(cudaDeviceSynchronize());
        it = g_scratch.emplace(key, sc).first;
    }
    *out = it->second;
    return AB2_OK;
}

int w4a16_prepare_stream(cudaStream_t s) {
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    GemvScratch sc;
    return gemv_scratch_for(s, &sc);
}

// One token: activations prepared per CTA (gemv_w4a16_m1.cuh).  K bounds the
// shared memory of a CTA, so very wide inputs stay on the general kernel.
template <int EPI, int STAGES, int NV, bool NORM, bool PEER_IN = false>
static cudaError_t launch_w4a16_m1_inst(const ab2_qweight *w, const __nv_bfloat16 *x, const float *norm_w,
                                        float eps, __nv_bfloat16 *y, const __nv_bfloat16 *resid, int grid,
                                        const GemvScratch &sc, int *status, cudaStream_t s,
                                        const ab2_tp_peer_desc *peers = nullptr, __nv_bfloat16 *x_out = nullptr) {
    const size_t smem = w4m1_smem_bytes<STAGES>(w->K);
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_w4a16_m1_kernel<EPI, STAGES, NV, NORM, PEER_IN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 74 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_kernel(gemv_w4a16_m1_kernel<EPI, STAGES, NV, NORM, PEER_IN>, dim3(grid), dim3(256), smem, s,
                         (const uint32_t *)w->codes, x, norm_w, eps, y, resid, w->N, w->K, sc.partials,
                         sc.counters, status, peers, x_out);
}

template <int EPI>
static cudaError_t launch_w4a16_m1(const ab2_qweight *w, const __nv_bfloat16 *x, const float *norm_w, float eps,
                                   __nv_bfloat16 *y, const __nv_bfloat16 *resid, int grid, const GemvScratch &sc,
                                   int *status, cudaStream_t s, const ab2_tp_peer_desc *peers = nullptr,
                                   __nv_bfloat16 *x_out = nullptr) {
    if (peers) {  // tensor parallel: the input is the residual plus the exchanged partial sums (norm fused)
        if constexpr (EPI == W4_EPI_STORE || EPI == W4_EPI_SWIGLU) {
            if (w->K <= 8192)
                return launch_w4a16_m1_inst<EPI, 3, 4, true, true>(w, x, norm_w, eps, y, resid, grid, sc, status, s, peers, x_out);
            return launch_w4a16_m1_inst<EPI, 2, 8, true, true>(w, x, norm_w, eps, y, resid, grid, sc, status, s, peers, x_out);
        } else {
            return cudaErrorInvalidValue;
        }
    }
    if (w->K <= 8192) {
        if (norm_w) return launch_w4a16_m1_inst<EPI, 3, 4, true>(w, x, norm_w, eps, y, resid, grid, sc, status, s);
        return launch_w4a16_m1_inst<EPI, 3, 4, false>(w, x, norm_w, eps, y, resid, grid, sc, status, s);
    }
    if (norm_w) return launch_w4a16_m1_inst<EPI, 2, 8, true>(w, x, norm_w, eps, y, resid, grid, sc, status, s);
    return launch_w4a16_m1_inst<EPI, 2, 8, false>(w, x, norm_w, eps, y, resid, grid, sc, status, s);
}

// 9..32 tokens: the register-tiled strip kernel (gemv_w4a16_strip.cuh), one CTA per SM.
template <class S, int EPI>
static cudaError_t launch_w4a16_strip(const ab2_qweight *w, const __nv_bfloat16 *x, int M, __nv_bfloat16 *y,
                                      const __nv_bfloat16 *resid, const GemvScratch &sc, int *status,
                                      cudaStream_t s) {
    static_assert(S::SLOT_FLOATS <= W4S_MAX_SLOT_FLOATS, "the scratch holds two partial tile sets per CTA");
    static_assert(S::SMEM <= 227 * 1024, "shared memory of a CTA");
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_w4a16_strip_kernel<S, EPI>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    const int tiles = (w->N + 15) / 16, sets = (tiles + S::WS * S::RT - 1) / (S::WS * S::RT);
    const long long total = (long long)sets * (w->K / 128);
    const int grid = (int)std::min<long long>(device_sm_count(), total);
    return launch_kernel(gemv_w4a16_strip_kernel<S, EPI>, dim3(grid), dim3(S::WARPS * 32), S::SMEM, s,
                         (const uint32_t *)w->codes, x, y, resid, w->N, w->K, M, sc.partials, sc.counters, status);
}

constexpr int W4M1_MAX_K = 16384;
constexpr int W4M1_PLAIN_MAX_K = 8192;

int qlinear_w4a16_tc_decode(const ab2_qweight *w, const void *x, int M, void *y, const void *resid, int epi,
                            float *partials, int *counters, int max_ctas, cudaStream_t s);

template <int EPI>
static int launch_w4a16_stream(const ab2_qweight *w, const void *x, int M, void *y, const void *resid,
                               cudaStream_t s, const float *norm_w = nullptr, float eps = 0.f,
                               const ab2_tp_peer_desc *peers = nullptr, void *x_out = nullptr) {
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    const int tiles = (w->N + 15) / 16;
    AB2_REQUIRE(tiles <= W4W_MAX_TILES, AB2_ERR_UNSUPPORTED, "out_features=%d exceeds the %d rows the decode GEMV serves",
                w->N, W4W_MAX_TILES * 16);
    GemvScratch sc;
    rc = gemv_scratch_for(s, &sc);
    if (rc != AB2_OK) return rc;
    // Three resident CTAs per SM at most, and at least eight blocks per warp: small
    // weights are latency-bound, and fewer, longer ranges keep most cut tiles inside
    // one CTA (finished through shared memory).
    const long long total = (long long)tiles * (w->K / 128);
    // Small weights are latency-bound: what a launch costs is the serial work of one warp plus the
    // finishing of cut tiles.  One 16-row tile per CTA (G / 8 blocks per warp) keeps every cut inside a
    // CTA (finished through shared memory; a tile cut between CTAs goes through partial sums and a
    // counter in L2) and halves the blocks a warp walks: taken whenever it fits the resident CTAs and
    // leaves a warp at least 4 blocks and the SMs at least 1.7 CTAs each (the Large block's qkv, o and
    // down projections, 384 and 256 tiles: 557 -> 592 tok/s.  With fewer tiles the SMs that hold two CTAs
    // set the time while the others idle: the 224-tile gate|up shard of an 8-way split ran the whole step
    // at 470 tok/s this way against 535 with equal ranges, same box, same run).
    // Large weights keep equal ranges over every resident CTA: for them balance across SMs matters more
    // (one tile set per CTA on the gate|up weight: 488 tok/s).
    static const bool align_off = getenv("AB2_GEMV_ALIGN") != nullptr && atoi(getenv("AB2_GEMV_ALIGN")) == 0;
    const int G = w->K / 128;
    int grid = (int)std::min<long long>(sc.max_ctas, std::max<long long>(1, (total / 8 + W4W_WARPS - 1) / W4W_WARPS));
    if (!align_off && G % W4W_WARPS == 0 && G / W4W_WARPS >= 4 && tiles <= sc.max_ctas && tiles * 10 >= device_sm_count() * 17) grid = tiles;
    const uint32_t *wt = (const uint32_t *)w->codes;
    const int out_n = EPI == W4_EPI_SWIGLU ? w->N / 2 : w->N;
    // More than 8 tokens go in chunks of up to 32:
    //   9..24 tokens (and 25..32 on a weight of 24576 rows or more): the strip kernel - a warp multiplies
    //     64 or 32 rows by all tokens, so the activations it loads serve several weight blocks and the
    //     codes are unpacked once for every token.  On the largest shape it takes 96 / 113 / 150 us for
    //     16 / 24 / 32 tokens; the warp kernel needs 155 us per 16 tokens.
    //   25..32 tokens on narrower weights: the tensor-memory decode GEMM, whose pass costs the same
    //     whatever the token count (170 us on the largest shape, 15 / 26 / 27 us on 4096 x 4096,
    //     4096 x 14336, 14336 x 4096 against the strip kernel's 17 / 29 / 30 us).
    static const bool strip_off = getenv("AB2_GEMV_NO_STRIP") != nullptr;
    static const int strip_wide_n = getenv("AB2_STRIP_WIDE_N") ? atoi(getenv("AB2_STRIP_WIDE_N")) : 24576;
    if constexpr (EPI != W4_EPI_F32_PEER) {
        if (M >= 9 && !norm_w) {
            const bool tc_ok = w->N % 16 == 0;
            // equal chunks, in whole token tiles: 40 tokens go as 24 + 16, not as 32 + 8
            const int nchunks = (M + 31) / 32, chunk = ((M + nchunks - 1) / nchunks + 7) / 8 * 8;
            for (int m0 = 0; m0 < M; m0 += chunk) {
                const int mv = std::min(chunk, M - m0);
                const __nv_bfloat16 *xp = (const __nv_bfloat16 *)x + (size_t)m0 * w->K;
                __nv_bfloat16 *yp = EPI == W4_EPI_F32 ? (__nv_bfloat16 *)((float *)y + (size_t)m0 * out_n)
                                                      : (__nv_bfloat16 *)y + (size_t)m0 * out_n;
                const __nv_bfloat16 *rp = resid ? (const __nv_bfloat16 *)resid + (size_t)m0 * out_n : nullptr;
                if (!strip_off && mv >= 9 && (mv <= 24 || w->N >= strip_wide_n || !tc_ok)) {
                    cudaError_t e;
                    // token tiles, tiles per strip, strips x K slices of a CTA
                    switch ((mv + 7) / 8) {
                    case 2: e = launch_w4a16_strip<W4sShape<2, 2, 8, 2>, EPI>(w, xp, mv, yp, rp, sc, status, s); break;
                    case 3: e = launch_w4a16_strip<W4sShape<3, 4, 4, 2>, EPI>(w, xp, mv, yp, rp, sc, status, s); break;
                    default: e = launch_w4a16_strip<W4sShape<4, 4, 4, 2>, EPI>(w, xp, mv, yp, rp, sc, status, s); break;
                    }
                    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "GEMV launch failed: %s", cudaGetErrorString(e));
                } else if (tc_ok && mv >= 17) {
                    rc = qlinear_w4a16_tc_decode(w, xp, mv, yp, rp, EPI, sc.partials, sc.counters, sc.max_ctas, s);
                    if (rc != AB2_OK) return rc;
                } else {
                    for (int m1 = 0; m1 < mv; m1 += 16) {
                        const int mw = std::min(16, mv - m1);
                        const __nv_bfloat16 *xq = xp + (size_t)m1 * w->K;
                        __nv_bfloat16 *yq = EPI == W4_EPI_F32 ? (__nv_bfloat16 *)((float *)yp + (size_t)m1 * out_n)
                                                              : yp + (size_t)m1 * out_n;
                        const __nv_bfloat16 *rq = rp ? rp + (size_t)m1 * out_n : nullptr;
                        cudaError_t e =
                            mw > 8 ? launch_kernel(gemv_w4a16_warp_kernel<2, EPI>, dim3(grid), dim3(256), 0, s, wt, xq, yq,
                                                   rq, w->N, w->K, mw, sc.partials, sc.counters, status)
                                   : launch_kernel(gemv_w4a16_warp_kernel<1, EPI>, dim3(grid), dim3(256), 0, s, wt, xq, yq,
                                                   rq, w->N, w->K, mw, sc.partials, sc.counters, status);
                        if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "GEMV launch failed: %s", cudaGetErrorString(e));
                    }
                }
            }
            AB2_LAUNCH_CHECK();
            return AB2_OK;
        }
    }
    for (int m0 = 0; m0 < M; m0 += 16) {
        const __nv_bfloat16 *xp = (const __nv_bfloat16 *)x + (size_t)m0 * w->K;
        __nv_bfloat16 *yp = EPI == W4_EPI_F32_PEER ? (__nv_bfloat16 *)y  // descriptor of the peer exchange (one pass)
                            : EPI == W4_EPI_F32  ? (__nv_bfloat16 *)((float *)y + (size_t)m0 * out_n)
                                                 : (__nv_bfloat16 *)y + (size_t)m0 * out_n;
        const __nv_bfloat16 *rp = resid ? (const __nv_bfloat16 *)resid + (size_t)m0 * out_n : nullptr;
        int mv = M - m0 < 16 ? M - m0 : 16;
        cudaError_t e;
        if (norm_w && !(M == 1 && w->K <= W4M1_MAX_K))
            return fail(AB2_ERR_UNSUPPORTED, "the fused RMSNorm serves one token and K <= %d", W4M1_MAX_K);
        // One token: the kernel that prepares the activations per CTA, while K is small
        // next to the rows a CTA streams (or there is a norm to fuse); else the general one.
        if (M == 1 && (norm_w || w->K <= W4M1_PLAIN_MAX_K) && w->K <= W4M1_MAX_K)
            e = launch_w4a16_m1<EPI>(w, xp, norm_w, eps, yp, rp, grid, sc, status, s, peers, (__nv_bfloat16 *)x_out);
        else if (mv > 8)
            e = launch_kernel(gemv_w4a16_warp_kernel<2, EPI>, dim3(grid), dim3(256), 0, s, wt, xp, yp, rp, w->N,
                              w->K, mv, sc.partials, sc.counters, status);
        else
            e = launch_kernel(gemv_w4a16_warp_kernel<1, EPI>, dim3(grid), dim3(256), 0, s, wt, xp, yp, rp, w->N,
                              w->K, mv, sc.partials, sc.counters, status);
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
// the same partial sums stored into every rank's inbox of the peer exchange
int qlinear_w4a16_mma_f32_peer(const ab2_qweight *w, const void *x, int M, ab2_tp *tp, cudaStream_t s) {
    AB2_REQUIRE(M <= 16 && tp_peer_ready(tp, (size_t)M * w->N), AB2_ERR_BAD_ARG,
                "the peer exchange cannot take %d x %d sums", M, w->N);
    return launch_w4a16_stream<W4_EPI_F32_PEER>(w, x, M, (void *)tp->desc_dev, nullptr, s);
}
// y[M][N/2] = silu(gate) * up for a gate|up weight interleaved in 8-row halves
int qlinear_w4a16_mma_swiglu(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    return launch_w4a16_stream<W4_EPI_SWIGLU>(w, x, M, y, nullptr, s);
}

// One token with the RMSNorm of the input fused into the GEMV: y = epi(norm(x) . W^T).
bool qlinear_w4a16_norm_fusable(const ab2_qweight *w, ab2_dtype dtype, int M) {
    static const bool off = getenv("AB2_NO_NORM_FUSION") != nullptr;
    return !off && qlinear_w4a16_mma_eligible(w, dtype) && M == 1 && w->K <= W4M1_MAX_K &&
           (w->N + 15) / 16 <= W4W_MAX_TILES;
}
int qlinear_w4a16_norm(const ab2_qweight *w, const void *x, const float *norm_w, float eps, void *y, int epi,
                       cudaStream_t s) {
    switch (epi) {
    case W4_EPI_STORE: return launch_w4a16_stream<W4_EPI_STORE>(w, x, 1, y, nullptr, s, norm_w, eps);
    case W4_EPI_SWIGLU: return launch_w4a16_stream<W4_EPI_SWIGLU>(w, x, 1, y, nullptr, s, norm_w, eps);
    case W4_EPI_F32: return launch_w4a16_stream<W4_EPI_F32>(w, x, 1, y, nullptr, s, norm_w, eps);
    default: return fail(AB2_ERR_BAD_ARG, "unsupported epilogue %d for the fused RMSNorm", epi);
    }
}

// The same with the tensor-parallel exchange consumed in the prologue: the input is
// x + bf16(sum over ranks of the partial sums in the inbox); the new residual stream is
// written to x_out (a buffer other than x).
int qlinear_w4a16_norm_peer(const ab2_qweight *w, const void *x, const float *norm_w, float eps, void *y, int epi,
                            ab2_tp *tp, void *x_out, cudaStream_t s) {
    AB2_REQUIRE(tp_peer_ready(tp, (size_t)w->K) && x_out && x_out != x, AB2_ERR_BAD_ARG,
                "the peer exchange is not attached, too small, or x_out aliases x");
    switch (epi) {
    case W4_EPI_STORE: return launch_w4a16_stream<W4_EPI_STORE>(w, x, 1, y, nullptr, s, norm_w, eps, tp->desc_dev, x_out);
    case W4_EPI_SWIGLU: return launch_w4a16_stream<W4_EPI_SWIGLU>(w, x, 1, y, nullptr, s, norm_w, eps, tp->desc_dev, x_out);
    default: return fail(AB2_ERR_BAD_ARG, "unsupported epilogue %d for the fused exchange", epi);
    }
}

int qlinear_w4a16_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s);
bool qlinear_i8_stream_eligible(const ab2_qweight *w, ab2_dtype dtype, int M);
bool qlinear_q4km_stream_eligible(const ab2_qweight *w, ab2_dtype dtype, int M);
int qlinear_q4km_stream(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s);
int qlinear_i8_stream(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s);
bool qlinear_i8_tc_eligible(const ab2_qweight *w, ab2_dtype dtype, int M);
int qlinear_i8_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s);

int qlinear_dispatch(const ab2_qweight *w, const void *x, int M, ab2_dtype dtype, void *y, cudaStream_t s) {
    if (qlinear_w4a16_mma_eligible(w, dtype)) {
        // Up to 64 tokens: the HBM-bound decode kernels (one token, 2..8 tokens, chunks of 9..32
        // tokens).  The tcgen05 GEMM tiles 128 output channels per CTA, which leaves most SMs
        // idle until the token count supplies the parallelism.
        if (M <= 64) return qlinear_w4a16_mma(w, x, M, y, s);
        return qlinear_w4a16_tc(w, x, M, y, s);
    }
    // INT8 weights, bf16 activations, a few tokens: the HBM-bound streaming GEMV
    if (qlinear_i8_stream_eligible(w, dtype, M)) return qlinear_i8_stream(w, x, M, y, s);
    // more tokens: tcgen05 GEMM, the codes converted to bf16 on the way into the operand stages
    if (qlinear_i8_tc_eligible(w, dtype, M)) return qlinear_i8_tc(w, x, M, y, s);
    // Q4_K_M blocks (GGUF-loaded models), bf16 activations, a few tokens: the streaming GEMV over the two planes
    if (qlinear_q4km_stream_eligible(w, dtype, M)) return qlinear_q4km_stream(w, x, M, y, s);
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
    if (*status_host != 0) ++g_recovery_epoch;
    return AB2_OK;
}
