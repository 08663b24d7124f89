// W8A16 decode GEMV: INT8 symmetric weights with one f32 scale per output row
// (per-output-channel absmax, crates/aarambh-studio-quant/src/qat.rs:140-169; a
// per-tensor scale, absmax.rs:7-24, is the same with the scale replicated), bf16
// activations, 1..8 tokens.  HBM-bound: the kernel streams K*N bytes of codes.
//
// One CTA owns a 16-row tile of the weight and its 8 warps split K in chunks of
// 64 columns.  A lane reads 16 bytes of row r and 16 of row r + 8 per chunk
// (every 32-byte sector fetched is used in full; several chunks are in flight
// per lane before the first is consumed).  A byte b becomes the f16 value
// 1152 + b exactly: (b ^ 0x80) is b + 128 as an unsigned byte, and PRMT places it
// under the exponent of 1024 (0x6400 | u) - one XOR per four weights and one PRMT
// per pair, no arithmetic.  The pairs feed mma.sync.m16n8k16 (f16 x f16 -> f32)
// with the 16 rows as A and up to 8 tokens as the columns of B; the 1152 leaves
// at the end through T = sum of the token's activations:
//     y[t][n] = scale[n] * (D[n][t] - 1152 T[t]) / 2^e[t].
// Activations are staged once per CTA as f16 scaled by a power of two per token
// (exact for bf16 inputs whose magnitudes lie within 2^25 of the token's largest).
#include <algorithm>

#include "common.cuh"
#include "gemv_w4a16_m1.cuh"

using namespace ab2;

namespace ab2 {
int device_sm_count();
namespace {

constexpr int I8S_WARPS = 8;
// Chunks in flight per warp are a template argument: 4 for K up to 8192 (6 gives 0.51 against 0.59 of
// HBM on 4096 x 14336, 8 gives 0.38: registers cost occupancy), 6 for longer rows (0.56 against 0.49 on
// 14336 x 4096: more iterations per warp to overlap).

template <typename T>
__device__ __forceinline__ void store_out(T *y, size_t i, float v) { y[i] = from_f32<T>(v); }

template <int RT, int I8S_UNROLL>  // RT: 16-row tiles per CTA (the activation fragments of a chunk serve all of them)
__global__ void __launch_bounds__(256)
gemv_i8_stream_kernel(const int8_t *__restrict__ codes, const float *__restrict__ scales,
                      const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y, int N, int K, int M) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half *xs = reinterpret_cast<__half *>(smem_raw);                 // [M][K] f16, scaled
    __shared__ float tok_T[8], tok_unscale[8];
    __shared__ float warp_red[I8S_WARPS][8][2];
    __shared__ float red[I8S_WARPS][16 * RT][8];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, c = lane & 3;
    const int tile = blockIdx.x;

    pdl_wait();
    pdl_launch_dependents();

    // ---- activations: per token, the largest magnitude picks the power of two ----
    const int nvec = K >> 3;
    for (int t = 0; t < M; ++t) {
        const uint4 *x4 = reinterpret_cast<const uint4 *>(x + (size_t)t * K);
        float amax = 0.f;
        for (int i = tid; i < nvec; i += 256) {
            const uint4 v = x4[i];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xffff0000u))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) warp_red[warp][t][0] = amax;
    }
    __syncthreads();
    for (int t = 0; t < M; ++t) {
        float amax = 0.f;
#pragma unroll
        for (int w = 0; w < I8S_WARPS; ++w) amax = fmaxf(amax, warp_red[w][t][0]);
        int e = 141 - (int)((__float_as_uint(amax) >> 23) & 0xffu);  // largest magnitude into [2^14, 2^15)
        e = max(-100, min(100, e));
        const float sc = __uint_as_float((uint32_t)(e + 127) << 23);
        const uint4 *x4 = reinterpret_cast<const uint4 *>(x + (size_t)t * K);
        float sum = 0.f;
        for (int i = tid; i < nvec; i += 256) {
            const uint4 v = x4[i];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 hh = __floats2half2_rn(__uint_as_float(w[j] << 16) * sc, __uint_as_float(w[j] & 0xffff0000u) * sc);
                h[j] = *reinterpret_cast<const uint32_t *>(&hh);
                const float2 back = __half22float2(hh);
                sum += back.x + back.y;
            }
            *reinterpret_cast<uint4 *>(xs + (size_t)t * K + (size_t)i * 8) = make_uint4(h[0], h[1], h[2], h[3]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) warp_red[warp][t][1] = sum;
        if (tid == 0) tok_unscale[t] = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    __syncthreads();
    if (tid < M) {
        float T = 0.f;
#pragma unroll
        for (int w = 0; w < I8S_WARPS; ++w) T += warp_red[w][tid][1];
        tok_T[tid] = T;
    }

    // ---- main loop: this warp's chunks of 64 columns ------------------------------
    const int8_t *pa[RT], *pb[RT];
#pragma unroll
    for (int q = 0; q < RT; ++q) {
        pa[q] = codes + (size_t)min((tile * RT + q) * 16 + r, N - 1) * K + c * 16;
        pb[q] = codes + (size_t)min((tile * RT + q) * 16 + r + 8, N - 1) * K + c * 16;
    }
    const int nchunks = K >> 6;
    const uint32_t xs_lane = smem_addr(xs) + (uint32_t)(r * K + c * 16) * 2;  // token r, this lane's 16 columns
    const uint32_t has_x = r < M ? 1u : 0u;
    float d[RT][4];
#pragma unroll
    for (int q = 0; q < RT; ++q) d[q][0] = d[q][1] = d[q][2] = d[q][3] = 0.f;
    uint4 xw0 = make_uint4(0u, 0u, 0u, 0u), xw1 = make_uint4(0u, 0u, 0u, 0u);
    for (int ch0 = warp; ch0 < nchunks; ch0 += I8S_WARPS * (I8S_UNROLL)) {
        uint4 wa[I8S_UNROLL][RT], wb[I8S_UNROLL][RT];
#pragma unroll
        for (int u = 0; u < I8S_UNROLL; ++u) {
            const int ch = ch0 + u * I8S_WARPS;
#pragma unroll
            for (int q = 0; q < RT; ++q) {
                if (ch < nchunks) {
                    wa[u][q] = __ldcs(reinterpret_cast<const uint4 *>(pa[q] + (size_t)ch * 64));
                    wb[u][q] = __ldcs(reinterpret_cast<const uint4 *>(pb[q] + (size_t)ch * 64));
                } else {
                    wa[u][q] = wb[u][q] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < I8S_UNROLL; ++u) {
            const int ch = ch0 + u * I8S_WARPS;
            if (ch >= nchunks) break;
            lds128_if(has_x, xs_lane + ch * 128, xw0);
            lds128_if(has_x, xs_lane + ch * 128 + 16, xw1);
            const uint32_t xb[8] = {xw0.x, xw0.y, xw0.z, xw0.w, xw1.x, xw1.y, xw1.z, xw1.w};
#pragma unroll
            for (int q = 0; q < RT; ++q) {
                const uint32_t ua[4] = {wa[u][q].x ^ 0x80808080u, wa[u][q].y ^ 0x80808080u, wa[u][q].z ^ 0x80808080u, wa[u][q].w ^ 0x80808080u};
                const uint32_t ub[4] = {wb[u][q].x ^ 0x80808080u, wb[u][q].y ^ 0x80808080u, wb[u][q].z ^ 0x80808080u, wb[u][q].w ^ 0x80808080u};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // word j = columns 4j .. 4j+3 of this lane's 16: pairs (0,1) and (2,3)
                    const uint32_t a0 = __byte_perm(ua[j], 0x64646464u, 0x4140), a2 = __byte_perm(ua[j], 0x64646464u, 0x4342);
                    const uint32_t a1 = __byte_perm(ub[j], 0x64646464u, 0x4140), a3 = __byte_perm(ub[j], 0x64646464u, 0x4342);
                    mma_f16_16816(d[q], a0, a1, a2, a3, xb[2 * j], xb[2 * j + 1]);
                }
            }
        }
    }
    // d[0], d[1]: row r, tokens 2c, 2c+1; d[2], d[3]: row r + 8
#pragma unroll
    for (int q = 0; q < RT; ++q) {
        red[warp][q * 16 + r][2 * c] = d[q][0];
        red[warp][q * 16 + r][2 * c + 1] = d[q][1];
        red[warp][q * 16 + r + 8][2 * c] = d[q][2];
        red[warp][q * 16 + r + 8][2 * c + 1] = d[q][3];
    }
    __syncthreads();
    if (tid < 128 * RT) {
        const int row = tid >> 3, tok = tid & 7;
        const int n = tile * 16 * RT + row;
        if (tok < M && n < N) {
            float D = 0.f;
#pragma unroll
            for (int w = 0; w < I8S_WARPS; ++w) D += red[w][row][tok];
            const float v = scales[n] * ((D - 1152.f * tok_T[tok]) * tok_unscale[tok]);
            y[(size_t)tok * N + n] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace

bool qlinear_i8_stream_eligible(const ab2_qweight *w, ab2_dtype dtype, int M) {
    return w->fmt == FMT_I8 && dtype == AB2_BF16 && M >= 1 && M <= 8 && w->K % 64 == 0 &&
           (size_t)M * w->K * 2 <= 96 * 1024;
}

int qlinear_i8_stream(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    const size_t smem = (size_t)M * w->K * 2;
    static bool configured[64] = {false};
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!configured[dev]) {
        AB2_CUDA(cudaFuncSetAttribute(gemv_i8_stream_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        AB2_CUDA(cudaFuncSetAttribute(gemv_i8_stream_kernel<1, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        AB2_CUDA(cudaFuncSetAttribute(gemv_i8_stream_kernel<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        configured[dev] = true;
    }
    // two 16-row tiles per CTA once that still leaves every SM a few CTAs (the activations are staged per CTA)
    const int tiles = (w->N + 15) / 16;
    // measured: two tiles per CTA are slower up to 4 tokens (one token: 0.47 against 0.59 of HBM on
    // 4096 x 14336) and faster at 8, where staging the activations per CTA weighs most (32.7 against 44.7 us)
    const bool two = M >= 8;
    const int8_t *codes = (const int8_t *)w->codes;
    const float *scales = (const float *)w->scales;
    cudaError_t e;
    if (two)
        e = launch_kernel(gemv_i8_stream_kernel<2, 4>, dim3((tiles + 1) / 2), dim3(256), smem, s, codes, scales,
                          (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, w->N, w->K, M);
    else if (w->K > 8192)
        e = launch_kernel(gemv_i8_stream_kernel<1, 6>, dim3(tiles), dim3(256), smem, s, codes, scales,
                          (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, w->N, w->K, M);
    else
        e = launch_kernel(gemv_i8_stream_kernel<1, 4>, dim3(tiles), dim3(256), smem, s, codes, scales,
                          (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, w->N, w->K, M);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "INT8 GEMV launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

}  // namespace ab2
