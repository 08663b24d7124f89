// Q4_K_M-style block weights (crates/aarambh-studio-quant/src/gguf_quant.rs:39-49: 256 values per
// block, 4-bit codes, one custom-f16 scale and minimum per block, w = q * scale + min), bf16
// activations, 1..8 tokens: the GEMV of a GGUF-loaded model, HBM-bound on K*N/2 bytes of codes plus
// 4 bytes of parameters per block.  The library keeps the codes and the parameters in two planes
// (split at load), which is what this kernel streams; K must be a multiple of 256 so that blocks do
// not straddle rows.
//
// One CTA owns a 16-row tile and its 8 warps take whole blocks of 256 columns in turn.  A lane
// reads 2 x 16 bytes of row r and of row r + 8 per block (its 32 columns of each half).  Codes stay
// in the reference's nibble order (element j of a 32-bit word at bits 4j): (w >> 4j) & 0x000F000F
// under 0x6400 is the f16 pair (1024 + q[j], 1024 + q[j + 4]), so the activations are staged with
// every group of 8 permuted to 0,4,1,5,2,6,3,7 and the pairs meet their columns in
// mma.sync.m16n8k16 (f16 x f16 -> f32; 16 rows as A, up to 8 tokens as the columns of B).  Per
// block the accumulator D and X = sum of the token's activations over the block give
//     y[t][n] += scale * (D - 1024 X) + min * X,
// in f32, and the power of two that scaled the token's activations into f16 range leaves at the end.
#include <algorithm>

#include "common.cuh"
#include "gemv_w4a16_m1.cuh"

using namespace ab2;

namespace ab2 {
namespace {

constexpr int Q4S_WARPS = 8;

__device__ __forceinline__ float f16_bits(uint32_t h) { return f16_bits_to_f32((uint16_t)h); }

__global__ void __launch_bounds__(256)
gemv_q4km_stream_kernel(const uint8_t *__restrict__ codes, const uint32_t *__restrict__ params,
                        const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y, int N, int K, int M) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KB = K >> 8;                                              // blocks per row
    __half *xs = reinterpret_cast<__half *>(smem_raw);                  // [M][K] f16, scaled, groups of 8 permuted
    float *xsum = reinterpret_cast<float *>(smem_raw + (size_t)M * K * 2);  // [KB][8]: X of token t over block b
    __shared__ float tok_unscale[8];
    __shared__ float warp_red[Q4S_WARPS][8];
    __shared__ float red[Q4S_WARPS][16][8];

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
        if (lane == 0) warp_red[warp][t] = amax;
    }
    for (int i = tid; i < KB * 8; i += 256) xsum[i] = 0.f;
    __syncthreads();
    for (int t = 0; t < M; ++t) {
        float amax = 0.f;
#pragma unroll
        for (int w = 0; w < Q4S_WARPS; ++w) amax = fmaxf(amax, warp_red[w][t]);
        int e = 141 - (int)((__float_as_uint(amax) >> 23) & 0xffu);  // largest magnitude into [2^14, 2^15)
        e = max(-100, min(100, e));
        const float sc = __uint_as_float((uint32_t)(e + 127) << 23);
        const uint4 *x4 = reinterpret_cast<const uint4 *>(x + (size_t)t * K);
        for (int i = tid; i < nvec; i += 256) {  // 32 consecutive vectors (one warp pass) are one block of 256
            const uint4 v = x4[i];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            __half h[8];
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                h[2 * j] = __float2half_rn(__uint_as_float(w[j] << 16) * sc);
                h[2 * j + 1] = __float2half_rn(__uint_as_float(w[j] & 0xffff0000u) * sc);
                sum += __half2float(h[2 * j]) + __half2float(h[2 * j + 1]);
            }
            // element order 0,4,1,5,2,6,3,7: the halves of a code-word pair are elements j and j + 4
            const __half2 p0 = __halves2half2(h[0], h[4]), p1 = __halves2half2(h[1], h[5]);
            const __half2 p2 = __halves2half2(h[2], h[6]), p3 = __halves2half2(h[3], h[7]);
            *reinterpret_cast<uint4 *>(xs + (size_t)t * K + (size_t)i * 8) =
                make_uint4(*reinterpret_cast<const uint32_t *>(&p0), *reinterpret_cast<const uint32_t *>(&p1),
                           *reinterpret_cast<const uint32_t *>(&p2), *reinterpret_cast<const uint32_t *>(&p3));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) xsum[(i >> 5) * 8 + t] = sum;  // nvec is a multiple of 32: the warp is whole
        }
        if (tid == 0) tok_unscale[t] = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    __syncthreads();

    // ---- main loop: this warp's blocks of 256 columns ------------------------------
    const int row_a = min(tile * 16 + r, N - 1), row_b = min(tile * 16 + r + 8, N - 1);
    const uint8_t *pa = codes + (size_t)row_a * (K >> 1) + c * 16;
    const uint8_t *pb = codes + (size_t)row_b * (K >> 1) + c * 16;
    const uint32_t *qa = params + (size_t)row_a * KB, *qb = params + (size_t)row_b * KB;
    const uint32_t xs_lane = smem_addr(xs) + (uint32_t)(r * K + c * 32) * 2;  // token r, this lane's 32 columns of a half
    const uint32_t has_x = r < M ? 1u : 0u;
    uint32_t k_mask = 0x000F000Fu, k_magic = 0x64006400u;
    asm volatile("" : "+r"(k_mask), "+r"(k_magic));
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // rows r (tokens 2c, 2c + 1) and r + 8
    uint4 xw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) xw[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int b0 = warp; b0 < KB; b0 += 2 * Q4S_WARPS) {
        // two blocks in flight per lane: 8 loads of 16 bytes and 4 parameter words
        uint4 wa[2][2], wb[2][2];
        uint32_t prm_a[2], prm_b[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int b = b0 + u * Q4S_WARPS;
            if (b < KB) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    wa[u][hf] = __ldcs(reinterpret_cast<const uint4 *>(pa + (size_t)b * 128 + hf * 64));
                    wb[u][hf] = __ldcs(reinterpret_cast<const uint4 *>(pb + (size_t)b * 128 + hf * 64));
                }
                prm_a[u] = __ldg(qa + b);
                prm_b[u] = __ldg(qb + b);
            } else {
                wa[u][0] = wa[u][1] = wb[u][0] = wb[u][1] = make_uint4(0u, 0u, 0u, 0u);
                prm_a[u] = prm_b[u] = 0u;
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int b = b0 + u * Q4S_WARPS;
            if (b >= KB) break;
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                for (int i = 0; i < 4; ++i) lds128_if(has_x, xs_lane + (uint32_t)(b * 256 + hf * 128) * 2 + i * 16, xw[i]);
                const uint32_t ua[4] = {wa[u][hf].x, wa[u][hf].y, wa[u][hf].z, wa[u][hf].w};
                const uint32_t ub[4] = {wb[u][hf].x, wb[u][hf].y, wb[u][hf].z, wb[u][hf].w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t xb[4] = {xw[w].x, xw[w].y, xw[w].z, xw[w].w};
                    const uint32_t a0 = and_or(ua[w], k_mask, k_magic), a1 = and_or(ub[w], k_mask, k_magic);
                    const uint32_t a2 = and_or(ua[w] >> 4, k_mask, k_magic), a3 = and_or(ub[w] >> 4, k_mask, k_magic);
                    const uint32_t a4 = and_or(ua[w] >> 8, k_mask, k_magic), a5 = and_or(ub[w] >> 8, k_mask, k_magic);
                    const uint32_t a6 = and_or(ua[w] >> 12, k_mask, k_magic), a7 = and_or(ub[w] >> 12, k_mask, k_magic);
                    mma_f16_16816(d, a0, a1, a2, a3, xb[0], xb[1]);
                    mma_f16_16816(d, a4, a5, a6, a7, xb[2], xb[3]);
                }
            }
            // y += scale (D - 1024 X) + min X, with X of tokens 2c and 2c + 1 over this block
            const float2 X = *reinterpret_cast<const float2 *>(xsum + b * 8 + 2 * c);
            const float sa = f16_bits(prm_a[u] & 0xffffu), ma = f16_bits(prm_a[u] >> 16);
            const float sb = f16_bits(prm_b[u] & 0xffffu), mb = f16_bits(prm_b[u] >> 16);
            acc[0] += fmaf(sa, d[0] - 1024.f * X.x, ma * X.x);
            acc[1] += fmaf(sa, d[1] - 1024.f * X.y, ma * X.y);
            acc[2] += fmaf(sb, d[2] - 1024.f * X.x, mb * X.x);
            acc[3] += fmaf(sb, d[3] - 1024.f * X.y, mb * X.y);
        }
    }
    red[warp][r][2 * c] = acc[0];
    red[warp][r][2 * c + 1] = acc[1];
    red[warp][r + 8][2 * c] = acc[2];
    red[warp][r + 8][2 * c + 1] = acc[3];
    __syncthreads();
    if (tid < 128) {
        const int row = tid >> 3, tok = tid & 7;
        const int n = tile * 16 + row;
        if (tok < M && n < N) {
            float D = 0.f;
#pragma unroll
            for (int w = 0; w < Q4S_WARPS; ++w) D += red[w][row][tok];
            y[(size_t)tok * N + n] = __float2bfloat16_rn(D * tok_unscale[tok]);
        }
    }
}

}  // namespace

bool qlinear_q4km_stream_eligible(const ab2_qweight *w, ab2_dtype dtype, int M) {
    return w->fmt == FMT_Q4KM && dtype == AB2_BF16 && M >= 1 && M <= 8 && w->K % 256 == 0 &&
           (size_t)M * w->K * 2 + (size_t)(w->K / 256) * 32 <= 96 * 1024;
}

int qlinear_q4km_stream(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    const size_t smem = (size_t)M * w->K * 2 + (size_t)(w->K / 256) * 32;
    static bool configured[64] = {false};
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!configured[dev]) {
        AB2_CUDA(cudaFuncSetAttribute(gemv_q4km_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        configured[dev] = true;
    }
    cudaError_t e = launch_kernel(gemv_q4km_stream_kernel, dim3((w->N + 15) / 16), dim3(256), smem, s, (const uint8_t *)w->codes,
                                  (const uint32_t *)w->block_params, (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, w->N, w->K, M);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "Q4_K_M GEMV launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

}  // namespace ab2
