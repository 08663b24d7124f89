// Fused dequantise + GEMV on CUDA cores with f32 arithmetic, for every weight
// format and activation type.  One warp owns one output row and walks K in
// 8-element words; each dequantised weight is formed exactly as the
// reference forms it ((q - z) * s, q * s + min, code * scale) before the FMA,
// so the only difference from dequantise-then-matmul is summation order.
// This is the path of the f32 Tiny model and of shapes the tensor-core GEMV
// does not take.
#pragma once

#include "common.cuh"
#include "w4a16_layout.cuh"

namespace ab2 {

struct GemvArgs {
    const void *codes;
    const float *scales, *zeros;
    const uint32_t *block_params;
    int N, K, group;
};

template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[8]) {
        float4 a = *reinterpret_cast<const float4 *>(p);
        float4 b = *reinterpret_cast<const float4 *>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(r[i] << 16);
            v[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
        }
    }
};
template <> struct Vec8<__half> {
    static __device__ __forceinline__ void load(const __half *p, float (&v)[8]) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};

// Dequantises the 8 weights of word `word` (elements k = 8*word .. 8*word+7) of row n.
template <int FMT>
__device__ __forceinline__ void dequant_word(const GemvArgs &a, int n, int word, float (&w)[8]) {
    if constexpr (FMT == FMT_I8) {
        const int8_t *c = (const int8_t *)a.codes + (size_t)n * a.K + (size_t)word * 8;
        uint2 raw = *reinterpret_cast<const uint2 *>(c);
        float s = a.scales[n];
        uint32_t r[2] = {raw.x, raw.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int8_t code = (int8_t)((r[j >> 2] >> (8 * (j & 3))) & 0xff);
            w[j] = __fmul_rn((float)code, s);
        }
    } else if constexpr (FMT == FMT_W4A16) {
        W4Layout L{a.N, a.K, a.group};
        const uint32_t *t = (const uint32_t *)a.codes;
        uint32_t raw = t[L.code_index(n, word)];
        uint32_t p = t[L.param_index(n, (word * 8) / a.group)];
        float s = bf16_bits_to_f32((uint16_t)(p & 0xffffu));
        float z = (float)((p >> 16) & 0xFu);
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // interleaved slots: element j sits in slot j/2 + 4*(j&1)
            int slot = (j >> 1) + 4 * (j & 1);
            w[j] = __fmul_rn(__fsub_rn((float)((raw >> (4 * slot)) & 0xFu), z), s);
        }
    } else {
        size_t flat = (size_t)n * a.K + (size_t)word * 8;
        uint32_t raw = ((const uint32_t *)a.codes)[flat >> 3];
        if constexpr (FMT == FMT_I4_AFFINE) {
            size_t g = flat / (size_t)a.group;
            float s = a.scales[g], z = a.zeros[g];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                w[j] = __fmul_rn(__fsub_rn((float)((raw >> (4 * j)) & 0xFu), z), s);
        } else if constexpr (FMT == FMT_Q4KM) {
            uint32_t p = a.block_params[flat >> 8];
            float s = f16_bits_to_f32((uint16_t)(p & 0xffffu));
            float m = f16_bits_to_f32((uint16_t)(p >> 16));
#pragma unroll
            for (int j = 0; j < 8; ++j)
                w[j] = __fadd_rn(__fmul_rn((float)((raw >> (4 * j)) & 0xFu), s), m);
        }
    }
}

// y[m, n] = sum_k x[m, k] * W[n, k] for M tokens, MT at a time: the warp keeps its row and
// walks the tokens itself (after the first group the row comes from the caches), so a call
// is one launch whatever M is.
template <int FMT, typename T, int MT>
__global__ void __launch_bounds__(256) gemv_generic_kernel(GemvArgs a, const T *x, T *y, int M) {
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= a.N) return;
    const int words = a.K >> 3;
    for (int m0 = 0; m0 < M; m0 += MT) {
        const int m_valid = min(MT, M - m0);
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;
        for (int word = lane; word < words; word += 32) {
            float w[8];
            dequant_word<FMT>(a, n, word, w);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m < m_valid) {
                    float xv[8];
                    Vec8<T>::load(x + (size_t)(m0 + m) * a.K + (size_t)word * 8, xv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[m] = fmaf(xv[j], w[j], acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < m_valid) y[(size_t)(m0 + m) * a.N + n] = from_f32<T>(v);
        }
    }
}

}  // namespace ab2
