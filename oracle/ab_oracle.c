/*
 * CPU ORACLE — TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of aarambh-studio's quantise + infer
 * path.  It is the checker for the CUDA library and the timed CPU baseline; it is
 * never linked into, imported by, or called from the shipped library.  Only the
 * test-suite, the smoke check and the benchmark's cpu_baseline / reference arm
 * may build or call it.
 *
 * Pinning: every function below cites the reference file:line it restates
 * (paths relative to the reference project root).  The codec functions are pinned
 * against the known-answer vectors held in the reference's own unit tests
 * (crates/aarambh-studio-quant/src/{int4,gguf_quant,qat,kv_quant}.rs test
 * modules, crates/aarambh-studio-weights/src/gguf.rs tests,
 * crates/aarambh-studio-kernel/tests/kernel_tests.rs,
 * crates/aarambh-studio-nn/src/{kvcache,rope}.rs tests).  The matmul / softmax
 * summation order of the third-party tensor library the reference calls (Candle
 * 0.10.2 -> gemm 0.19, not vendored) is unspecified, so linear and end-to-end
 * logits are pinned only to tolerance: end-to-end token streams are
 * "parity unpinned" and are defined by this file's documented order.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: Rust never fuses a*b+c, so neither may this file.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* small helpers                                                              */
/* ------------------------------------------------------------------------- */

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of the parallel loops (a launcher may have exported
 * OMP_NUM_THREADS=1 for its worker processes). */
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Rust `x as i8` / `x as u8` after clamp: saturating, NaN -> 0
 * (crates/aarambh-studio-quant/src/absmax.rs:17, int4.rs:31). */
static inline int8_t cast_i8(float v) {
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}
static inline uint8_t cast_u8(float v) {
    if (v != v) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 255.0f) return 255;
    return (uint8_t)v;
}
/* Rust f32::clamp(lo, hi): NaN stays NaN. */
static inline float clampf(float v, float lo, float hi) {
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}
/* Rust f32::max / f32::min ignore a NaN operand (fold(…, f32::max)). */
static inline float rmaxf(float a, float b) { return fmaxf(a, b); }
static inline float rminf(float a, float b) { return fminf(a, b); }

/* ------------------------------------------------------------------------- */
/* custom f16 codec  (crates/aarambh-studio-quant/src/gguf_quant.rs:52-110)    */
/* ------------------------------------------------------------------------- */

/* Hand-written conversion: rounds half UP on bit 12 (not round-to-nearest-even),
 * flushes half_exp < -10 to signed zero (gguf_quant.rs:52-83). */
ORC_API uint16_t orc_f32_to_f16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int32_t exp = (int32_t)((bits >> 23) & 0xffu);
    uint32_t mant = bits & 0x7fffffu;
    if (exp == 255) return sign | (mant == 0 ? 0x7c00u : 0x7e00u);
    int32_t half_exp = exp - 127 + 15;
    if (half_exp >= 31) return sign | 0x7c00u;
    if (half_exp <= 0) {
        if (half_exp < -10) return sign;
        mant |= 0x800000u;
        int shift = 14 - half_exp;
        uint16_t half_mant = (uint16_t)(mant >> shift);
        if ((mant >> (shift - 1)) & 1u) half_mant = (uint16_t)(half_mant + 1u);
        return sign | half_mant;
    }
    uint16_t half = (uint16_t)(sign | ((uint16_t)half_exp << 10) | (uint16_t)(mant >> 13));
    if (mant & 0x1000u) half = (uint16_t)(half + 1u);
    return half;
}

/* Exact widening (gguf_quant.rs:86-110). */
ORC_API float orc_f16_to_f32(uint16_t value) {
    uint32_t sign = ((uint32_t)(value & 0x8000u)) << 16;
    int32_t exp = (value >> 10) & 0x1f;
    uint32_t mant = value & 0x03ffu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            uint32_t m = mant;
            int32_t e = -14;
            while ((m & 0x0400u) == 0) { m <<= 1; e -= 1; }
            m &= 0x03ffu;
            bits = sign | ((uint32_t)(e + 127) << 23) | (m << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (mant << 13);
    } else {
        bits = sign | ((uint32_t)(exp - 15 + 127) << 23) | (mant << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* IEEE round-to-nearest-even f32 -> f16, the conversion the `half` crate (2.7.1,
 * a crates.io dependency, not vendored) performs for Candle's to_dtype(F16)
 * used by the tensor-op fake-quant formula (qat.rs:100-108). */
ORC_API uint16_t orc_f32_to_f16_rne(float value) {
    uint32_t x;
    memcpy(&x, &value, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t man = x & 0x007fffffu;
    int32_t exp = (int32_t)((x >> 23) & 0xff);
    if (exp == 255) return (uint16_t)(sign | 0x7c00u | (man ? (0x0200u | (man >> 13)) : 0));
    int32_t unbiased = exp - 127;
    int32_t half_exp = unbiased + 15;
    if (half_exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (half_exp <= 0) {
        if (14 - half_exp > 24) return (uint16_t)sign;
        man |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - half_exp);
        uint32_t half_man = man >> shift;
        uint32_t round_bit = 1u << (shift - 1);
        if ((man & round_bit) != 0 && (man & (3u * round_bit - 1u)) != 0) half_man += 1;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = sign | ((uint32_t)half_exp << 10) | (man >> 13);
    uint32_t round_bit = 0x00001000u;
    if ((man & round_bit) != 0 && (man & (3u * round_bit - 1u)) != 0) half += 1;
    return (uint16_t)half;
}

/* bf16 helpers for the W4A16 formats (exact widening; RNE narrowing). */
ORC_API float orc_bf16_to_f32(uint16_t v) {
    uint32_t bits = ((uint32_t)v) << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}
ORC_API uint16_t orc_f32_to_bf16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

/* ------------------------------------------------------------------------- */
/* INT8 absmax                                                                */
/* ------------------------------------------------------------------------- */

/* Per-tensor: crates/aarambh-studio-quant/src/absmax.rs:7-24.  Returns scale. */
ORC_API float orc_quantise_absmax_i8(const float *values, size_t n, int8_t *codes) {
    float max_abs = 0.0f;
    for (size_t i = 0; i < n; ++i) max_abs = rmaxf(max_abs, fabsf(values[i]));
    float scale = (max_abs <= FLT_EPSILON) ? 1.0f : max_abs / 127.0f;
    for (size_t i = 0; i < n; ++i)
        codes[i] = cast_i8(clampf(roundf(values[i] / scale), -127.0f, 127.0f));
    return scale;
}

/* dequantise_i8: crates/aarambh-studio-quant/src/dequant.rs:8-16. */
ORC_API void orc_dequantise_i8(const int8_t *codes, size_t n, float scale, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = (float)codes[i] * scale;
}

/* Per-output-channel symmetric (one scale per row of a [N,K] matrix):
 * fake_quant_symmetric(…, OutputChannel) + safe_scale,
 * crates/aarambh-studio-quant/src/qat.rs:140-169.  The reference divides a Candle
 * tensor by the scalar 127.0; this restatement uses true f32 division, the same
 * expression absmax.rs:13 uses, which the reference's own test
 * (qat.rs:478-495) shows to be bit-identical on its vector. */
ORC_API void orc_quantise_absmax_i8_rows(const float *w, int N, int K, int8_t *codes,
                                         float *scales) {
    for (int n = 0; n < N; ++n) {
        const float *row = w + (size_t)n * K;
        float max_abs = 0.0f;
        for (int k = 0; k < K; ++k) max_abs = rmaxf(max_abs, fabsf(row[k]));
        float scale = (max_abs <= FLT_EPSILON) ? 1.0f : max_abs / 127.0f;
        scales[n] = scale;
        for (int k = 0; k < K; ++k)
            codes[(size_t)n * K + k] = cast_i8(clampf(roundf(row[k] / scale), -127.0f, 127.0f));
    }
}

ORC_API void orc_dequantise_i8_rows(const int8_t *codes, int N, int K, const float *scales,
                                    float *out) {
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k)
            out[(size_t)n * K + k] = (float)codes[(size_t)n * K + k] * scales[n];
}

/* ------------------------------------------------------------------------- */
/* affine INT4, 2 nibbles per byte, low nibble first                          */
/* (crates/aarambh-studio-quant/src/int4.rs:7-91)                              */
/* ------------------------------------------------------------------------- */

/* pack_i4_values: int4.rs:46-55. `packed` holds ceil(n/2) bytes. */
ORC_API void orc_pack_i4(const uint8_t *values, size_t n, uint8_t *packed) {
    for (size_t i = 0; i < n; i += 2) {
        uint8_t lo = values[i] & 0x0f;
        uint8_t hi = (i + 1 < n) ? (values[i + 1] & 0x0f) : 0;
        packed[i / 2] = (uint8_t)(lo | (hi << 4));
    }
}

/* unpack_i4_values: int4.rs:58-69. */
ORC_API void orc_unpack_i4(const uint8_t *packed, size_t n, uint8_t *values) {
    for (size_t i = 0; i < n; ++i) {
        uint8_t byte = packed[i / 2];
        values[i] = (i & 1) ? ((byte >> 4) & 0x0f) : (byte & 0x0f);
    }
}

/* quantise_affine_i4: int4.rs:7-43.  Groups are chunks of `group` over the
 * flattened tensor; scales/zeros hold ceil(n/group) entries. */
ORC_API void orc_quantise_affine_i4(const float *values, size_t n, size_t group,
                                    uint8_t *packed, float *scales, float *zeros) {
    uint8_t *q = (uint8_t *)malloc(n ? n : 1);
    size_t g = 0;
    for (size_t start = 0; start < n; start += group, ++g) {
        size_t end = start + group < n ? start + group : n;
        float mn = INFINITY, mx = -INFINITY;
        for (size_t i = start; i < end; ++i) {
            mn = rminf(mn, values[i]);
            mx = rmaxf(mx, values[i]);
        }
        float scale = (fabsf(mx - mn) <= FLT_EPSILON) ? 1.0f : (mx - mn) / 15.0f;
        float zero = roundf(-mn / scale);
        scales[g] = scale;
        zeros[g] = zero;
        for (size_t i = start; i < end; ++i)
            q[i] = cast_u8(clampf(roundf(values[i] / scale + zero), 0.0f, 15.0f));
    }
    orc_pack_i4(q, n, packed);
    free(q);
}

/* dequantise_packed_i4_to_vec: int4.rs:72-91 — (q - zero) * scale in f32. */
ORC_API void orc_dequantise_i4(const uint8_t *packed, size_t n, size_t group,
                               const float *scales, const float *zeros, float *out) {
    for (size_t i = 0; i < n; ++i) {
        uint8_t byte = packed[i / 2];
        uint8_t q = (i & 1) ? ((byte >> 4) & 0x0f) : (byte & 0x0f);
        size_t g = i / group;
        out[i] = ((float)q - zeros[g]) * scales[g];
    }
}

/* ------------------------------------------------------------------------- */
/* Q4_K_M-style 256-value blocks, 132 bytes each                              */
/* (crates/aarambh-studio-quant/src/gguf_quant.rs:1-49)                        */
/* ------------------------------------------------------------------------- */

#define Q4KM_BLOCK 256
#define Q4KM_BYTES 132

/* quantise_block_q4_k_m: gguf_quant.rs:7-36. */
ORC_API void orc_quantise_block_q4km(const float *w256, uint8_t *enc132) {
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < Q4KM_BLOCK; ++i) {
        mn = rminf(mn, w256[i]);
        mx = rmaxf(mx, w256[i]);
    }
    float scale = (fabsf(mx - mn) <= FLT_EPSILON) ? 1.0f : (mx - mn) / 15.0f;
    uint16_t hs = orc_f32_to_f16(scale), hm = orc_f32_to_f16(mn);
    enc132[0] = (uint8_t)(hs & 0xff);
    enc132[1] = (uint8_t)(hs >> 8);
    enc132[2] = (uint8_t)(hm & 0xff);
    enc132[3] = (uint8_t)(hm >> 8);
    for (int p = 0; p < Q4KM_BLOCK / 2; ++p) {
        float a = w256[2 * p], b = w256[2 * p + 1];
        uint8_t qa = cast_u8(clampf(roundf((a - mn) / scale), 0.0f, 15.0f));
        uint8_t qb = cast_u8(clampf(roundf((b - mn) / scale), 0.0f, 15.0f));
        enc132[4 + p] = (uint8_t)(qa | (qb << 4));
    }
}

/* dequantise_block_q4_k_m: gguf_quant.rs:39-49 — q * scale16 + min16. */
ORC_API void orc_dequantise_block_q4km(const uint8_t *enc132, float *out256) {
    float scale = orc_f16_to_f32((uint16_t)(enc132[0] | (enc132[1] << 8)));
    float mn = orc_f16_to_f32((uint16_t)(enc132[2] | (enc132[3] << 8)));
    for (int p = 0; p < Q4KM_BLOCK / 2; ++p) {
        uint8_t byte = enc132[4 + p];
        out256[2 * p] = (float)(byte & 0x0f) * scale + mn;
        out256[2 * p + 1] = (float)(byte >> 4) * scale + mn;
    }
}

/* encode_q4_k_m_tensor: crates/aarambh-studio-weights/src/gguf.rs:214-224.
 * Blocks over the flattened tensor, zero-padded tail.  `payload` holds
 * ceil(n/256)*132 bytes. */
ORC_API void orc_encode_q4km_tensor(const float *values, size_t n, uint8_t *payload) {
    size_t nblocks = (n + Q4KM_BLOCK - 1) / Q4KM_BLOCK;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < nblocks; ++b) {
        float block[Q4KM_BLOCK];
        size_t start = b * Q4KM_BLOCK;
        size_t len = n - start < Q4KM_BLOCK ? n - start : Q4KM_BLOCK;
        memset(block, 0, sizeof(block));
        memcpy(block, values + start, len * sizeof(float));
        orc_quantise_block_q4km(block, payload + b * Q4KM_BYTES);
    }
}

/* decode_q4_k_m_tensor: gguf.rs:226-241 (padding truncated). */
ORC_API void orc_decode_q4km_tensor(const uint8_t *payload, size_t n, float *out) {
    size_t nblocks = (n + Q4KM_BLOCK - 1) / Q4KM_BLOCK;
#pragma omp parallel for schedule(static)
    for (size_t b = 0; b < nblocks; ++b) {
        float block[Q4KM_BLOCK];
        orc_dequantise_block_q4km(payload + b * Q4KM_BYTES, block);
        size_t start = b * Q4KM_BLOCK;
        size_t len = n - start < Q4KM_BLOCK ? n - start : Q4KM_BLOCK;
        memcpy(out + start, block, len * sizeof(float));
    }
}

/* fake_quant_export_q4_k_m: crates/aarambh-studio-quant/src/qat.rs:83-112 — the
 * reference's second, independent statement of the same codec with tensor ops:
 * codes = clamp(round((v - min) / scale), 0, 15) from the f32 range, then
 * codes * f16(scale) + f16(min) with IEEE (nearest-even) f16 conversion. */
ORC_API void orc_fake_quant_export_q4km(const float *values, size_t n, float *out) {
    size_t nblocks = (n + Q4KM_BLOCK - 1) / Q4KM_BLOCK;
    for (size_t b = 0; b < nblocks; ++b) {
        float block[Q4KM_BLOCK];
        size_t start = b * Q4KM_BLOCK;
        size_t len = n - start < Q4KM_BLOCK ? n - start : Q4KM_BLOCK;
        memset(block, 0, sizeof(block));
        memcpy(block, values + start, len * sizeof(float));
        float mn = INFINITY, mx = -INFINITY;
        for (int i = 0; i < Q4KM_BLOCK; ++i) {
            mn = rminf(mn, block[i]);
            mx = rmaxf(mx, block[i]);
        }
        float range = mx - mn;
        float scale = (range <= FLT_EPSILON) ? 1.0f : range / 15.0f;
        float s16 = orc_f16_to_f32(orc_f32_to_f16_rne(scale));
        float m16 = orc_f16_to_f32(orc_f32_to_f16_rne(mn));
        for (size_t i = 0; i < len; ++i) {
            float code = clampf(roundf((block[i] - mn) / scale), 0.0f, 15.0f);
            out[start + i] = code * s16 + m16;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* W4A16 group-wise formats of the microbenchmarks                            */
/* ------------------------------------------------------------------------- */

/* GPTQ-style: qweight[N][K/8] u32, nibble j of a word (bits 4j..4j+3) is element
 * k = 8*word + j; scales[N][K/group] bf16; qzeros[N][ceil(K/group/8)] u32 with the same
 * nibble order along groups.  Dequant follows int4.rs:88 with the stored
 * parameters widened to f32: (q - z) * s. */
ORC_API void orc_dequant_w4a16(const uint32_t *qweight, const uint16_t *scales_bf16,
                               const uint32_t *qzeros, int N, int K, int group,
                               int awq_order, float *out) {
    static const int awq_slot_of[8] = {0, 4, 1, 5, 2, 6, 3, 7}; /* element -> slot */
    int G = K / group;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        for (int k = 0; k < K; ++k) {
            int g = k / group;
            uint32_t word = qweight[(size_t)n * (K / 8) + k / 8];
            int slot = awq_order ? awq_slot_of[k & 7] : (k & 7);
            float q = (float)((word >> (4 * slot)) & 0xfu);
            uint32_t zw = qzeros[(size_t)n * ((G + 7) / 8) + g / 8];
            int zslot = awq_order ? awq_slot_of[g & 7] : (g & 7);
            float z = (float)((zw >> (4 * zslot)) & 0xfu);
            float s = orc_bf16_to_f32(scales_bf16[(size_t)n * G + g]);
            out[(size_t)n * K + k] = (q - z) * s;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Linear: y = x . W^T   (crates/aarambh-studio-quant/src/qat.rs:315-348)      */
/* x [M,K], W [N,K] row-major, y [M,N]; f32, sequential k order per output.   */
/* ------------------------------------------------------------------------- */
ORC_API void orc_linear_f32(const float *x, const float *w, float *y, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        const float *wr = w + (size_t)n * K;
        for (int m = 0; m < M; ++m) {
            const float *xr = x + (size_t)m * K;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
            y[(size_t)m * N + n] = acc;
        }
    }
}

/* The same contraction as a SIMD GEMV would run it: 32 independent partial sums per
 * output (two vector registers of lanes), lanes added at the end.
 * The reference's CPU path calls Candle's matmul, which lands in the `gemm` crate's
 * SIMD micro-kernels (crates/aarambh-studio-quant/src/qat.rs:323; gemm 0.19 is not
 * vendored); their exact summation order is not published, so this form is not a
 * parity definition - it brackets the SPEED of that path next to the strict-order
 * loop above, and is used only by the timed CPU baseline.  Results differ from
 * orc_linear_f32 by summation order only. */
typedef float orc_v16 __attribute__((vector_size(64), aligned(4), may_alias));
__attribute__((target_clones("arch=skylake-avx512", "arch=haswell", "default")))
static float orc_dot_lanes(const float *x, const float *w, int K) {
    orc_v16 acc0 = {0}, acc1 = {0};
    int k = 0;
    for (; k + 32 <= K; k += 32) {
        acc0 += *(const orc_v16 *)(x + k) * *(const orc_v16 *)(w + k);
        acc1 += *(const orc_v16 *)(x + k + 16) * *(const orc_v16 *)(w + k + 16);
    }
    float sum = 0.0f;
    for (int j = 0; j < 16; ++j) sum += acc0[j] + acc1[j];
    for (; k < K; ++k) sum += x[k] * w[k];
    return sum;
}

ORC_API void orc_linear_f32_lanes(const float *x, const float *w, float *y, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        const float *wr = w + (size_t)n * K;
        for (int m = 0; m < M; ++m) y[(size_t)m * N + n] = orc_dot_lanes(x + (size_t)m * K, wr, K);
    }
}

/* Same contraction with f64 accumulation, used only to report how far both the
 * f32 oracle and the GPU are from the exact answer. */
ORC_API void orc_linear_f64acc(const float *x, const float *w, float *y, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) {
        const float *wr = w + (size_t)n * K;
        for (int m = 0; m < M; ++m) {
            const float *xr = x + (size_t)m * K;
            double acc = 0.0;
            for (int k = 0; k < K; ++k) acc += (double)xr[k] * (double)wr[k];
            y[(size_t)m * N + n] = (float)acc;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* RMSNorm                                                                    */
/* ------------------------------------------------------------------------- */

/* cpu_rms_norm_scalar: crates/aarambh-studio-kernel/src/cpu/simd_norm.rs:51-57. */
ORC_API void orc_rms_norm_scalar(const float *x, const float *w, float eps, float *out,
                                 int rows, int d) {
    for (int r = 0; r < rows; ++r) {
        const float *in = x + (size_t)r * d;
        float sum_sq = 0.0f;
        for (int i = 0; i < d; ++i) sum_sq += in[i] * in[i];
        float inv_rms = 1.0f / sqrtf(sum_sq / (float)d + eps);
        for (int i = 0; i < d; ++i) out[(size_t)r * d + i] = in[i] * inv_rms * w[i];
    }
}

/* rms_norm_row_avx2_fma summation order (simd_norm.rs:246-284): eight lane-wise
 * fused accumulators over blocks of 8, lanes added 0..7, then the scalar tail. */
ORC_API void orc_rms_norm_avx2fma_order(const float *x, const float *w, float eps, float *out,
                                        int rows, int d) {
    for (int r = 0; r < rows; ++r) {
        const float *in = x + (size_t)r * d;
        float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int idx = 0;
        while (idx + 8 <= d) {
            for (int l = 0; l < 8; ++l) lanes[l] = fmaf(in[idx + l], in[idx + l], lanes[l]);
            idx += 8;
        }
        float sum_sq = 0.0f;
        for (int l = 0; l < 8; ++l) sum_sq += lanes[l];
        for (int i = idx; i < d; ++i) sum_sq += in[i] * in[i];
        float inv_rms = 1.0f / sqrtf(sum_sq / (float)d + eps);
        for (int i = 0; i < d; ++i) out[(size_t)r * d + i] = in[i] * inv_rms * w[i];
    }
}

/* ------------------------------------------------------------------------- */
/* RoPE                                                                       */
/* ------------------------------------------------------------------------- */

/* base_inverse_frequencies (crates/aarambh-studio-nn/src/rope_scaling.rs:6-11) and
 * the cos/sin tables of RopeCache::from_inverse_frequencies
 * (crates/aarambh-studio-nn/src/rope.rs:43-72): f64 pow cast to f32, then
 * pos as f32 * freq in f32, cosf / sinf.  Tables are [max_seq, head_dim/2]. */
ORC_API void orc_rope_tables(int max_seq, int head_dim, double theta, float *cos_t,
                             float *sin_t) {
    int half = head_dim / 2;
    float *inv = (float *)malloc(sizeof(float) * (size_t)(half ? half : 1));
    for (int i = 0; i < half; ++i)
        inv[i] = (float)(1.0 / pow(theta, 2.0 * (double)i / (double)head_dim));
    for (int pos = 0; pos < max_seq; ++pos)
        for (int i = 0; i < half; ++i) {
            float val = (float)pos * inv[i];
            cos_t[(size_t)pos * half + i] = cosf(val);
            sin_t[(size_t)pos * half + i] = sinf(val);
        }
    free(inv);
}

/* RopeCache::apply_rotate (rope.rs:107-126): x [b, seq, heads, hd]; half-split
 * pairs (d, d+hd/2): x1*c - x2*s, x1*s + x2*c, table row offset+token. */
ORC_API void orc_rope_apply(const float *x, float *out, const float *cos_t, const float *sin_t,
                            int b, int seq, int heads, int hd, int offset) {
    int half = hd / 2;
    for (int bi = 0; bi < b; ++bi)
        for (int t = 0; t < seq; ++t)
            for (int h = 0; h < heads; ++h) {
                size_t base = (((size_t)bi * seq + t) * heads + h) * hd;
                const float *c = cos_t + (size_t)(offset + t) * half;
                const float *s = sin_t + (size_t)(offset + t) * half;
                for (int i = 0; i < half; ++i) {
                    float x1 = x[base + i], x2 = x[base + half + i];
                    float a = x1 * c[i], bb = x2 * s[i];
                    float cc = x1 * s[i], dd = x2 * c[i];
                    out[base + i] = a - bb;
                    out[base + half + i] = cc + dd;
                }
            }
}

/* ------------------------------------------------------------------------- */
/* SwiGLU  (crates/aarambh-studio-nn/src/ffn.rs:29-37; kernel formula          */
/* crates/aarambh-studio-kernel/kernels/swiglu_fused.cu:50-53)                 */
/* ------------------------------------------------------------------------- */
ORC_API void orc_swiglu(const float *gate, const float *up, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float g = gate[i];
        out[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

/* ------------------------------------------------------------------------- */
/* Attention: single-pass online softmax, one task per (b,h,q) row            */
/* (crates/aarambh-studio-kernel/src/cpu/parallel_attn.rs:97-234)              */
/* q [b,h,q_seq,hd], k,v [b,h,kv_seq,hd]; mask optional [1|b,1|h,q_seq,kv_seq] */
/* ------------------------------------------------------------------------- */
ORC_API void orc_attention(const float *q, const float *k, const float *v, const float *mask,
                           int mask_b, int mask_h, int causal, float scale, float *out, int b,
                           int h, int q_seq, int kv_seq, int hd, int parallel) {
    long rows = (long)b * h * q_seq;
#pragma omp parallel for schedule(static) if (parallel)
    for (long row = 0; row < rows; ++row) {
        int q_idx = (int)(row % q_seq);
        int head = (int)((row / q_seq) % h);
        int batch = (int)(row / ((long)h * q_seq));
        const float *qr = q + (((size_t)batch * h + head) * q_seq + q_idx) * hd;
        float *o = out + (size_t)row * hd;
        for (int d = 0; d < hd; ++d) o[d] = 0.0f;
        float running_max = -INFINITY, running_sum = 0.0f;
        for (int kv = 0; kv < kv_seq; ++kv) {
            float mask_value = 0.0f;
            if (mask) {
                int mb = mask_b == 1 ? 0 : batch, mh = mask_h == 1 ? 0 : head;
                mask_value = mask[(((size_t)mb * mask_h + mh) * q_seq + q_idx) * kv_seq + kv];
            }
            int shift = kv_seq > q_seq ? kv_seq - q_seq : 0;
            if ((causal && kv > shift + q_idx) || mask_value == -INFINITY) continue;
            const float *kr = k + (((size_t)batch * h + head) * kv_seq + kv) * hd;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot += qr[d] * kr[d];
            float score = dot * scale + mask_value;
            float next_max = rmaxf(running_max, score);
            float old_scale = expf(running_max - next_max);
            float new_scale = expf(score - next_max);
            const float *vr = v + (((size_t)batch * h + head) * kv_seq + kv) * hd;
            for (int d = 0; d < hd; ++d) o[d] = o[d] * old_scale + new_scale * vr[d];
            running_sum = running_sum * old_scale + new_scale;
            running_max = next_max;
        }
        if (running_sum > 0.0f) {
            float inv = 1.0f / running_sum;
            for (int d = 0; d < hd; ++d) o[d] *= inv;
        }
    }
}

/* Grouped-query decode attention over a cache held as [b, kv_len, kv_heads, hd]
 * (the KVCache storage layout, crates/aarambh-studio-nn/src/kvcache.rs:349-368):
 * equals repeat_heads (attention.rs:415-428: query head j uses kv head
 * j / (h/kvh)) + transpose + attention_forward_causal with q_seq = 1, without
 * materialising the repeated heads.  q,out [b,h,hd]; kv_lens[b] gives each
 * row's length (ragged batched decode, attention.rs:265-283); row stride in the
 * cache is `cap`. */
ORC_API void orc_attention_decode_gqa(const float *q, const float *kc, const float *vc,
                                      const int *kv_lens, int cap, float scale, float *out,
                                      int b, int h, int kvh, int hd) {
    int rep = h / kvh;
    long rows = (long)b * h;
#pragma omp parallel for schedule(dynamic, 1)
    for (long row = 0; row < rows; ++row) {
        int head = (int)(row % h), batch = (int)(row / h);
        int kvhead = head / rep;
        int kv_len = kv_lens[batch];
        const float *qr = q + (size_t)row * hd;
        float *o = out + (size_t)row * hd;
        for (int d = 0; d < hd; ++d) o[d] = 0.0f;
        float running_max = -INFINITY, running_sum = 0.0f;
        for (int kv = 0; kv < kv_len; ++kv) {
            size_t off = (((size_t)batch * cap + kv) * kvh + kvhead) * hd;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot += qr[d] * kc[off + d];
            float score = dot * scale + 0.0f;
            float next_max = rmaxf(running_max, score);
            float old_scale = expf(running_max - next_max);
            float new_scale = expf(score - next_max);
            for (int d = 0; d < hd; ++d) o[d] = o[d] * old_scale + new_scale * vc[off + d];
            running_sum = running_sum * old_scale + new_scale;
            running_max = next_max;
        }
        if (running_sum > 0.0f) {
            float inv = 1.0f / running_sum;
            for (int d = 0; d < hd; ++d) o[d] *= inv;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* KV quantisation                                                            */
/* ------------------------------------------------------------------------- */

/* Per-(token, kv-head) symmetric INT8 with the absmax.rs:7-24 arithmetic applied
 * to each head_dim vector: x [rows, hd] -> codes [rows, hd], scales [rows]. */
ORC_API void orc_quantise_kv_rows(const float *x, long rows, int hd, int8_t *codes,
                                  float *scales) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        scales[r] = orc_quantise_absmax_i8(x + (size_t)r * hd, (size_t)hd, codes + (size_t)r * hd);
}

/* ------------------------------------------------------------------------- */
/* argmax: last index among equal maxima under f32::total_cmp                 */
/* (crates/aarambh-studio-inference/src/sampler.rs:217-224)                    */
/* ------------------------------------------------------------------------- */
static inline int32_t total_key(float f) {
    int32_t b;
    memcpy(&b, &f, 4);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return b;
}
ORC_API int orc_argmax(const float *values, int n) {
    if (n <= 0) return 0;
    int best = 0;
    int32_t best_key = total_key(values[0]);
    for (int i = 1; i < n; ++i) {
        int32_t key = total_key(values[i]);
        if (key >= best_key) { best_key = key; best = i; }
    }
    return best;
}

/* ------------------------------------------------------------------------- */
/* Dense decoder model (the reference's CPU inference path after load-time    */
/* dequantisation, crates/aarambh-studio-weights/src/gguf.rs:80-88)            */
/* ------------------------------------------------------------------------- */

typedef struct {
    int n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_hidden, vocab, max_seq;
    float eps;
    double rope_theta;
    /* dense f32 weights, [out,in] row-major (qat.rs:315-348) */
    const float *embedding; /* [vocab, d_model] */
    const float *lm_head;   /* [vocab, d_model] (same pointer when tied) */
    const float *final_norm;
    const float **wq, **wk, **wv, **wo, **w_gate, **w_up, **w_down, **norm1, **norm2;
    float *cos_t, *sin_t;
    /* KV caches: [layer][b][cap][kvh][hd] (kvcache.rs:349-368) */
    int batch, cap;
    float **kc, **vc;
    int *lens; /* [batch] committed length per sequence */
    int norm_simd_order; /* 1: AVX2+FMA summation order (simd_norm.rs:246-284) */
    int linear_lanes;    /* 1: projections in 16-lane SIMD order (timed baseline only) */
} orc_model;

ORC_API orc_model *orc_model_create(int n_layers, int d_model, int n_heads, int n_kv_heads,
                                    int head_dim, int ffn_hidden, int vocab, int max_seq,
                                    float eps, double rope_theta, int batch, int cap) {
    orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
    m->n_layers = n_layers; m->d_model = d_model; m->n_heads = n_heads;
    m->n_kv_heads = n_kv_heads; m->head_dim = head_dim; m->ffn_hidden = ffn_hidden;
    m->vocab = vocab; m->max_seq = max_seq; m->eps = eps; m->rope_theta = rope_theta;
    m->batch = batch; m->cap = cap; m->norm_simd_order = 1; m->linear_lanes = 0;
    size_t L = (size_t)n_layers;
    m->wq = calloc(L, sizeof(float *)); m->wk = calloc(L, sizeof(float *));
    m->wv = calloc(L, sizeof(float *)); m->wo = calloc(L, sizeof(float *));
    m->w_gate = calloc(L, sizeof(float *)); m->w_up = calloc(L, sizeof(float *));
    m->w_down = calloc(L, sizeof(float *)); m->norm1 = calloc(L, sizeof(float *));
    m->norm2 = calloc(L, sizeof(float *));
    m->kc = calloc(L, sizeof(float *)); m->vc = calloc(L, sizeof(float *));
    size_t kv_elems = (size_t)batch * cap * n_kv_heads * head_dim;
    for (size_t l = 0; l < L; ++l) {
        m->kc[l] = calloc(kv_elems ? kv_elems : 1, sizeof(float));
        m->vc[l] = calloc(kv_elems ? kv_elems : 1, sizeof(float));
    }
    m->lens = calloc((size_t)(batch ? batch : 1), sizeof(int));
    m->cos_t = malloc(sizeof(float) * (size_t)max_seq * (head_dim / 2));
    m->sin_t = malloc(sizeof(float) * (size_t)max_seq * (head_dim / 2));
    orc_rope_tables(max_seq, head_dim, rope_theta, m->cos_t, m->sin_t);
    return m;
}

/* which: 0 wq 1 wk 2 wv 3 wo 4 gate 5 up 6 down 7 norm1 8 norm2 (per layer);
 * layer = -1: 0 embedding, 1 lm_head, 2 final_norm.  Pointers are borrowed. */
ORC_API void orc_model_set_weight(orc_model *m, int layer, int which, const float *ptr) {
    if (layer < 0) {
        if (which == 0) m->embedding = ptr;
        else if (which == 1) m->lm_head = ptr;
        else m->final_norm = ptr;
        return;
    }
    const float ***slots[9] = {&m->wq, &m->wk, &m->wv, &m->wo, &m->w_gate,
                               &m->w_up, &m->w_down, &m->norm1, &m->norm2};
    (*slots[which])[layer] = ptr;
}

ORC_API void orc_model_set_norm_order(orc_model *m, int simd_order) { m->norm_simd_order = simd_order; }
/* 0: strict k order per output (the parity definition); 1: 16-lane SIMD order (timed baseline only). */
ORC_API void orc_model_set_linear_order(orc_model *m, int lanes) { m->linear_lanes = lanes; }
static void model_linear(const orc_model *m, const float *x, const float *w, float *y, int M, int N, int K) {
    if (m->linear_lanes) orc_linear_f32_lanes(x, w, y, M, N, K);
    else orc_linear_f32(x, w, y, M, N, K);
}

ORC_API void orc_model_reset(orc_model *m) {
    for (int b = 0; b < m->batch; ++b) m->lens[b] = 0;
}
ORC_API int orc_model_seq_len(const orc_model *m, int b) { return m->lens[b]; }
/* KVCache::truncate (kvcache.rs:293-323): cannot grow. Returns 0 ok, -1 error. */
ORC_API int orc_model_truncate(orc_model *m, int b, int new_len) {
    if (new_len > m->lens[b] || new_len < 0) return -1;
    m->lens[b] = new_len;
    return 0;
}

/* Test/benchmark helper (no reference counterpart): fills the first `len`
 * positions of one sequence's caches in every layer with small pseudo-random
 * values and sets its length, so that decode steps at a given context can be
 * timed without running the prefill on the CPU. */
ORC_API void orc_model_fill_cache(orc_model *m, int row, int len, uint32_t seed) {
    size_t per_tok = (size_t)m->n_kv_heads * m->head_dim;
    for (int l = 0; l < m->n_layers; ++l) {
        uint32_t state = seed + 7919u * (uint32_t)l;
        float *k = m->kc[l] + (size_t)row * m->cap * per_tok, *v = m->vc[l] + (size_t)row * m->cap * per_tok;
        for (size_t i = 0; i < (size_t)len * per_tok; ++i) {
            state = state * 1664525u + 1013904223u;
            k[i] = ((float)(state >> 8) / 16777216.0f - 0.5f) * 2.0f;
            state = state * 1664525u + 1013904223u;
            v[i] = ((float)(state >> 8) / 16777216.0f - 0.5f) * 2.0f;
        }
    }
    m->lens[row] = len;
}

ORC_API void orc_model_destroy(orc_model *m) {
    if (!m) return;
    for (int l = 0; l < m->n_layers; ++l) { free(m->kc[l]); free(m->vc[l]); }
    free(m->wq); free(m->wk); free(m->wv); free(m->wo); free(m->w_gate); free(m->w_up);
    free(m->w_down); free(m->norm1); free(m->norm2); free(m->kc); free(m->vc);
    free(m->lens); free(m->cos_t); free(m->sin_t); free(m);
}

static void model_norm(const orc_model *m, const float *x, const float *w, float *out, int rows) {
    if (m->norm_simd_order) orc_rms_norm_avx2fma_order(x, w, m->eps, out, rows, m->d_model);
    else orc_rms_norm_scalar(x, w, m->eps, out, rows, m->d_model);
}

/* One forward over `S` new tokens for each of `B` rows.
 *  - prefill form (AarambhModel::forward_with_cache,
 *    crates/aarambh-studio-model/src/model.rs:508-587): B = 1 row `row0`, S tokens
 *    starting at offsets[0];
 *  - batched decode form (forward_decode_batch, model.rs:590-641): S = 1, rows
 *    row0..row0+B-1 with per-row offsets.
 * Block structure: crates/aarambh-studio-nn/src/block.rs:331-371; attention:
 * crates/aarambh-studio-nn/src/attention.rs:170-288; FFN: ffn.rs:29-37.
 * logits: [B, S, vocab].  Returns 0, or -1 on capacity overflow
 * (kvcache.rs:337-342) / offset >= max_seq (model.rs:609-615). */
ORC_API int orc_model_forward(orc_model *m, const uint32_t *ids, int B, int S, int row0,
                              const int *offsets, float *logits) {
    int d = m->d_model, h = m->n_heads, kvh = m->n_kv_heads, hd = m->head_dim;
    int ffn = m->ffn_hidden, V = m->vocab, rep = h / kvh;
    long T = (long)B * S;
    for (int b = 0; b < B; ++b) {
        if (offsets[b] + S > m->max_seq) return -1;
        if (m->lens[row0 + b] + S > m->cap) return -1;
    }
    float *x = malloc(sizeof(float) * T * d), *xn = malloc(sizeof(float) * T * d);
    float *qb = malloc(sizeof(float) * T * h * hd), *qr = malloc(sizeof(float) * T * h * hd);
    float *kb = malloc(sizeof(float) * T * kvh * hd), *kr = malloc(sizeof(float) * T * kvh * hd);
    float *vb = malloc(sizeof(float) * T * kvh * hd);
    float *att = malloc(sizeof(float) * T * h * hd), *proj = malloc(sizeof(float) * T * d);
    float *gate = malloc(sizeof(float) * T * ffn), *up = malloc(sizeof(float) * T * ffn);
    float *hid = malloc(sizeof(float) * T * ffn);
    float scale = (float)(1.0 / sqrt((double)hd));

    /* TokenEmbedding::forward (crates/aarambh-studio-model/src/embedding.rs:26-28) */
    for (long t = 0; t < T; ++t)
        memcpy(x + t * d, m->embedding + (size_t)ids[t] * d, sizeof(float) * d);

    for (int l = 0; l < m->n_layers; ++l) {
        model_norm(m, x, m->norm1[l], xn, (int)T);
        model_linear(m, xn, m->wq[l], qb, (int)T, h * hd, d);
        model_linear(m, xn, m->wk[l], kb, (int)T, kvh * hd, d);
        model_linear(m, xn, m->wv[l], vb, (int)T, kvh * hd, d);
        for (int b = 0; b < B; ++b) {
            int row = row0 + b, off = offsets[b], len0 = m->lens[row];
            orc_rope_apply(qb + (size_t)b * S * h * hd, qr + (size_t)b * S * h * hd, m->cos_t,
                           m->sin_t, 1, S, h, hd, off);
            orc_rope_apply(kb + (size_t)b * S * kvh * hd, kr + (size_t)b * S * kvh * hd,
                           m->cos_t, m->sin_t, 1, S, kvh, hd, off);
            /* KVCache::update slice_set at len (kvcache.rs:358-363) */
            size_t cbase = ((size_t)row * m->cap + len0) * kvh * hd;
            memcpy(m->kc[l] + cbase, kr + (size_t)b * S * kvh * hd, sizeof(float) * S * kvh * hd);
            memcpy(m->vc[l] + cbase, vb + (size_t)b * S * kvh * hd, sizeof(float) * S * kvh * hd);
            int kv_len = len0 + S;
            /* causal attention, cut at kv_len - q_len + q_idx (parallel_attn.rs:205-209) */
            long arows = (long)S * h;
#pragma omp parallel for schedule(static)
            for (long ar = 0; ar < arows; ++ar) {
                int qi = (int)(ar / h), head = (int)(ar % h), kvhead = head / rep;
                const float *qv = qr + (((size_t)b * S + qi) * h + head) * hd;
                float *o = att + (((size_t)b * S + qi) * h + head) * hd;
                for (int dd = 0; dd < hd; ++dd) o[dd] = 0.0f;
                float rmax = -INFINITY, rsum = 0.0f;
                int shift = kv_len > S ? kv_len - S : 0;
                for (int kv = 0; kv < kv_len; ++kv) {
                    if (kv > shift + qi) continue;
                    size_t coff = (((size_t)row * m->cap + kv) * kvh + kvhead) * hd;
                    float dot = 0.0f;
                    for (int dd = 0; dd < hd; ++dd) dot += qv[dd] * m->kc[l][coff + dd];
                    float score = dot * scale + 0.0f;
                    float nmax = rmaxf(rmax, score);
                    float os = expf(rmax - nmax), ns = expf(score - nmax);
                    for (int dd = 0; dd < hd; ++dd) o[dd] = o[dd] * os + ns * m->vc[l][coff + dd];
                    rsum = rsum * os + ns;
                    rmax = nmax;
                }
                if (rsum > 0.0f) {
                    float inv = 1.0f / rsum;
                    for (int dd = 0; dd < hd; ++dd) o[dd] *= inv;
                }
            }
        }
        model_linear(m, att, m->wo[l], proj, (int)T, d, h * hd);
        for (long i = 0; i < T * d; ++i) x[i] = x[i] + proj[i];
        model_norm(m, x, m->norm2[l], xn, (int)T);
        model_linear(m, xn, m->w_gate[l], gate, (int)T, ffn, d);
        model_linear(m, xn, m->w_up[l], up, (int)T, ffn, d);
        orc_swiglu(gate, up, hid, (size_t)T * ffn);
        model_linear(m, hid, m->w_down[l], proj, (int)T, d, ffn);
        for (long i = 0; i < T * d; ++i) x[i] = x[i] + proj[i];
    }
    for (int b = 0; b < B; ++b) m->lens[row0 + b] += S;
    model_norm(m, x, m->final_norm, xn, (int)T);
    model_linear(m, xn, m->lm_head, logits, (int)T, V, d);
    free(x); free(xn); free(qb); free(qr); free(kb); free(kr); free(vb); free(att);
    free(proj); free(gate); free(up); free(hid);
    return 0;
}
