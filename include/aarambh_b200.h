/*
 * aarambh_b200.h — C ABI of libaarambh_b200.so
 *
 * B200 (sm_100a) implementation of aarambh-studio's quantised decode path:
 * weight-only quantised linears and grouped-query attention over a (quantised)
 * KV cache.  Every entry point names the reference interface it stands in for
 * (paths relative to the reference project root).
 *
 * Conventions
 *  - Every function returns an ab2_status (0 = ok, negative = error) and never
 *    aborts; ab2_last_error() gives the thread-local message of the last
 *    failure on the calling thread.  The reference reports errors as
 *    Err(String) and its callers fall back (crates/aarambh-studio-kernel/src/
 *    dispatch.rs:57-72); this library has no fallback of its own.
 *  - Pointers named *_dev are device pointers on the current CUDA device;
 *    pointers named *_host are host pointers.  Pointers without a suffix in
 *    the *_from_* constructors may be either (copied with cudaMemcpyDefault).
 *  - `stream` is a cudaStream_t passed as void*.  Compute entry points are
 *    asynchronous on it; constructors synchronise.
 *  - One caller thread per device, as in the reference's serving worker
 *    (crates/aarambh-studio-serve/src/batching.rs:85-110).
 *  - Tensors are contiguous; weights are [out_features, in_features] row-major
 *    (crates/aarambh-studio-quant/src/qat.rs:315-348).
 */
#ifndef AARAMBH_B200_H
#define AARAMBH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    AB2_OK = 0,
    AB2_ERR_BAD_SHAPE = -1,
    AB2_ERR_BAD_ALIGN = -2,
    AB2_ERR_BAD_DTYPE = -3,
    AB2_ERR_CAPACITY = -4,
    AB2_ERR_CUDA = -5,
    AB2_ERR_TIMEOUT = -6,
    AB2_ERR_BAD_ARG = -7,
    AB2_ERR_UNSUPPORTED = -8
} ab2_status;

/* Activation / output element types (the reference's CUDA dtypes,
 * crates/aarambh-studio-kernel/src/flash_attn.rs:189-255). */
typedef enum { AB2_F32 = 0, AB2_F16 = 1, AB2_BF16 = 2 } ab2_dtype;

/* Storage type of a KV cache. */
typedef enum { AB2_KV_F32 = 0, AB2_KV_BF16 = 1, AB2_KV_INT8 = 2 } ab2_kv_dtype;

typedef void *ab2_stream;
typedef struct ab2_qweight ab2_qweight;
typedef struct ab2_kv ab2_kv;
typedef struct ab2_model ab2_model;
typedef struct ab2_tp ab2_tp;

/* ---- library ----------------------------------------------------------- */
int ab2_version(void);
const char *ab2_last_error(void);
/* Synchronises the current device and returns (then clears) its status word:
 * AB2_OK, or AB2_ERR_TIMEOUT when a kernel's bounded wait ran out.  No
 * counterpart in the reference, whose kernels never wait on one another. */
int ab2_device_status(int *status_host);

/* ---- quantised weights --------------------------------------------------
 * An ab2_qweight owns the packed bytes of one [N,K] weight in device memory.
 * The packed bytes stay on the GPU; the reference instead dequantises to dense
 * f32 at load (crates/aarambh-studio-weights/src/gguf.rs:152-163,195-241). */

/* I8QuantizedTensor, one scale per tensor
 * (crates/aarambh-studio-quant/src/absmax.rs:7-24, types.rs:66-75). */
int ab2_qweight_from_i8_tensor(ab2_qweight **out, const int8_t *codes, float scale, int N, int K);
/* One scale per output row (fake_quant_symmetric(…, OutputChannel),
 * crates/aarambh-studio-quant/src/qat.rs:140-156). */
int ab2_qweight_from_i8_channel(ab2_qweight **out, const int8_t *codes, const float *scales_N,
                                int N, int K);
/* PackedInt4Tensor: 2 nibbles per byte (low first), f32 scale and f32 zero per
 * group of `group` values of the flattened tensor
 * (crates/aarambh-studio-quant/src/types.rs:77-90, int4.rs:7-91). */
int ab2_qweight_from_i4_affine(ab2_qweight **out, const uint8_t *packed, const float *scales,
                               const float *zeros, int N, int K, int group);
/* Payload of encode_q4_k_m_tensor: ceil(N*K/256) blocks of 132 bytes
 * (crates/aarambh-studio-quant/src/gguf_quant.rs:1-49,
 *  crates/aarambh-studio-weights/src/gguf.rs:214-241). */
int ab2_qweight_from_q4km_blocks(ab2_qweight **out, const uint8_t *blocks132, int N, int K);
/* W4A16 group-wise layout: qweight [N, K/8] u32 with element k = 8*word + j in
 * bits 4j..4j+3, scales [N, K/group] bf16, qzeros [N, ceil(K/group/8)] u32 (zero
 * points 0..15, same nibble order along groups, rows padded to whole words).  Dequantisation is
 * (q - z) * s in f32 (crates/aarambh-studio-quant/src/int4.rs:88). */
int ab2_qweight_from_w4a16_gptq(ab2_qweight **out, const uint32_t *qweight,
                                const uint16_t *scales_bf16, const uint32_t *qzeros, int N, int K,
                                int group);
/* Same, with the interleaved nibble order: slot i of a word holds element
 * {0,2,4,6,1,3,5,7}[i] of its group of eight (weights and zero points). */
int ab2_qweight_from_w4a16_awq(ab2_qweight **out, const uint32_t *qweight,
                               const uint16_t *scales_bf16, const uint32_t *qzeros, int N, int K,
                               int group);

/* Device-side quantisers: read a dense f32 [N,K] weight in device memory and
 * build the packed weight with the reference arithmetic. */
/* quantise_absmax_i8 (absmax.rs:7-24); per_channel != 0 -> qat.rs:140-156. */
int ab2_qweight_quantise_i8(ab2_qweight **out, const float *w_dev, int N, int K, int per_channel,
                            ab2_stream stream);
/* quantise_affine_i4 (int4.rs:7-43); requires K % group == 0. */
int ab2_qweight_quantise_i4_affine(ab2_qweight **out, const float *w_dev, int N, int K, int group,
                                   ab2_stream stream);
/* encode_q4_k_m_tensor (gguf.rs:214-224), zero-padded tail block. */
int ab2_qweight_quantise_q4km(ab2_qweight **out, const float *w_dev, int N, int K,
                              ab2_stream stream);
/* int4.rs:7-43 evaluated with storable parameters: s = bf16((max-min)/15),
 * z = clamp(round(-min/s), 0, 15), q = clamp(round(v/s + z), 0, 15). */
int ab2_qweight_quantise_w4a16(ab2_qweight **out, const float *w_dev, int N, int K, int group,
                               ab2_stream stream);

int ab2_qweight_destroy(ab2_qweight *w);
int ab2_qweight_shape(const ab2_qweight *w, int *N, int *K, int *group, int *format);
/* Bytes of packed storage held on the device (codes + parameters). */
int ab2_qweight_nbytes(const ab2_qweight *w, size_t *nbytes);
/* Copies the packed code bytes / parameters back (host or device dst) in the
 * layout of the corresponding *_from_* constructor; NULL pointers are skipped. */
int ab2_qweight_export(const ab2_qweight *w, void *codes, void *scales, void *zeros);

/* dequantise_i8 / dequantise_i4 / decode_q4_k_m_tensor
 * (crates/aarambh-studio-quant/src/dequant.rs:8-22, gguf.rs:226-241):
 * writes the dense [N,K] weight as `dtype` (f32 is bit-exact with the
 * reference arithmetic; f16/bf16 are that value rounded to nearest even). */
int ab2_qweight_dequant(const ab2_qweight *w, void *out_dev, ab2_dtype dtype, ab2_stream stream);

/* QatLinear::forward without bias (crates/aarambh-studio-quant/src/qat.rs:315-348):
 * y[M,N] = x[M,K] . W^T with the dequantisation fused into the contraction.
 * x and y have element type `dtype`; accumulation is f32. */
int ab2_qlinear_forward(const ab2_qweight *w, const void *x_dev, int M, ab2_dtype dtype,
                        void *y_dev, ab2_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* AARAMBH_B200_H */
