// Device functions and launchers shared by ops.cu, the KV cache and the decoder.
#pragma once

#include "common.cuh"

namespace ab2 {

// Half-split rotation of one pair (d, d + hd/2): x1*c - x2*s, x1*s + x2*c with
// separately rounded products (crates/aarambh-studio-nn/src/rope.rs:118-124).
__device__ __forceinline__ void rope_rotate(float x1, float x2, float c, float s, float &o1,
                                            float &o2) {
    o1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
    o2 = __fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c));
}

// silu(g) * up with silu(g) = g / (1 + exp(-g))
// (crates/aarambh-studio-kernel/kernels/swiglu_fused.cu:50-53).
__device__ __forceinline__ float swiglu_value(float g, float up) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), up);
}

int launch_rms_norm(const void *x, const float *w, void *out, int rows, int d, float eps,
                    ab2_dtype dtype, cudaStream_t s);
int launch_swiglu_fused(const void *gu, void *out, int tokens, int ffn, ab2_dtype dtype,
                        cudaStream_t s);
int launch_add(const void *a, const void *b, void *out, size_t n, ab2_dtype dtype, cudaStream_t s);
int launch_add_rms_norm(void *x, const void *p, const float *w, void *out, int rows, int d, float eps,
                        ab2_dtype dtype, cudaStream_t s);
int launch_argmax(const void *logits, int rows, int vocab, ab2_dtype dtype, uint32_t *out,
                  cudaStream_t s);
int launch_embedding(const ab2_qweight *table, const uint32_t *ids, int tokens, void *out,
                     ab2_dtype dtype, cudaStream_t s);

}  // namespace ab2
