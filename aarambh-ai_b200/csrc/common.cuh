// Shared declarations for the library's translation units (internal header).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdlib>
#include <cstdio>
#include <string>

#include "aarambh_b200.h"

#define AB2_API extern "C" __attribute__((visibility("default")))

namespace ab2 {

// Records `msg` as the calling thread's last error and returns `code`.
int fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

#define AB2_CUDA(expr)                                                                      \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            return ab2::fail(AB2_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                  \
                             cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define AB2_LAUNCH_CHECK()                                                                  \
    do {                                                                                    \
        cudaError_t _e = cudaGetLastError();                                                \
        if (_e != cudaSuccess)                                                              \
            return ab2::fail(AB2_ERR_CUDA, "kernel launch failed: %s (%s:%d)",              \
                             cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define AB2_REQUIRE(cond, code, ...)                                                        \
    do {                                                                                    \
        if (!(cond)) return ab2::fail((code), __VA_ARGS__);                                 \
    } while (0)

enum Format : int {
    FMT_I8 = 0,         // int8 codes [N][K], f32 scale per row
    FMT_I4_AFFINE = 1,  // nibbles [N*K/2], f32 scale + f32 zero per flat group
    FMT_Q4KM = 2,       // nibbles [ceil(N*K/256)*128], (f16 scale, f16 min) per 256-block
    FMT_W4A16 = 3       // tile-major blocks of code and parameter words (w4a16_layout.cuh)
};

}  // namespace ab2

struct ab2_qweight {
    int fmt;
    int N, K, group;
    int per_tensor;        // FMT_I8: scales replicated from one tensor-wide scale
    int device;
    void *codes;           // packed codes, kernel-native layout
    float *scales;         // FMT_I8: [N]; FMT_I4_AFFINE: [ngroups]
    float *zeros;          // FMT_I4_AFFINE: [ngroups]
    uint32_t *block_params;  // FMT_Q4KM: lo16 = f16 scale, hi16 = f16 min, per block
    size_t codes_bytes, param_bytes;
};

namespace ab2 {

static inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

template <typename T> struct ActType;
template <> struct ActType<float> { static constexpr ab2_dtype value = AB2_F32; };
template <> struct ActType<__half> { static constexpr ab2_dtype value = AB2_F16; };
template <> struct ActType<__nv_bfloat16> { static constexpr ab2_dtype value = AB2_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(((uint32_t)b) << 16);
}
__device__ __forceinline__ float f16_bits_to_f32(uint16_t b) {
    return __half2float(__ushort_as_half(b));
}

static inline size_t dtype_size(ab2_dtype d) { return d == AB2_F32 ? 4 : 2; }

// ---- programmatic dependent launch ------------------------------------------
// Kernels of the decoder step are launched so that a kernel may start while its
// predecessor is still draining: everything that does not depend on the
// predecessor (barrier set-up, the first bulk copies of the constant weights)
// runs ahead of pdl_wait(), which returns once the predecessor grid has
// completed and its writes are visible.  Every kernel of the chain calls
// pdl_wait() before it finishes, so completion stays transitive.  Without the
// launch attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

// Set by the decoder step around its launches.
extern thread_local bool g_pdl_launch;

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t s, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool force = getenv("AB2_FORCE_PDL") != nullptr;  // experiments: chain every launch
    cfg.numAttrs = (g_pdl_launch || force) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace ab2
