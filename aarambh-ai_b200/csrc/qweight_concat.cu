// Row-wise concatenation of packed weights that share in_features and format:
// the fused QKV and gate|up projections of a decoder block are one packed
// weight, so one launch serves the three (two) reference linears
// (crates/aarambh-studio-nn/src/attention.rs:182-184, ffn.rs:30-31).
#include <cstring>

#include "common.cuh"
#include "w4a16_layout.cuh"

using namespace ab2;

AB2_API int ab2_qweight_concat_rows(ab2_qweight **out, const ab2_qweight *const *parts, int count) {
    AB2_REQUIRE(out && parts && count > 0, AB2_ERR_BAD_ARG, "null or empty argument");
    const ab2_qweight *first = parts[0];
    AB2_REQUIRE(first != nullptr, AB2_ERR_BAD_ARG, "null weight handle");
    long long N = 0;
    for (int i = 0; i < count; ++i) {
        const ab2_qweight *p = parts[i];
        AB2_REQUIRE(p != nullptr, AB2_ERR_BAD_ARG, "null weight handle");
        AB2_REQUIRE(p->fmt == first->fmt && p->K == first->K && p->group == first->group, AB2_ERR_BAD_SHAPE,
                    "parts must share format, in_features and group size");
        if (p->fmt == FMT_W4A16)
            AB2_REQUIRE(p->N % 16 == 0 || i == count - 1, AB2_ERR_BAD_SHAPE, "W4A16 parts need out_features that are multiples of 16, got %d", p->N);
        if (p->fmt == FMT_I4_AFFINE)
            AB2_REQUIRE(((long long)p->N * p->K) % p->group == 0 && ((long long)p->N * p->K) % 32 == 0 || i == count - 1,
                        AB2_ERR_BAD_SHAPE, "int4 parts must end on a group boundary");
        if (p->fmt == FMT_Q4KM)
            AB2_REQUIRE(((long long)p->N * p->K) % 256 == 0 || i == count - 1, AB2_ERR_BAD_SHAPE, "Q4 parts must end on a block boundary");
        N += p->N;
    }
    ab2_qweight *w = new ab2_qweight();
    memset(w, 0, sizeof(*w));
    w->fmt = first->fmt; w->N = (int)N; w->K = first->K; w->group = first->group; w->per_tensor = 0;
    cudaGetDevice(&w->device);
    const int K = first->K;
    cudaError_t e = cudaSuccess;
    auto copy_parts = [&](void **dst, size_t total, auto size_of, auto src_of) {
        if (e != cudaSuccess) return;
        e = cudaMalloc(dst, total ? (total + 15) / 16 * 16 : 16);
        size_t off = 0;
        for (int i = 0; i < count && e == cudaSuccess; ++i) {
            size_t n = size_of(parts[i]);
            e = cudaMemcpy((char *)*dst + off, src_of(parts[i]), n, cudaMemcpyDeviceToDevice);
            off += n;
        }
    };
    switch (first->fmt) {
    case FMT_I8:
        w->codes_bytes = (size_t)N * K; w->param_bytes = (size_t)N * 4;
        copy_parts(&w->codes, w->codes_bytes, [&](const ab2_qweight *p) { return (size_t)p->N * K; },
                   [](const ab2_qweight *p) { return (const void *)p->codes; });
        copy_parts((void **)&w->scales, (size_t)N * 4, [](const ab2_qweight *p) { return (size_t)p->N * 4; },
                   [](const ab2_qweight *p) { return (const void *)p->scales; });
        break;
    case FMT_I4_AFFINE: {
        size_t ng = ceil_div((size_t)N * K, (size_t)first->group);
        w->codes_bytes = ceil_div((size_t)N * K, 2); w->param_bytes = ng * 8;
        auto groups = [&](const ab2_qweight *p) { return ceil_div((size_t)p->N * K, (size_t)p->group) * 4; };
        copy_parts(&w->codes, w->codes_bytes, [&](const ab2_qweight *p) { return ceil_div((size_t)p->N * K, 2); },
                   [](const ab2_qweight *p) { return (const void *)p->codes; });
        copy_parts((void **)&w->scales, ng * 4, groups, [](const ab2_qweight *p) { return (const void *)p->scales; });
        copy_parts((void **)&w->zeros, ng * 4, groups, [](const ab2_qweight *p) { return (const void *)p->zeros; });
        break;
    }
    case FMT_Q4KM: {
        size_t nb = ceil_div((size_t)N * K, 256);
        w->codes_bytes = nb * 128; w->param_bytes = nb * 4;
        copy_parts(&w->codes, w->codes_bytes, [&](const ab2_qweight *p) { return ceil_div((size_t)p->N * K, 256) * 128; },
                   [](const ab2_qweight *p) { return (const void *)p->codes; });
        copy_parts((void **)&w->block_params, nb * 4, [&](const ab2_qweight *p) { return ceil_div((size_t)p->N * K, 256) * 4; },
                   [](const ab2_qweight *p) { return (const void *)p->block_params; });
        break;
    }
    case FMT_W4A16: {
        W4Layout L{(int)N, K, first->group};
        w->codes_bytes = (size_t)L.tiles() * 16 * K / 2;
        w->param_bytes = (size_t)L.tiles() * 16 * L.G() * 4;
        copy_parts(&w->codes, L.total_words() * 4,
                   [&](const ab2_qweight *p) { return W4Layout{p->N, K, p->group}.total_words() * 4; },
                   [](const ab2_qweight *p) { return (const void *)p->codes; });
        break;
    }
    default:
        delete w;
        return fail(AB2_ERR_BAD_ARG, "unknown weight format %d", first->fmt);
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        ab2_qweight_destroy(w);
        return fail(AB2_ERR_CUDA, "concatenation failed: %s", cudaGetErrorString(e));
    }
    *out = w;
    return AB2_OK;
}

// gate|up of a SwiGLU block as one W4A16 weight whose 16-row tiles hold 8 gate
// rows followed by the 8 matching up rows, so the GEMV epilogue can form
// silu(gate) * up without writing the two projections out
// (crates/aarambh-studio-nn/src/ffn.rs:29-37).
__global__ void w4a16_interleave8_kernel(const uint32_t *gate, const uint32_t *up, W4Layout src,
                                         W4Layout dst, uint32_t *out) {
    // one thread per destination word of the code and parameter planes
    const int wpr = dst.words_per_row(), G = dst.G();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t per_row = (size_t)G * (wpr + 1);
    if (i >= (size_t)dst.N * per_row) return;
    int n = (int)(i / per_row), rest = (int)(i % per_row);
    int g = rest / (wpr + 1), j = rest % (wpr + 1);
    int tile = n >> 4, r = n & 15;
    int src_row = tile * 8 + (r & 7);
    const uint32_t *from = (r < 8) ? gate : up;
    if (src_row >= src.N) return;  // padded rows stay zero
    if (j < wpr) out[dst.code_index(n, g * wpr + j)] = from[src.code_index(src_row, g * wpr + j)];
    else out[dst.param_index(n, g)] = from[src.param_index(src_row, g)];
}

AB2_API int ab2_qweight_interleave_gate_up(ab2_qweight **out, const ab2_qweight *gate, const ab2_qweight *up) {
    AB2_REQUIRE(out && gate && up, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(gate->fmt == FMT_W4A16 && up->fmt == FMT_W4A16, AB2_ERR_UNSUPPORTED, "interleaving is defined for W4A16 weights");
    AB2_REQUIRE(gate->N == up->N && gate->K == up->K && gate->group == up->group, AB2_ERR_BAD_SHAPE, "gate and up must have the same shape and group size");
    AB2_REQUIRE(gate->N % 8 == 0, AB2_ERR_BAD_SHAPE, "out_features must be a multiple of 8, got %d", gate->N);
    ab2_qweight *w = new ab2_qweight();
    memset(w, 0, sizeof(*w));
    w->fmt = FMT_W4A16; w->N = 2 * gate->N; w->K = gate->K; w->group = gate->group;
    cudaGetDevice(&w->device);
    W4Layout src{gate->N, gate->K, gate->group}, dst{w->N, w->K, w->group};
    w->codes_bytes = (size_t)dst.tiles() * 16 * w->K / 2;
    w->param_bytes = (size_t)dst.tiles() * 16 * dst.G() * 4;
    cudaError_t e = cudaMalloc(&w->codes, dst.total_words() * 4);
    if (e == cudaSuccess) e = cudaMemset(w->codes, 0, dst.total_words() * 4);
    if (e == cudaSuccess) {
        size_t n = (size_t)dst.N * dst.G() * (dst.words_per_row() + 1);
        w4a16_interleave8_kernel<<<(unsigned)ceil_div(n, 256), 256>>>((const uint32_t *)gate->codes, (const uint32_t *)up->codes, src, dst, (uint32_t *)w->codes);
        e = cudaDeviceSynchronize();
    }
    if (e != cudaSuccess) {
        ab2_qweight_destroy(w);
        return fail(AB2_ERR_CUDA, "interleaving failed: %s", cudaGetErrorString(e));
    }
    *out = w;
    return AB2_OK;
}
