// KV cache handle and the device-side view kernels receive (internal header).
#pragma once

#include "common.cuh"

#define AB2_KV_MAX_SPLITS 64

struct ab2_kv {
    int L, B, cap, kvh, hd, h;
    int dtype;        // ab2_kv_dtype
    void *k, *v;      // [L][B][kvh][cap][hd]
    float *ks, *vs;   // INT8 only: [L][B][kvh][cap]
    int *lens_dev;    // [B] committed length of each sequence
    int *lens_host;   // pinned host mirror (authoritative for host-side checks)
    // scratch of the split-context decode attention
    float *part_acc;  // [B][h][max_splits][hd]
    float *part_ml;   // [B][h][max_splits][2]  (running max, running sum)
    int max_splits;
    int *counters;    // [B][kvh] split-arrival counters of the fused decode attention (zero at rest)
    // Row selection: while `rows_on` is set, row index i of a call addresses cache row rows[i]
    // (an arbitrary set of live sequences served in one pass); otherwise rows are row0 + i.
    int *rows_dev;    // [B]
    int *rows_host;   // [B], pinned
    bool rows_on;
};

namespace ab2 {

struct KvView {
    int B, cap, kvh, hd, dtype;
    void *k, *v;
    float *ks, *vs;
    int *lens;
    const int *rows;  // selected cache rows of this call, or null (rows are row0 + i)
};

// Cache row addressed by index i of a call that starts at row0.
__device__ __forceinline__ int kv_row(const KvView &kv, int row0, int i) {
    return kv.rows ? kv.rows[row0 + i] : row0 + i;
}
static inline int kv_row_host(const ab2_kv *kv, int row0, int i) {
    return kv->rows_on ? kv->rows_host[row0 + i] : row0 + i;
}

KvView kv_view(const ab2_kv *kv, int layer);

// Writes S tokens per row at the rows' current lengths (no advance).  k / v
// element (row, s, head, d) sits at (row * S + s) * in_stride + head * hd + d.
// With `q_rot` (rows of the same stride, `q_heads` heads of hd) the same launch
// rotates the query heads in place.
int kv_append_device(ab2_kv *kv, int layer, const void *k, const void *v, long long in_stride, int S,
                     int row0, int nrows, ab2_dtype dtype, const float *cos_t, const float *sin_t,
                     const int *rope_pos, cudaStream_t s, void *q_rot = nullptr, int q_heads = 0);
int kv_commit_device(ab2_kv *kv, int S, int row0, int nrows, cudaStream_t s);

// Attention of S new queries per row over the cache.  `pending` is the number of
// appended but not yet committed tokens per row (S during a model step, 0 after
// a commit): query qi of a row sees cache positions [0, len + pending - S + qi].
// `len_hint` bounds the context length used to choose the number of splits
// (pass the capacity when the launch is captured in a graph).
// q / out element (row, qi, head, d) sits at row*stride_b + qi*stride_s + head*stride_h + d.
struct AttnStrides {
    long long q_b, q_s, q_h, o_b, o_s, o_h;
};
int attention_cached_device(const ab2_kv *kv, int layer, const void *q, void *out, int S, int pending,
                            int row0, int nrows, float scale, ab2_dtype dtype, AttnStrides st,
                            int len_hint, cudaStream_t s);

// Tensor-core INT8 flash-decode (head_dim 128): query head (row, head) sits at
// row * q_stride + head * 128, out is [nrows][h][128]; `pending` appended but
// uncommitted tokens per row are attended too; partials go to the given split
// scratch, merged by the caller when nsplit > 1.
int attention_decode_mma_device(const ab2_kv *kv, int layer, const void *q, void *out, int row0, int nrows,
                                float scale, ab2_dtype dtype, int nsplit, float *part_acc, float *part_ml,
                                int pending, long long q_stride, cudaStream_t s);
// Causal attention of S > 1 new queries per row over an INT8 cache (head_dim 128, up to 4 query
// heads per KV head) on the tensor cores; AB2_ERR_UNSUPPORTED for other layouts.
int attention_prefill_mma_device(const ab2_kv *kv, int layer, const void *q, void *out, int S, int pending, int row0,
                                 int nrows, float scale, ab2_dtype dtype, AttnStrides st, cudaStream_t s);
int attention_decode_fused_device(ab2_kv *kv, int layer, const void *qkv, long long stride, void *out,
                                  int row0, int nrows, float scale, ab2_dtype dtype, const float *cos_t,
                                  const float *sin_t, const int *rope_pos, int len_hint, cudaStream_t s);
// The same step for an INT8 cache with head_dim 128 and bf16 activations, one
// thread-block cluster per (row, kv head); `max_len` bounds the context length.
bool attention_decode_cluster_eligible(const ab2_kv *kv, ab2_dtype dtype, int max_len);
int attention_decode_cluster_device(ab2_kv *kv, int layer, const void *qkv, long long stride, void *out,
                                    int row0, int nrows, float scale, const float *cos_t, const float *sin_t,
                                    const int *rope_pos, int max_len, cudaStream_t s);

}  // namespace ab2
