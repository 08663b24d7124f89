// The one-token decode step as one persistent kernel (internal header; see
// decode_step_persistent.cu).
#pragma once

#include "common.cuh"
#include "kv_cache.cuh"

namespace ab2 {

// What the persistent step needs to know about a finalised decoder.  All
// pointers are borrowed from the model, which outlives the step object.
struct PsLayerDesc {
    const ab2_qweight *wqkv, *wo, *wgu, *wdown;  // wgu: gate|up interleaved in 8-row halves
    const float *norm1, *norm2;
};
struct PsModelDesc {
    int n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_hidden, vocab;
    float eps;
    const ab2_qweight *embedding, *lm_head;
    const float *final_norm;
    const PsLayerDesc *layers;
    void *x, *qkv, *attn, *hid;  // bf16 workspaces of one token
    const float *cos_t, *sin_t;
};

struct PersistentStep;

// AB2_OK with *out == nullptr when the model or the device cannot take this path
// (formats other than W4A16 g128, head_dim other than 128, no cooperative launch).
int persistent_step_create(PersistentStep **out, const PsModelDesc &desc);
void persistent_step_destroy(PersistentStep *ps);
// Whether one row of this cache, at most `len_bound` tokens long after the step, can be served.
bool persistent_step_serves(const PersistentStep *ps, const ab2_kv *kv, int len_bound);
// One decode step of cache row `row`: ids_dev[0] in, logits (bf16 [vocab], never null) and
// optionally the greedy token out; appends to the cache and advances the row's device length.
int persistent_step_launch(PersistentStep *ps, ab2_kv *kv, const uint32_t *ids_dev, int row, void *logits_dev,
                           uint32_t *argmax_dev, cudaStream_t s);

// Timestamps (ns, GPU wall clock) of the last step: [3 CTAs: first, middle, last][phase][10];
// entries 0..3 = phase start, prologue done, CTA done, barrier passed; 4..9 = points inside the
// phase (0 where a phase has none).
int persistent_step_trace(const PersistentStep *ps, unsigned long long *out, int capacity, int *nphases);

}  // namespace ab2
