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

/* One packed weight holding the rows of `count` weights that share format,
 * in_features and group size (Q|K|V and gate|up of a block, so that the three
 * / two reference linears of crates/aarambh-studio-nn/src/attention.rs:182-184
 * and ffn.rs:30-31 are one launch).  The parts stay valid and separate. */
int ab2_qweight_concat_rows(ab2_qweight **out, const ab2_qweight *const *parts, int count);
/* gate|up of SwiGluFfn (crates/aarambh-studio-nn/src/ffn.rs:29-37) as one W4A16
 * weight of 2 * ffn rows whose every 16 rows are 8 gate rows followed by the 8
 * matching up rows: the layout the decoder's fused projection + SwiGLU uses. */
int ab2_qweight_interleave_gate_up(ab2_qweight **out, const ab2_qweight *gate, const ab2_qweight *up);
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

/* ---- element-wise operators of the decoder block ------------------------- */

/* dispatch::rms_norm / RMSNorm::forward (crates/aarambh-studio-kernel/src/
 * dispatch.rs:57-72, cpu/simd_norm.rs:51-57, kernels/rms_norm_fused.cu:56-84):
 * out = x * (1 / sqrt(mean(x^2) + eps)) * weight over rows of length d.
 * The weight is f32; x and out have element type `dtype`. */
int ab2_rms_norm(const void *x_dev, const float *weight_dev, void *out_dev, int rows, int d, float eps,
                 ab2_dtype dtype, ab2_stream stream);
/* fused_rope_apply / RopeCache::apply_rotate (crates/aarambh-studio-kernel/src/
 * fused_rope.rs:139-196, crates/aarambh-studio-nn/src/rope.rs:107-126):
 * x [batch, seq, heads, head_dim]; half-split pairs (d, d + head_dim/2); token t
 * uses table row offset + t.  Tables are f32 [max_seq, head_dim/2] whatever `dtype` is: the
 * reference casts its tables to the model dtype (rope.rs:62-63), so with bf16 or f16 activations
 * this rotation is slightly more exact than the reference's (the products use unrounded cos / sin);
 * with f32 activations the two are bit-identical. */
int ab2_rope_apply(const void *x_dev, void *out_dev, const float *cos_dev, const float *sin_dev,
                   int batch, int seq, int heads, int head_dim, int offset, int max_seq,
                   ab2_dtype dtype, ab2_stream stream);
/* fused_swiglu (crates/aarambh-studio-kernel/src/fused_ffn.rs:9-21,
 * kernels/swiglu_fused.cu:43-54): out = gate / (1 + exp(-gate)) * up. */
int ab2_swiglu(const void *gate_dev, const void *up_dev, void *out_dev, size_t n, ab2_dtype dtype,
               ab2_stream stream);
/* Greedy argmax of Sampler (crates/aarambh-studio-inference/src/sampler.rs:217-224)
 * on the device: per row of logits [rows, vocab], the LAST index among equal
 * maxima under the f32 total order.  Writes rows u32 indices. */
int ab2_argmax(const void *logits_dev, int rows, int vocab, ab2_dtype dtype, uint32_t *out_dev,
               ab2_stream stream);
/* TokenEmbedding::forward (crates/aarambh-studio-model/src/embedding.rs:26-28) on a
 * packed table (GGUF export quantises the embedding too, crates/
 * aarambh-studio-weights/src/gguf.rs:133-150): out[t, :] = dequant(table[ids[t], :]). */
int ab2_embedding_forward(const ab2_qweight *table, const uint32_t *ids_dev, int tokens, void *out_dev,
                          ab2_dtype dtype, ab2_stream stream);

/* ---- KV cache --------------------------------------------------------------
 * KVCache with preallocated storage (crates/aarambh-studio-nn/src/kvcache.rs:
 * 236-369) for `batch` independent sequences; INT8 storage quantises every
 * (token, kv head) vector with the absmax arithmetic of
 * crates/aarambh-studio-quant/src/absmax.rs:7-24 and f32 scales.  The reference's
 * QuantisedKvCache (crates/aarambh-studio-quant/src/kv_quant.rs:16-74) uses one
 * scale per tensor and re-quantises the whole cache on every append; this cache
 * quantises each vector once.  n_heads is the number of query heads that will
 * attend to it (sizes the split-context scratch). */
int ab2_kv_create(ab2_kv **out, int n_layers, int batch, int capacity, int kv_heads, int head_dim,
                  int n_heads, ab2_kv_dtype dtype);
int ab2_kv_destroy(ab2_kv *kv);
/* KVCache::update (kvcache.rs:335-368) for a single-layer cache: k, v
 * [nrows, S, kv_heads, head_dim] of element type `dtype` are appended to rows
 * row0..row0+nrows-1 at their current lengths, which then grow by S.
 * AB2_ERR_CAPACITY when a row would exceed its capacity. */
int ab2_kv_update(ab2_kv *kv, const void *k_dev, const void *v_dev, int S, int row0, int nrows,
                  ab2_dtype dtype, ab2_stream stream);
/* The two halves of update for the multi-layer cache the engine holds
 * (KvCache, crates/aarambh-studio-inference/src/kvcache.rs:7-80: one length shared
 * by all layers): ab2_kv_append writes layer `layer`'s S new tokens per row at
 * the rows' current lengths without advancing them, optionally rotating K first
 * (rope.apply_inference before update, crates/aarambh-studio-nn/src/attention.rs:
 * 190-196,269-270; token s of a row uses table row positions_dev[row] + s, or its
 * cache position when positions_dev is NULL; pass NULL tables for no rotation);
 * ab2_kv_commit advances the rows' lengths by S once every layer has appended. */
int ab2_kv_append(ab2_kv *kv, int layer, const void *k_dev, const void *v_dev, int S, int row0,
                  int nrows, ab2_dtype dtype, const float *cos_dev, const float *sin_dev,
                  const int *positions_dev, int max_seq, ab2_stream stream);
int ab2_kv_commit(ab2_kv *kv, int S, int row0, int nrows, ab2_stream stream);
/* KVCache::truncate (kvcache.rs:293-323): cannot grow (AB2_ERR_CAPACITY). */
int ab2_kv_truncate(ab2_kv *kv, int row, int new_len, ab2_stream stream);
/* KVCache::clear (kvcache.rs:284-290). */
int ab2_kv_clear(ab2_kv *kv, ab2_stream stream);
/* KVCache::seq_len / capacity (kvcache.rs:326-333). */
int ab2_kv_seq_len(const ab2_kv *kv, int row, int *len);
int ab2_kv_capacity(const ab2_kv *kv, int *capacity);
/* KvCache::snapshot (crates/aarambh-studio-inference/src/kvcache.rs:57-64). */
int ab2_kv_clone(ab2_kv **out, const ab2_kv *src, ab2_stream stream);
/* The cached tensors KVCache::update returns, for one row, dequantised to f32
 * in the reference layout [len, kv_heads, head_dim], for layer `layer`. */
int ab2_kv_read(const ab2_kv *kv, int layer, int row, float *k_out_dev, float *v_out_dev,
                ab2_stream stream);

/* ---- attention --------------------------------------------------------------
 * GroupedQueryAttention::forward_decode_batch attention step
 * (crates/aarambh-studio-nn/src/attention.rs:265-283 -> dispatch::
 * attention_forward_causal, crates/aarambh-studio-kernel/src/dispatch.rs:145-160):
 * q, out [nrows, n_heads, head_dim]; one query per row over that row's cache
 * (ragged lengths), query head j uses kv head j / (n_heads / kv_heads). */
int ab2_attention_decode(const ab2_kv *kv, int layer, const void *q_dev, void *out_dev, int row0,
                         int nrows, float scale, ab2_dtype dtype, ab2_stream stream);
/* Same operation and result as ab2_attention_decode for callers that cannot
 * allocate device memory (a serving loop whose memory pool owns all free HBM,
 * a caller inside a lock the allocator needs, a fixed memory budget).  It has
 * no counterpart in the reference.  It calls no cudaMalloc / cudaFree: the
 * partial results of the context splits go to one fixed 8 MiB array inside the
 * library, which every GPU that loads the library holds until the process
 * exits.  Limit: (row0 + nrows) * n_heads * splits * (head_dim + 2) floats must
 * fit in 2 Mi floats, otherwise AB2_ERR_CAPACITY (the message names the sizes).
 * The first call on a device looks up the array's device address; make that
 * first call before any stream capture.  All calls share the array: nothing in
 * it needs clearing between calls (every slot a call reads it has written
 * first), but two calls that overlap on the GPU (different streams) race. */
int ab2_attention_decode_static(const ab2_kv *kv, int layer, const void *q_dev, void *out_dev, int row0,
                                int nrows, float scale, ab2_dtype dtype, ab2_stream stream);
/* GroupedQueryAttention::forward attention step (attention.rs:170-226) for S new
 * tokens per row that are already in the cache: q, out [nrows, S, n_heads,
 * head_dim]; causal cut at len - S + query index
 * (crates/aarambh-studio-kernel/src/cpu/parallel_attn.rs:205-209). */
int ab2_attention_cached(const ab2_kv *kv, int layer, const void *q_dev, void *out_dev, int S, int row0,
                         int nrows, float scale, ab2_dtype dtype, ab2_stream stream);
/* dispatch::attention_forward_causal on explicit tensors (dispatch.rs:145-160):
 * q, out [b, h, q_len, head_dim]; k, v [b, kv_heads, kv_len, head_dim] (the
 * kv heads are NOT repeated).  Synchronises the stream. */
int ab2_attention_causal(const void *q_dev, const void *k_dev, const void *v_dev, void *out_dev, int b,
                         int h, int kv_heads, int q_len, int kv_len, int head_dim, float scale,
                         ab2_dtype dtype, ab2_stream stream);

/* ---- decoder -----------------------------------------------------------------
 * The dense grouped-query decoder of AarambhModel (crates/aarambh-studio-model/
 * src/model.rs) over packed weights.  Field names follow ModelConfig
 * (crates/aarambh-studio-core/src/config.rs:734-868). */
typedef struct {
    int n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_hidden, vocab, max_seq;
    float rms_eps;      /* RMSNorm epsilon (1e-5) */
    double rope_theta;  /* RoPE base (10000) */
    int tied;           /* tied embeddings: lm_head shares the embedding weight */
} ab2_model_config;

/* `dtype` is the activation type of the whole model (the reference's model
 * dtype); `max_tokens` bounds rows * S of one forward call (workspace size). */
int ab2_model_create(ab2_model **out, const ab2_model_config *cfg, ab2_dtype dtype, int max_tokens);
int ab2_model_destroy(ab2_model *m);
/* Borrows a packed weight.  layer >= 0: which = 0 wq, 1 wk, 2 wv, 3 wo, 4 w_gate,
 * 5 w_up, 6 w_down; layer < 0: which = 0 embedding, 1 lm_head. */
int ab2_model_set_linear(ab2_model *m, int layer, int which, const ab2_qweight *w);
/* Copies an f32 RMSNorm weight of d_model values (host or device).  layer >= 0:
 * which = 0 norm1, 1 norm2; layer < 0: the final norm. */
int ab2_model_set_norm(ab2_model *m, int layer, int which, const float *weight);
/* Checks that every tensor is set, builds the fused projections, the RoPE
 * tables (RopeCache::new, crates/aarambh-studio-nn/src/rope.rs:33-72) and the
 * workspace. */
int ab2_model_finalize(ab2_model *m);
int ab2_model_rope_tables(const ab2_model *m, const float **cos_dev, const float **sin_dev);

/* ---- tensor parallelism ------------------------------------------------------
 * Megatron-style sharding of the decoder over the GPUs of one box, one process
 * per GPU.  The reference is data-parallel only; what is kept from it is the
 * bootstrap convention of its NCCL path (a 128-byte unique id made by rank 0
 * and handed to every rank, crates/aarambh-studio-train/src/distributed.rs:
 * 526-591) and the sum all-reduce (distributed.rs:494-503).
 * A rank's model is created with its LOCAL head counts and FFN width
 * (n_heads / world, n_kv_heads / world, ffn_hidden / world; d_model and vocab
 * whole): wq/wk/wv/w_gate/w_up hold the rank's rows (column parallel), wo and
 * w_down the rank's input columns (row parallel; the split falls on group
 * boundaries), lm_head the rank's vocab / world rows, the embedding is whole.
 * After wo and w_down the partial sums are all-reduced; the logits shards are
 * all-gathered.  ab2_model_set_tp must precede the lm_head and ab2_model_finalize. */
int ab2_tp_unique_id(void *id128_host);
/* id128_host may be NULL for world > 1: the context then has no NCCL communicator and serves
 * the peer exchange only (ab2_tp_all_reduce and a vocabulary-parallel head need the communicator). */
int ab2_tp_create(ab2_tp **out, int rank, int world, const void *id128_host);
int ab2_tp_destroy(ab2_tp *tp);
/* In-place sum over ranks of `count` elements (NCCL all-reduce). */
int ab2_tp_all_reduce(ab2_tp *tp, void *buf_dev, size_t count, ab2_dtype dtype, ab2_stream stream);
/* One-shot exchange of f32 partial sums over NVLink peer memory instead of NCCL (no counterpart
 * in the reference, whose only collective is the NCCL all-reduce above).  Every rank owns an
 * inbox; a partial sum travels as ONE 8-byte word {f32 sum, u32 exchange number} stored straight
 * into every rank's inbox, and a reader that finds the exchange number it waits for has the sum
 * that came with it: no flag, no fence, no signal round trip.  Inboxes are double-buffered by the
 * parity of a per-rank exchange count kept in device memory.
 *
 * Set-up: every rank calls ab2_tp_peer_export (allocates its inbox for up to max_elems sums per
 * rank, a multiple of 8, and writes a 64-byte CUDA IPC handle to handle64_host, which may be
 * NULL), the caller gathers the handles of all ranks in rank order (world x 64 bytes, the same
 * channel that carried the unique id), and every rank calls ab2_tp_peer_attach with them.  A
 * single process that drives several GPUs (or a test that plays a peer itself) instead reads
 * each context's block with ab2_tp_peer_block and calls ab2_tp_peer_attach_ptrs with the
 * device pointers of all ranks' blocks as seen from this rank (peer access enabled by the
 * caller); such contexts may be created with a NULL unique id (no NCCL communicator).
 *
 * Use: a decoder whose step has at most 16 tokens and tokens x d_model <= max_elems lets its
 * row-parallel projections store their sums into every rank's inbox and consumes them in the
 * next projection's prologue.  The same exchange is callable directly: ab2_tp_peer_deposit
 * stores this rank's `count` partial sums with every rank, ab2_tp_peer_reduce_add adds the sum
 * over ranks (in rank order, rounded to bf16 once) to x_bf16_dev; every rank must call the pair
 * the same number of times with the same count.
 *
 * A reader waits at most the wait limit (default two seconds, ab2_tp_set_wait_limit_ns) for a
 * peer's words; when it runs out the kernel records AB2_ERR_TIMEOUT in the device status word
 * and returns, leaving the exchange count as it was.  Callers that can lose a peer should read
 * ab2_device_status every few steps; after a time-out the ranks' counts may differ, and every
 * rank calls ab2_tp_peer_reset (between two host-side barriers of the caller's) to clear its
 * inbox and count before the exchange is used again.  The ranks must be on GPUs of one box with
 * peer access; attach before the first step is captured in a graph. */
int ab2_tp_peer_export(ab2_tp *tp, size_t max_elems, void *handle64_host);
int ab2_tp_peer_attach(ab2_tp *tp, const void *handles_host);
int ab2_tp_peer_block(ab2_tp *tp, void **block_dev, size_t *bytes);
int ab2_tp_peer_attach_ptrs(ab2_tp *tp, void *const *blocks_dev);
int ab2_tp_set_wait_limit_ns(ab2_tp *tp, unsigned long long limit_ns);
int ab2_tp_peer_reset(ab2_tp *tp);
int ab2_tp_peer_deposit(ab2_tp *tp, const float *partial_dev, size_t count, ab2_stream stream);
int ab2_tp_peer_reduce_add(ab2_tp *tp, void *x_bf16_dev, size_t count, ab2_stream stream);
int ab2_model_set_tp(ab2_model *m, ab2_tp *tp);
/* AarambhModel::forward_with_cache (model.rs:508-587; nrows = 1, S = prompt
 * length) and forward_decode_batch (model.rs:590-641; S = 1): ids_dev
 * [nrows, S] u32, rows row0..row0+nrows-1 of the cache.  offsets_host [nrows]
 * are the seqlen offsets (RoPE positions); NULL uses the cache lengths.
 * logits_mode 0: none; 1: last token of each row -> logits_dev [nrows, vocab];
 * 2: every token -> [nrows, S, vocab] (element type = model dtype).
 * argmax_dev (optional) receives the greedy token of each row's last position.
 * Errors: AB2_ERR_BAD_SHAPE when offset + S exceeds max_seq (model.rs:609-615),
 * AB2_ERR_CAPACITY when a cache row would overflow (kvcache.rs:337-342). */
int ab2_model_forward(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, int S, int row0, int nrows,
                      const int *offsets_host, int logits_mode, void *logits_dev, uint32_t *argmax_dev,
                      ab2_stream stream);
/* One decode step (S = 1, positions = cache lengths) replayed from a CUDA graph
 * captured on first use for this (cache, ids buffer, rows, outputs)
 * combination: InferenceEngine::decode_sessions
 * (crates/aarambh-studio-inference/src/engine.rs:323-355) without the per-token
 * host work.  ids_dev is read when the graph runs, so the previous step's
 * argmax_dev may be passed as the next ids_dev. */
int ab2_model_decode_step(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, int row0, int nrows,
                          void *logits_dev, uint32_t *argmax_dev, ab2_stream stream);
/* The same step for a caller that keeps its tokens in HOST memory, as the reference's serving
 * loop does (InferenceEngine::decode_sessions takes and returns host tokens,
 * crates/aarambh-studio-inference/src/engine.rs:323-355): copies ids_host [nrows] to the device,
 * replays the step, copies the greedy token of each row to argmax_host [nrows] and waits for the
 * stream.  With pinned host buffers both copies are asynchronous and the call waits once. */
int ab2_model_decode_step_host(ab2_model *m, ab2_kv *kv, const uint32_t *ids_host, int row0, int nrows,
                               uint32_t *argmax_host, ab2_stream stream);
/* The same two calls over an arbitrary set of cache rows: row i of ids / logits / argmax belongs
 * to cache row rows_host[i] (distinct rows, any order), positions are the rows' cache lengths.
 * This is what the serving batcher does each tick - every live session advances in ONE
 * forward whatever rows they occupy (decode_sessions over `session_indices`,
 * crates/aarambh-studio-serve/src/batching.rs:439-452; InferenceEngine::decode_sessions,
 * crates/aarambh-studio-inference/src/engine.rs:323-355).  The decode step keeps one graph per
 * (row count, context bound): the graph reads the row list from the cache's device copy, which
 * each call refreshes in stream order. */
int ab2_model_forward_rows(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, int S, const int *rows_host,
                           int nrows, int logits_mode, void *logits_dev, uint32_t *argmax_dev,
                           ab2_stream stream);
int ab2_model_decode_step_rows(ab2_model *m, ab2_kv *kv, const uint32_t *ids_dev, const int *rows_host,
                               int nrows, void *logits_dev, uint32_t *argmax_dev, ab2_stream stream);
/* Profiling aid (no counterpart in the reference): when the last one-row decode step ran as
 * the single persistent kernel, copies the GPU wall-clock timestamps (ns) of its phases to
 * values_host as [3 CTAs: first, middle, last][phase][10]: entries 0..3 = {phase start,
 * prologue done, CTA done, grid barrier passed}, 4..9 = points inside the phase (0 where a
 * phase has none); phases are embedding, then per block {qkv, attention, o,
 * gate|up, down}, the LM head, and the tail (argmax, length commit).  *nphases receives the
 * phase count.  The timestamps are recorded only by processes started with AB2_PS_TRACE set in
 * the environment (the default build of the kernel carries no probes); AB2_ERR_UNSUPPORTED
 * otherwise or when the model does not use that kernel, AB2_ERR_CAPACITY
 * when `capacity` (in values) is less than 30 * phases.  Synchronises the device. */
int ab2_model_step_trace(const ab2_model *m, unsigned long long *values_host, int capacity, int *nphases);

#ifdef __cplusplus
}
#endif
#endif /* AARAMBH_B200_H */
