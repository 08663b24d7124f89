// Tensor-parallel plumbing: one NCCL communicator per process (one process per
// GPU) and the sum all-reduce / all-gather the sharded decoder needs after its
// row-parallel projections.  The reference has data-parallel training only; its
// single collective is an NCCL sum all-reduce bootstrapped from a 128-byte
// unique id (crates/aarambh-studio-train/src/distributed.rs:474-514,526-591),
// and this keeps that convention: the caller distributes the id.
//
// NCCL is resolved at run time from the library the host process already
// loaded (libnccl.so.2), so the shared object has no link-time dependency on it.
//
// The all-reduce of the decoder's row-parallel projections does not have to go
// through NCCL: once the ranks have exchanged CUDA IPC handles
// (ab2_tp_peer_export / ab2_tp_peer_attach), the projection kernel stores its f32
// partial sums straight into every rank's inbox over NVLink, each as one 8-byte
// word {sum, exchange number}; the consumer (the next projection's prologue, or
// one small kernel) waits (bounded) until the words it needs carry the current
// exchange number, adds the partials in rank order and applies the residual -
// no flag, no fence, no signal round trip.  Inboxes are double-buffered by the
// parity of a per-rank exchange count kept in device memory, so graph replays
// need no host-side sequence number.  Only plain stores and loads touch peer
// memory.
#include <dlfcn.h>
#include <nccl.h>

#include <cstddef>
#include <cstring>

#include "common.cuh"
#include "tp.cuh"

using namespace ab2;

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

int load_nccl() {
    if (g_nccl.handle) return AB2_OK;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (!h) return fail(AB2_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded: %s", dlerror());
#define SYM(field, name)                                                                 \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));                \
    if (!g_nccl.field) return fail(AB2_ERR_UNSUPPORTED, "NCCL symbol %s is missing", name)
    SYM(GetUniqueId, "ncclGetUniqueId");
    SYM(CommInitRank, "ncclCommInitRank");
    SYM(CommDestroy, "ncclCommDestroy");
    SYM(AllReduce, "ncclAllReduce");
    SYM(AllGather, "ncclAllGather");
    SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
    g_nccl.handle = h;
    return AB2_OK;
}

ncclDataType_t nccl_type(ab2_dtype d) {
    return d == AB2_F32 ? ncclFloat32 : d == AB2_F16 ? ncclFloat16 : ncclBfloat16;
}

}  // namespace

#define AB2_NCCL(expr)                                                                          \
    do {                                                                                        \
        ncclResult_t _r = (expr);                                                               \
        if (_r != ncclSuccess)                                                                  \
            return fail(AB2_ERR_CUDA, "%s failed: %s", #expr, g_nccl.GetErrorString(_r));       \
    } while (0)

namespace ab2 {

int device_status_word(int **out);

namespace {

// The partial sums of exchange e = epoch + 1 arrive in buffer e & 1 of every inbox (stored there
// by the projection kernels of each rank, or by tp_peer_deposit_kernel), every word tagged with
// e.  x += bf16(sum_r partial_r), summed in rank order on every rank.
__global__ void __launch_bounds__(256)
tp_peer_reduce_add_kernel(__nv_bfloat16 *x, size_t count, const ab2_tp_peer_desc *desc, int *status) {
    __shared__ int failed;
    pdl_wait();  // this rank's partial sums (and x) come from the preceding kernels
    pdl_launch_dependents();
    const ab2_tp_peer_desc d = *desc;
    const uint32_t e = *d.epoch + 1;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    const unsigned long long *box = d.inbox[d.rank] + (size_t)(e & 1u) * d.world * d.max_elems;
    const size_t nvec = count >> 3;  // 8 elements per thread and pass
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < d.world; ++r) {
            float pv[8];
            if (!tp_ll_wait8(box + (size_t)r * d.max_elems + 8 * i, e, d.wait_limit_ns, pv)) {
                failed = 1;
#pragma unroll
                for (int j = 0; j < 8; ++j) pv[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] += pv[j];
        }
        const uint4 xv = reinterpret_cast<const uint4 *>(x)[i];
        uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f0 = __uint_as_float(w[j] << 16) + __bfloat162float(__float2bfloat16_rn(sum[2 * j]));
            const float f1 = __uint_as_float(w[j] & 0xffff0000u) + __bfloat162float(__float2bfloat16_rn(sum[2 * j + 1]));
            w[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f0)) |
                   ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f1)) << 16);
        }
        reinterpret_cast<uint4 *>(x)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (blockIdx.x == 0)  // a tail of fewer than 8 elements
        for (size_t i = (nvec << 3) + threadIdx.x; i < count; i += blockDim.x) {
            float sum = 0.f;
            for (int r = 0; r < d.world; ++r) {
                const unsigned long long *p = box + (size_t)r * d.max_elems + i;
                unsigned long long w = 0, t0 = 0;
                bool ok = false;
                for (int spin = 0;; ++spin) {
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(w) : "l"(p) : "memory");
                    if ((uint32_t)(w >> 32) == e) { ok = true; break; }
                    if ((spin & 15) == 15) {
                        const unsigned long long now = tp_wall_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > d.wait_limit_ns) break;
                    }
                }
                if (!ok) failed = 1;
                sum += ok ? __uint_as_float((uint32_t)w) : 0.f;
            }
            x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + __bfloat162float(__float2bfloat16_rn(sum)));
        }
    __syncthreads();
    if (failed) {
        // a peer's sums did not arrive within the limit (x holds what did arrive): record it; the
        // exchange count stays, ab2_tp_peer_reset puts the ranks back in step
        if (threadIdx.x == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
        return;
    }
    // every CTA has read the exchange count and its share of the inbox: the last one closes the exchange
    if (threadIdx.x == 0 && atomicAdd(d.done, 1u) == gridDim.x - 1) {
        *d.done = 0;
        __threadfence();
        *d.epoch = e;
    }
}

// This rank's partial sums of the current exchange into every rank's inbox.
__global__ void __launch_bounds__(256)
tp_peer_deposit_kernel(const float *partial, size_t count, const ab2_tp_peer_desc *desc) {
    pdl_wait();
    pdl_launch_dependents();
    const ab2_tp_peer_desc d = *desc;
    const uint32_t e = *d.epoch + 1;
    const size_t off = ((size_t)(e & 1u) * d.world + d.rank) * d.max_elems;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned long long w = tp_ll_pack(partial[i], e);
        for (int p = 0; p < d.world; ++p) tp_ll_store(d.inbox[p] + off + i, w);
    }
}

// Key of the argmax: monotone in the f32 total order, ties to the larger index (the last maximum,
// crates/aarambh-studio-inference/src/sampler.rs:217-224).
__device__ __forceinline__ long long tp_argmax_key(float v, uint32_t idx) {
    int b = __float_as_int(v);
    b ^= (int)(((unsigned)(b >> 31)) >> 1);
    return ((long long)b << 32) | idx;
}

// One CTA per row: argmax of this rank's shard, then one (value, index) pair to every rank (two
// tagged 8-byte words), a bounded wait for the world's pairs, and the same winner on every rank.
template <typename T>
__global__ void __launch_bounds__(1024)
tp_argmax_exchange_kernel(const ab2_tp_peer_desc *desc, const T *__restrict__ logits, int vn, uint32_t *out, int *status) {
    __shared__ long long warp_best[32];
    pdl_wait();  // the logits come from the preceding kernel
    pdl_launch_dependents();
    const ab2_tp_peer_desc d = *desc;
    const T *row = logits + (size_t)blockIdx.x * vn;
    const uint32_t base = (uint32_t)d.rank * (uint32_t)vn;
    long long best = LLONG_MIN;
    for (int i = threadIdx.x; i < vn; i += blockDim.x) best = max(best, tp_argmax_key(to_f32(row[i]), base + (uint32_t)i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x >= 32) return;
    best = threadIdx.x < (blockDim.x >> 5) ? warp_best[threadIdx.x] : LLONG_MIN;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    const uint32_t e = *d.argmax_epoch + 1;
    const size_t slot = d.argmax_off + (size_t)(e & 1u) * d.world * (2 * AB2_TP_ARGMAX_ROWS) + 2 * (size_t)blockIdx.x;
    // lane p stores this rank's pair with rank p, then waits for rank p's pair in the local inbox
    bool ok = true;
    long long theirs = LLONG_MIN;
    if ((int)threadIdx.x < d.world) {
        const int p = (int)threadIdx.x;
        unsigned long long *dst = d.inbox[p] + slot + (size_t)d.rank * (2 * AB2_TP_ARGMAX_ROWS);
        tp_ll_store(dst, ((unsigned long long)e << 32) | (uint32_t)(best >> 32));
        tp_ll_store(dst + 1, ((unsigned long long)e << 32) | (uint32_t)best);
        const unsigned long long *src = d.inbox[d.rank] + slot + (size_t)p * (2 * AB2_TP_ARGMAX_ROWS);
        unsigned long long hi = 0, lo = 0, t0 = 0;
        for (int spin = 0;; ++spin) {
            tp_ll_load2(src, hi, lo);
            if ((uint32_t)(hi >> 32) == e && (uint32_t)(lo >> 32) == e) break;
            if ((spin & 15) == 15) {
                const unsigned long long now = tp_wall_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > d.wait_limit_ns) { ok = false; break; }
            }
        }
        theirs = (long long)(((unsigned long long)(uint32_t)hi << 32) | (uint32_t)lo);
    }
    ok = __all_sync(0xffffffffu, ok);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) theirs = max(theirs, __shfl_xor_sync(0xffffffffu, theirs, o));
    if (threadIdx.x != 0) return;
    if (!ok) {  // a peer's pair did not arrive within the limit: the exchange count stays (ab2_tp_peer_reset)
        atomicExch(status, (int)AB2_ERR_TIMEOUT);
        return;
    }
    out[blockIdx.x] = (uint32_t)theirs;
    if (atomicAdd(d.argmax_done, 1u) == gridDim.x - 1) {  // every row has read the exchange count: close the exchange
        *d.argmax_done = 0;
        __threadfence();
        *d.argmax_epoch = e;
    }
}

}  // namespace

bool tp_peer_ready(const ab2_tp *tp, size_t count) {
    return tp && tp->world > 1 && tp->attached && count <= tp->max_elems;
}

int tp_peer_reduce_add(ab2_tp *tp, void *x_bf16, size_t count, cudaStream_t s) {
    AB2_REQUIRE(tp_peer_ready(tp, count), AB2_ERR_BAD_ARG, "the peer exchange is not attached or %zu elements exceed it", count);
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    AB2_REQUIRE(((uintptr_t)x_bf16 & 15) == 0, AB2_ERR_BAD_ALIGN, "the residual stream must be 16-byte aligned");
    const unsigned ctas = (unsigned)std::max<size_t>(1, std::min<size_t>(32, (count / 8 + 255) / 256));
    cudaError_t e = launch_kernel(tp_peer_reduce_add_kernel, dim3(ctas), dim3(256), 0, s, (__nv_bfloat16 *)x_bf16, count,
                                  (const ab2_tp_peer_desc *)tp->desc_dev, status);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "peer reduce launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

int tp_peer_deposit(ab2_tp *tp, const float *partial_f32, size_t count, cudaStream_t s) {
    AB2_REQUIRE(tp_peer_ready(tp, count), AB2_ERR_BAD_ARG, "the peer exchange is not attached or %zu elements exceed it", count);
    const unsigned ctas = (unsigned)std::max<size_t>(1, std::min<size_t>(64, (count + 255) / 256));
    cudaError_t e = launch_kernel(tp_peer_deposit_kernel, dim3(ctas), dim3(256), 0, s, partial_f32, count,
                                  (const ab2_tp_peer_desc *)tp->desc_dev);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "peer deposit launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

int tp_peer_argmax(ab2_tp *tp, const void *logits_local, int rows, int vn, ab2_dtype dtype, uint32_t *out, cudaStream_t s) {
    AB2_REQUIRE(tp && tp->world > 1 && tp->attached, AB2_ERR_BAD_ARG, "the peer exchange is not attached");
    AB2_REQUIRE(rows >= 1 && rows <= AB2_TP_ARGMAX_ROWS, AB2_ERR_CAPACITY, "the argmax exchange serves up to %d rows, got %d",
                AB2_TP_ARGMAX_ROWS, rows);
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    const ab2_tp_peer_desc *desc = tp->desc_dev;
    cudaError_t e;
    switch (dtype) {
    case AB2_F32: e = launch_kernel(tp_argmax_exchange_kernel<float>, dim3(rows), dim3(1024), 0, s, desc, (const float *)logits_local, vn, out, status); break;
    case AB2_F16: e = launch_kernel(tp_argmax_exchange_kernel<__half>, dim3(rows), dim3(1024), 0, s, desc, (const __half *)logits_local, vn, out, status); break;
    default: e = launch_kernel(tp_argmax_exchange_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), 0, s, desc, (const __nv_bfloat16 *)logits_local, vn, out, status); break;
    }
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "argmax exchange launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

int tp_all_reduce(ab2_tp *tp, void *buf, size_t count, ab2_dtype dtype, cudaStream_t s) {
    if (!tp || tp->world == 1) return AB2_OK;
    AB2_REQUIRE(tp->comm != nullptr, AB2_ERR_UNSUPPORTED, "this tensor-parallel context was created without a communicator");
    AB2_NCCL(g_nccl.AllReduce(buf, buf, count, nccl_type(dtype), ncclSum, (ncclComm_t)tp->comm, s));
    return AB2_OK;
}

int tp_all_gather(ab2_tp *tp, const void *send, void *recv, size_t count, ab2_dtype dtype, cudaStream_t s) {
    AB2_REQUIRE(tp != nullptr, AB2_ERR_BAD_ARG, "null tensor-parallel context");
    AB2_REQUIRE(tp->comm != nullptr, AB2_ERR_UNSUPPORTED, "this tensor-parallel context was created without a communicator");
    AB2_NCCL(g_nccl.AllGather(send, recv, count, nccl_type(dtype), (ncclComm_t)tp->comm, s));
    return AB2_OK;
}

}  // namespace ab2

AB2_API int ab2_tp_unique_id(void *id128) {
    AB2_REQUIRE(id128 != nullptr, AB2_ERR_BAD_ARG, "null argument");
    int rc = load_nccl();
    if (rc != AB2_OK) return rc;
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
    ncclUniqueId id;
    AB2_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id128, &id, 128);
    return AB2_OK;
}

AB2_API int ab2_tp_create(ab2_tp **out, int rank, int world, const void *id128) {
    AB2_REQUIRE(out != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(world >= 1 && rank >= 0 && rank < world, AB2_ERR_BAD_ARG, "rank %d outside world size %d", rank, world);
    ab2_tp *tp = new ab2_tp();
    tp->rank = rank; tp->world = world; tp->comm = nullptr;
    tp->local_block = nullptr; tp->desc_dev = nullptr; tp->max_elems = 0; tp->attached = false;
    for (int i = 0; i < AB2_TP_MAX_WORLD; ++i) tp->peer_block[i] = nullptr;
    tp->wait_limit_ns = 2000000000ull;
    if (world > 1 && id128 != nullptr) {
        int rc = load_nccl();
        if (rc != AB2_OK) { delete tp; return rc; }
        ncclUniqueId id;
        memcpy(&id, id128, 128);
        ncclComm_t comm;
        ncclResult_t r = g_nccl.CommInitRank(&comm, world, id, rank);
        if (r != ncclSuccess) {
            delete tp;
            return fail(AB2_ERR_CUDA, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
        }
        tp->comm = comm;
    }
    *out = tp;
    return AB2_OK;
}

AB2_API int ab2_tp_destroy(ab2_tp *tp) {
    if (!tp) return AB2_OK;
    if (tp->comm) g_nccl.CommDestroy((ncclComm_t)tp->comm);
    for (int i = 0; i < AB2_TP_MAX_WORLD; ++i)
        if (tp->peer_block[i]) cudaIpcCloseMemHandle(tp->peer_block[i]);
    if (tp->desc_dev) cudaFree(tp->desc_dev);
    if (tp->local_block) cudaFree(tp->local_block);
    delete tp;
    return AB2_OK;
}

AB2_API int ab2_tp_all_reduce(ab2_tp *tp, void *buf_dev, size_t count, ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(tp && buf_dev, AB2_ERR_BAD_ARG, "null argument");
    return tp_all_reduce(tp, buf_dev, count, dtype, (cudaStream_t)stream);
}

// Layout of a rank's block: inbox [2][world][max_elems] 8-byte words, then 32 words of counters
// (epoch, done, argmax epoch, argmax done), then the argmax inbox [2][world][2 * AB2_TP_ARGMAX_ROWS] words.
static size_t peer_inbox_words(int world, size_t max_elems) { return 2 * (size_t)world * max_elems; }
static size_t peer_argmax_off(int world, size_t max_elems) { return peer_inbox_words(world, max_elems) + 32; }
static size_t peer_block_bytes(int world, size_t max_elems) {
    return (peer_argmax_off(world, max_elems) + 2 * (size_t)world * 2 * AB2_TP_ARGMAX_ROWS) * 8;
}

static int peer_fill_desc(ab2_tp *tp, void *const *blocks) {
    ab2_tp_peer_desc d;
    memset(&d, 0, sizeof(d));
    for (int p = 0; p < tp->world; ++p) d.inbox[p] = (unsigned long long *)blocks[p];
    uint32_t *words = (uint32_t *)((unsigned long long *)tp->local_block + peer_inbox_words(tp->world, tp->max_elems));
    d.epoch = words;
    d.done = words + 1;
    d.argmax_epoch = words + 2;
    d.argmax_done = words + 3;
    d.argmax_off = peer_argmax_off(tp->world, tp->max_elems);
    d.rank = tp->rank; d.world = tp->world; d.max_elems = tp->max_elems;
    d.wait_limit_ns = tp->wait_limit_ns;
    if (!tp->desc_dev) AB2_CUDA(cudaMalloc((void **)&tp->desc_dev, sizeof(d)));
    AB2_CUDA(cudaMemcpy(tp->desc_dev, &d, sizeof(d), cudaMemcpyHostToDevice));
    tp->attached = true;
    return AB2_OK;
}

AB2_API int ab2_tp_peer_export(ab2_tp *tp, size_t max_elems, void *handle64_host) {
    AB2_REQUIRE(tp != nullptr, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tp->world > 1 && tp->world <= AB2_TP_MAX_WORLD, AB2_ERR_UNSUPPORTED,
                "the peer exchange serves 2..%d ranks, got %d", AB2_TP_MAX_WORLD, tp->world);
    AB2_REQUIRE(max_elems > 0 && max_elems % 8 == 0, AB2_ERR_BAD_SHAPE, "max_elems must be a positive multiple of 8");
    AB2_REQUIRE(tp->local_block == nullptr, AB2_ERR_BAD_ARG, "the peer exchange was exported already");
    const size_t bytes = peer_block_bytes(tp->world, max_elems);
    AB2_CUDA(cudaMalloc(&tp->local_block, bytes));
    AB2_CUDA(cudaMemset(tp->local_block, 0, bytes));
    AB2_CUDA(cudaDeviceSynchronize());
    tp->max_elems = max_elems;
    if (handle64_host) {  // a single-process caller that attaches by pointer needs no IPC handle
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle is 64 bytes");
        cudaIpcMemHandle_t h;
        AB2_CUDA(cudaIpcGetMemHandle(&h, tp->local_block));
        memcpy(handle64_host, &h, 64);
    }
    return AB2_OK;
}

AB2_API int ab2_tp_peer_block(ab2_tp *tp, void **block_dev, size_t *bytes) {
    AB2_REQUIRE(tp && block_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tp->local_block != nullptr, AB2_ERR_BAD_ARG, "export the local block first");
    *block_dev = tp->local_block;
    if (bytes) *bytes = peer_block_bytes(tp->world, tp->max_elems);
    return AB2_OK;
}

AB2_API int ab2_tp_peer_attach(ab2_tp *tp, const void *handles_host) {
    AB2_REQUIRE(tp && handles_host, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tp->local_block != nullptr && !tp->attached, AB2_ERR_BAD_ARG, "export the local block first (once)");
    void *blocks[AB2_TP_MAX_WORLD] = {nullptr};
    for (int p = 0; p < tp->world; ++p) {
        blocks[p] = tp->local_block;
        if (p != tp->rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const char *)handles_host + (size_t)p * 64, 64);
            AB2_CUDA(cudaIpcOpenMemHandle(&tp->peer_block[p], h, cudaIpcMemLazyEnablePeerAccess));
            blocks[p] = tp->peer_block[p];
        }
    }
    return peer_fill_desc(tp, blocks);
}

AB2_API int ab2_tp_peer_attach_ptrs(ab2_tp *tp, void *const *blocks_dev) {
    AB2_REQUIRE(tp && blocks_dev, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tp->local_block != nullptr && !tp->attached, AB2_ERR_BAD_ARG, "export the local block first (once)");
    void *blocks[AB2_TP_MAX_WORLD] = {nullptr};
    for (int p = 0; p < tp->world; ++p) {
        blocks[p] = p == tp->rank ? tp->local_block : blocks_dev[p];
        AB2_REQUIRE(blocks[p] != nullptr && ((uintptr_t)blocks[p] & 15) == 0, AB2_ERR_BAD_ARG, "block of rank %d is null or misaligned", p);
    }
    return peer_fill_desc(tp, blocks);
}

AB2_API int ab2_tp_set_wait_limit_ns(ab2_tp *tp, unsigned long long limit_ns) {
    AB2_REQUIRE(tp != nullptr && limit_ns > 0, AB2_ERR_BAD_ARG, "null context or zero limit");
    tp->wait_limit_ns = limit_ns;
    if (tp->desc_dev) {
        AB2_CUDA(cudaDeviceSynchronize());
        AB2_CUDA(cudaMemcpy((char *)tp->desc_dev + offsetof(ab2_tp_peer_desc, wait_limit_ns), &limit_ns, sizeof(limit_ns),
                            cudaMemcpyHostToDevice));
    }
    return AB2_OK;
}

AB2_API int ab2_tp_peer_reset(ab2_tp *tp) {
    AB2_REQUIRE(tp != nullptr && tp->local_block != nullptr, AB2_ERR_BAD_ARG, "the peer exchange was not exported");
    AB2_CUDA(cudaDeviceSynchronize());
    AB2_CUDA(cudaMemset(tp->local_block, 0, peer_block_bytes(tp->world, tp->max_elems)));
    AB2_CUDA(cudaDeviceSynchronize());
    return AB2_OK;
}

AB2_API int ab2_tp_peer_deposit(ab2_tp *tp, const float *partial_dev, size_t count, ab2_stream stream) {
    AB2_REQUIRE(tp && partial_dev, AB2_ERR_BAD_ARG, "null argument");
    return tp_peer_deposit(tp, partial_dev, count, (cudaStream_t)stream);
}

AB2_API int ab2_tp_peer_reduce_add(ab2_tp *tp, void *x_bf16_dev, size_t count, ab2_stream stream) {
    AB2_REQUIRE(tp && x_bf16_dev, AB2_ERR_BAD_ARG, "null argument");
    return tp_peer_reduce_add(tp, x_bf16_dev, count, (cudaStream_t)stream);
}
