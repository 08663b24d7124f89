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
// partial sums straight into every rank's inbox over NVLink, and one small
// kernel per exchange signals the peers, waits (bounded) for their signals,
// adds the partials in rank order and applies the residual.  Inboxes are
// double-buffered by the parity of a per-rank exchange count kept in device
// memory, so graph replays need no host-side sequence number.  Only plain
// stores and loads touch peer memory.
#include <dlfcn.h>
#include <nccl.h>

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

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA.  The partial sums of exchange e = epoch + 1 sit in buffer e & 1 of
// every inbox (stored there by the projection kernels that ran before this one
// on each rank).  x += bf16(sum_r partial_r), summed in rank order on every rank.
__global__ void __launch_bounds__(256)
tp_peer_reduce_add_kernel(__nv_bfloat16 *x, size_t count, const ab2_tp_peer_desc *desc, int *status) {
    __shared__ int failed;
    pdl_wait();  // this rank's partial sums (and x) come from the preceding kernels
    pdl_launch_dependents();
    const ab2_tp_peer_desc d = *desc;
    const uint32_t e = *d.epoch + 1;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    // CTA 0 exchanges the arrival signals with the peers and publishes the outcome in a local
    // word; the other CTAs (a few, all resident at once) wait for that word.
    if (blockIdx.x == 0) {
        if ((int)threadIdx.x < d.world && (int)threadIdx.x != d.rank) {
            const int p = threadIdx.x;
            __threadfence_system();
            st_release_sys(d.flags[p] + d.rank, e);  // "my partial sums of exchange e are in your inbox"
            const uint32_t *mine = d.flags[d.rank] + p;
            bool ok = false;
            unsigned long long t0, now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
            for (int spin = 0;; ++spin) {
                // the count only grows; a peer that is ahead has already passed e
                if ((int32_t)(ld_acquire_sys(mine) - e) >= 0) { ok = true; break; }
                if ((spin & 63) == 63) {
                    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
                    if (now - t0 > 2000000000ull) break;  // two seconds
                }
                __nanosleep(20);
            }
            if (!ok) failed = 1;
        }
        __syncthreads();
        if (threadIdx.x == 0 && !failed)
            asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(d.ready), "r"(e) : "memory");
    } else {
        if (threadIdx.x == 0) {
            bool ok = false;
            unsigned long long t0, now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
            for (int spin = 0;; ++spin) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(d.ready) : "memory");
                if ((int32_t)(v - e) >= 0) { ok = true; break; }
                if ((spin & 63) == 63) {
                    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
                    if (now - t0 > 3000000000ull) break;  // CTA 0's own limit plus a margin
                }
                __nanosleep(20);
            }
            if (!ok) failed = 1;
        }
        __syncthreads();
    }
    if (failed) {
        if (threadIdx.x == 0) atomicExch(status, (int)AB2_ERR_TIMEOUT);
        return;
    }
    const float *box = d.inbox[d.rank] + (size_t)(e & 1u) * d.world * d.max_elems;
    const size_t nvec = count >> 3;  // 8 elements per thread and pass
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < d.world; ++r) {
            const float4 p0 = __ldcg(reinterpret_cast<const float4 *>(box + (size_t)r * d.max_elems) + 2 * i);
            const float4 p1 = __ldcg(reinterpret_cast<const float4 *>(box + (size_t)r * d.max_elems) + 2 * i + 1);
            sum[0] += p0.x; sum[1] += p0.y; sum[2] += p0.z; sum[3] += p0.w;
            sum[4] += p1.x; sum[5] += p1.y; sum[6] += p1.z; sum[7] += p1.w;
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
            for (int r = 0; r < d.world; ++r) sum += __ldcg(box + (size_t)r * d.max_elems + i);
            x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + __bfloat162float(__float2bfloat16_rn(sum)));
        }
    __syncthreads();
    // every CTA has read the exchange count and its share of the inbox: the last one closes the exchange
    if (threadIdx.x == 0 && atomicAdd(d.done, 1u) == gridDim.x - 1) {
        *d.done = 0;
        __threadfence();
        *d.epoch = e;
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

int tp_all_reduce(ab2_tp *tp, void *buf, size_t count, ab2_dtype dtype, cudaStream_t s) {
    if (!tp || tp->world == 1) return AB2_OK;
    AB2_NCCL(g_nccl.AllReduce(buf, buf, count, nccl_type(dtype), ncclSum, (ncclComm_t)tp->comm, s));
    return AB2_OK;
}

int tp_all_gather(ab2_tp *tp, const void *send, void *recv, size_t count, ab2_dtype dtype, cudaStream_t s) {
    AB2_REQUIRE(tp != nullptr, AB2_ERR_BAD_ARG, "null tensor-parallel context");
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
    if (world > 1) {
        AB2_REQUIRE(id128 != nullptr, AB2_ERR_BAD_ARG, "a unique id is needed for more than one rank");
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

// Layout of a rank's block: inbox [2][world][max_elems] f32, then flags [world] u32, the epoch, done and ready words.
static size_t peer_block_bytes(int world, size_t max_elems) {
    return 2 * (size_t)world * max_elems * sizeof(float) + ((size_t)world + 3) * sizeof(uint32_t) + 256;
}

AB2_API int ab2_tp_peer_export(ab2_tp *tp, size_t max_elems, void *handle64_host) {
    AB2_REQUIRE(tp && handle64_host, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tp->world > 1 && tp->world <= AB2_TP_MAX_WORLD, AB2_ERR_UNSUPPORTED,
                "the peer exchange serves 2..%d ranks, got %d", AB2_TP_MAX_WORLD, tp->world);
    AB2_REQUIRE(max_elems > 0 && max_elems % 4 == 0, AB2_ERR_BAD_SHAPE, "max_elems must be a positive multiple of 4");
    AB2_REQUIRE(tp->local_block == nullptr, AB2_ERR_BAD_ARG, "the peer exchange was exported already");
    const size_t bytes = peer_block_bytes(tp->world, max_elems);
    AB2_CUDA(cudaMalloc(&tp->local_block, bytes));
    AB2_CUDA(cudaMemset(tp->local_block, 0, bytes));
    AB2_CUDA(cudaDeviceSynchronize());
    tp->max_elems = max_elems;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle is 64 bytes");
    cudaIpcMemHandle_t h;
    AB2_CUDA(cudaIpcGetMemHandle(&h, tp->local_block));
    memcpy(handle64_host, &h, 64);
    return AB2_OK;
}

AB2_API int ab2_tp_peer_attach(ab2_tp *tp, const void *handles_host) {
    AB2_REQUIRE(tp && handles_host, AB2_ERR_BAD_ARG, "null argument");
    AB2_REQUIRE(tp->local_block != nullptr && !tp->attached, AB2_ERR_BAD_ARG, "export the local block first (once)");
    ab2_tp_peer_desc d;
    memset(&d, 0, sizeof(d));
    const size_t inbox_floats = 2 * (size_t)tp->world * tp->max_elems;
    for (int p = 0; p < tp->world; ++p) {
        void *base = tp->local_block;
        if (p != tp->rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const char *)handles_host + (size_t)p * 64, 64);
            AB2_CUDA(cudaIpcOpenMemHandle(&tp->peer_block[p], h, cudaIpcMemLazyEnablePeerAccess));
            base = tp->peer_block[p];
        }
        d.inbox[p] = (float *)base;
        d.flags[p] = (uint32_t *)((float *)base + inbox_floats);
    }
    d.epoch = d.flags[tp->rank] + tp->world;
    d.done = d.epoch + 1;
    d.ready = d.epoch + 2;
    d.rank = tp->rank; d.world = tp->world; d.max_elems = tp->max_elems;
    AB2_CUDA(cudaMalloc((void **)&tp->desc_dev, sizeof(d)));
    AB2_CUDA(cudaMemcpy(tp->desc_dev, &d, sizeof(d), cudaMemcpyHostToDevice));
    tp->attached = true;
    return AB2_OK;
}
