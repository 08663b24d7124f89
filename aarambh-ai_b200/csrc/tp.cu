// Tensor-parallel plumbing: one NCCL communicator per process (one process per
// GPU) and the sum all-reduce / all-gather the sharded decoder needs after its
// row-parallel projections.  The reference has data-parallel training only; its
// single collective is an NCCL sum all-reduce bootstrapped from a 128-byte
// unique id (crates/aarambh-studio-train/src/distributed.rs:474-514,526-591),
// and this keeps that convention: the caller distributes the id.
//
// NCCL is resolved at run time from the library the host process already
// loaded (libnccl.so.2), so the shared object has no link-time dependency on it.
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
    delete tp;
    return AB2_OK;
}

AB2_API int ab2_tp_all_reduce(ab2_tp *tp, void *buf_dev, size_t count, ab2_dtype dtype, ab2_stream stream) {
    AB2_REQUIRE(tp && buf_dev, AB2_ERR_BAD_ARG, "null argument");
    return tp_all_reduce(tp, buf_dev, count, dtype, (cudaStream_t)stream);
}
