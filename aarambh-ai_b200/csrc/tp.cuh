// Tensor-parallel context (internal header).
#pragma once

#include "common.cuh"

struct ab2_tp {
    int rank, world;
    void *comm;  // ncclComm_t; null when world == 1
};

namespace ab2 {
int tp_all_reduce(ab2_tp *tp, void *buf, size_t count, ab2_dtype dtype, cudaStream_t s);
int tp_all_gather(ab2_tp *tp, const void *send, void *recv, size_t count, ab2_dtype dtype, cudaStream_t s);
}
