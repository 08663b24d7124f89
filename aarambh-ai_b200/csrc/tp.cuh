// Tensor-parallel context (internal header).
#pragma once

#include "common.cuh"

constexpr int AB2_TP_MAX_WORLD = 8;

// What a kernel needs to deposit partial sums with every rank and to meet the
// other ranks.  Lives in device memory (one copy per rank, filled at attach
// time); all pointers are device pointers valid on this rank, the peers' ones
// mapped through CUDA IPC.
struct ab2_tp_peer_desc {
    float *inbox[AB2_TP_MAX_WORLD];       // inbox[p]: rank p's inbox [2][world][max_elems] f32
    uint32_t *flags[AB2_TP_MAX_WORLD];    // flags[p]: rank p's arrival words [world]; I write flags[p][rank]
    uint32_t *epoch;                      // this rank's count of finished exchanges
    uint32_t *done;                       // CTAs of the consuming kernel that have read the exchange
    uint32_t *ready;                      // last exchange whose partial sums have all arrived (set by CTA 0)
    int rank, world;
    unsigned long long max_elems;
};

struct ab2_tp {
    int rank, world;
    void *comm;  // ncclComm_t; null when world == 1
    // one-shot exchange over NVLink peer memory (null until ab2_tp_peer_attach)
    void *local_block;                    // this rank's inbox + flags + epoch, one allocation
    void *peer_block[AB2_TP_MAX_WORLD];   // IPC mappings of the peers' blocks
    ab2_tp_peer_desc *desc_dev;
    size_t max_elems;
    bool attached;
};

namespace ab2 {
int tp_all_reduce(ab2_tp *tp, void *buf, size_t count, ab2_dtype dtype, cudaStream_t s);
int tp_all_gather(ab2_tp *tp, const void *send, void *recv, size_t count, ab2_dtype dtype, cudaStream_t s);
// True when `count` f32 partial sums per rank can go through the peer exchange.
bool tp_peer_ready(const ab2_tp *tp, size_t count);
// x[i] += bf16(sum over ranks of the partial sums deposited for the current
// exchange), i < count; meets the other ranks first (bounded wait).
int tp_peer_reduce_add(ab2_tp *tp, void *x_bf16, size_t count, cudaStream_t s);
}
