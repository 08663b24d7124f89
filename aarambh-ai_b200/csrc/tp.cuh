// Tensor-parallel context (internal header).
#pragma once

#include "common.cuh"

constexpr int AB2_TP_MAX_WORLD = 8;

// What a kernel needs to deposit partial sums with every rank and to meet the
// other ranks.  Lives in device memory (one copy per rank, filled at attach
// time); all pointers are device pointers valid on this rank, the peers' ones
// mapped through CUDA IPC (or handed in by a single-process caller).
//
// The exchange carries its own arrival signal: an inbox entry is one 8-byte word
// {f32 partial sum, u32 exchange number}, written with one 8-byte store (atomic
// over NVLink), so a reader that sees the exchange number it waits for has the
// sum that came with it - no flag, no fence and no round trip besides the store
// itself.  Exchange numbers only grow, so a stale word never matches.
struct ab2_tp_peer_desc {
    unsigned long long *inbox[AB2_TP_MAX_WORLD];  // inbox[p]: rank p's inbox [2][world][max_elems] words
    uint32_t *epoch;                      // this rank's count of finished exchanges
    uint32_t *done;                       // CTAs of the consuming kernel that have read the exchange
    int rank, world;
    unsigned long long max_elems;
    unsigned long long wait_limit_ns;     // how long a reader waits for a peer's words (default two seconds)
    // exchange of (largest logit, its index) per row of a vocabulary-parallel head: a second small
    // inbox [2][world][2 * AB2_TP_ARGMAX_ROWS] words at this word offset of every rank's block
    unsigned long long argmax_off;
    uint32_t *argmax_epoch, *argmax_done;
};
constexpr int AB2_TP_ARGMAX_ROWS = 64;

__device__ __forceinline__ unsigned long long tp_ll_pack(float v, uint32_t exchange) {
    return (unsigned long long)__float_as_uint(v) | ((unsigned long long)exchange << 32);
}
__device__ __forceinline__ void tp_ll_store(unsigned long long *p, unsigned long long w) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(p), "l"(w) : "memory");
}
// Two adjacent inbox words (16-byte aligned); each half is a single-copy-atomic 8-byte access.
__device__ __forceinline__ void tp_ll_load2(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];\n" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long tp_wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
// Waits until the eight words at p (elements 8i .. 8i+7 of one rank's slot) carry `exchange`
// and returns their sums in v; false when the limit ran out.
__device__ __forceinline__ bool tp_ll_wait8(const unsigned long long *p, uint32_t exchange, unsigned long long limit_ns,
                                            float (&v)[8]) {
    unsigned long long t0 = 0;
    for (int spin = 0;; ++spin) {
        unsigned long long w[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) tp_ll_load2(p + 2 * j, w[2 * j], w[2 * j + 1]);
        bool ok = true;
#pragma unroll
        for (int j = 0; j < 8; ++j) ok = ok && (uint32_t)(w[j] >> 32) == exchange;
        if (ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float((uint32_t)w[j]);
            return true;
        }
        if ((spin & 15) == 15) {
            const unsigned long long now = tp_wall_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}

struct ab2_tp {
    int rank, world;
    void *comm;  // ncclComm_t; null when world == 1
    // one-shot exchange over NVLink peer memory (null until ab2_tp_peer_attach)
    void *local_block;                    // this rank's inbox + flags + epoch, one allocation
    void *peer_block[AB2_TP_MAX_WORLD];   // IPC mappings of the peers' blocks
    ab2_tp_peer_desc *desc_dev;
    size_t max_elems;
    bool attached;
    unsigned long long wait_limit_ns;
};

namespace ab2 {
int tp_all_reduce(ab2_tp *tp, void *buf, size_t count, ab2_dtype dtype, cudaStream_t s);
int tp_all_gather(ab2_tp *tp, const void *send, void *recv, size_t count, ab2_dtype dtype, cudaStream_t s);
// True when `count` f32 partial sums per rank can go through the peer exchange.
bool tp_peer_ready(const ab2_tp *tp, size_t count);
// x[i] += bf16(sum over ranks of the partial sums deposited for the current
// exchange), i < count; meets the other ranks first (bounded wait).
int tp_peer_reduce_add(ab2_tp *tp, void *x_bf16, size_t count, cudaStream_t s);
// This rank's `count` f32 partial sums of the current exchange into every rank's inbox.
int tp_peer_deposit(ab2_tp *tp, const float *partial_f32, size_t count, cudaStream_t s);
// out[row] = index (in the whole vocabulary) of the last maximum of the row's logits, whose shard
// [rows][vn] this rank holds: local argmax, one (value, index) pair per rank through the peer
// exchange, the same choice on every rank.  rows <= AB2_TP_ARGMAX_ROWS.
int tp_peer_argmax(ab2_tp *tp, const void *logits_local, int rows, int vn, ab2_dtype dtype, uint32_t *out, cudaStream_t s);
}
