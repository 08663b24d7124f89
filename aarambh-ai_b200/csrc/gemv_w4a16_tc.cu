// W4A16 (group 128, bf16) decode GEMM for 2..32 tokens on the 5th-generation
// tensor cores, built so that the packed weights cross HBM once and cost one
// shift and one logic op per pair of codes whatever the token count.
//
//   Y[M, N] = X[M, K] . W^T,  W packed 4-bit in tile-major blocks (w4a16_layout.cuh)
//
// The 128 output channels of a channel tile are the M dimension of the MMA, the
// tokens (padded to NTOK) its N dimension.  Operand A is the integer q - zero in
// bf16, not the dequantised weight: the unpack warps turn codes into 128 + q
// (0x4300 | q, one shift and one logic op per pair of codes), add the channel's
// -(128 + zero) as one packed bf16 add (exact: both are small integers) and write
// the pair to the swizzled operand stage.  The scale is applied per quantisation
// group in f32 by the epilogue warps: after the MMAs of a group
//   d[c][t] = sum_k x[t][k] (q[c][k] - zero[c])        (tensor memory)
// and the group adds scale[c] * d[c][t] to the running f32 output kept in the
// epilogue threads' registers (thread = channel).  Four accumulators rotate in
// tensor memory, so the epilogue of a group overlaps the MMAs of the next ones.
// (An earlier form kept the zero point out of operand A and obtained the
// per-group activation sums from a second MMA against an all-ones tile; halving
// the MMA count this way gave 3-8 % per GEMM and 8 % on the 32-row decode step.)
//
// Work is the sequence of (channel tile, group) units in tile-major order, cut
// into one contiguous range per CTA (one CTA per SM), so small weights are split
// over K.  A channel tile cut by a range boundary is finished by the CTA that
// arrives last: partial sums go to a global scratch slot per contributor, a
// counter per tile tells who is last, and the slots are added in contributor
// order.  One CTA per SM, warp-specialised:
//   warp 0        TMA tile loads of X (two 64-wide halves per group, 128-byte
//                 swizzle) into the operand-B stages
//   warps 1, 14   tcgen05.mma issue and commits on alternate units (warp 1 also
//                 allocates the tensor memory)
//   warps 2-9     unpack: thread = (channel, half of the group), reading the 32
//                 channels' two packed blocks from the ring the warp shares with
//                 its partner warp
//   warps 10-13   epilogue: tcgen05.ld of D, scale, running sums, the tile's final
//                 store (or partial + hand-over)
//   warp 15       packed weights: lane b copies block b of a unit into the rings
//                 (eight bulk copies in parallel; issuing one keeps a warp busy for
//                 a few hundred cycles, which the unpack warps cannot afford)
// Every wait on an mbarrier is bounded; on a time-out the CTA records
// AB2_ERR_TIMEOUT, stops issuing work, still frees its tensor memory and returns.
#include <algorithm>

#include "common.cuh"
#include "gemv_w4a16_mma.cuh"
#include "ops.cuh"
#include "tcgen05_util.cuh"

using namespace ab2;
using namespace ab2::tc;

namespace ab2 {
int device_status_word(int **out);
int device_sm_count();
namespace {

constexpr int DG_STAGES = 4;         // operand-A stages of 64 K-elements (two per group)
constexpr int DG_XSTAGES = 8;        // operand-B (activation) stages: small, so the ring is deeper
constexpr int DG_WSLOTS = 12;        // depth of a packed-weight ring (two blocks = 32 channels of one unit per slot)
constexpr int DG_WSLOT_BYTES = 2 * W4_BLOCK_WORDS * 4;  // per ring; four rings (one per 32 channels) = ~100 KB in flight per SM
constexpr int DG_A_BYTES = 128 * 128;  // 128 channels x 64 bf16
constexpr int DG_MMA_WARPS = 2;        // MMA-issue warps, taking alternate units (warp 1 and the warps after the epilogue)
constexpr int DG_THREADS = 448 + 32 * (DG_MMA_WARPS - 1) + 32;  // the last warp fetches the packed weights
constexpr int DG_ACC = 4;             // accumulator pairs (D, S) in tensor memory
// An MMA-issue warp must see every phase of the barriers it waits on (a parity wait cannot tell
// phase k from phase k + 2), so the stages, activation stages and accumulators a unit uses must come
// back to the same warp: their counts are multiples of what DG_MMA_WARPS units use.
static_assert(DG_STAGES % (2 * DG_MMA_WARPS) == 0 && DG_XSTAGES % (2 * DG_MMA_WARPS) == 0 && DG_ACC % DG_MMA_WARPS == 0,
              "ring depths must be multiples of the MMA-issue warps' stride");
constexpr int DG_PARAM_BUFS = 16;      // a buffer is rewritten 16 units later: its reader is long done

struct DgShared {
    uint64_t wfull[4][DG_WSLOTS], wempty[4][DG_WSLOTS];
    uint64_t xfull[DG_XSTAGES], xempty[DG_XSTAGES], afull[DG_STAGES], sempty[DG_STAGES];
    uint64_t accfull[DG_ACC], accempty[DG_ACC];
    uint32_t params[DG_PARAM_BUFS][128];  // scale | -(128 + zero) of the unit's 128 channels
    uint32_t tmem_base;
    int failed;
    int last_flag;
};

template <int NTOK>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[NTOK]);
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}

// units [u0, u1) of this CTA; the first `rem` CTAs take base + 1 units
struct DgRange { int base, rem, u0, u1; };
__device__ __forceinline__ DgRange dg_range(int total, int ctas, int cta) {
    DgRange r;
    r.base = total / ctas;
    r.rem = total - r.base * ctas;
    r.u0 = cta * r.base + min(cta, r.rem);
    r.u1 = r.u0 + r.base + (cta < r.rem ? 1 : 0);
    return r;
}
__device__ __forceinline__ int dg_owner(const DgRange &r, int u) {
    const int cut = r.rem * (r.base + 1);
    return u < cut ? u / (r.base + 1) : r.rem + (u - cut) / r.base;
}

// partials: [gridDim.x][2][NTOK][128] f32; counters: one int per channel tile, zero on entry and exit.
template <int NTOK, int EPI>
__global__ void __launch_bounds__(DG_THREADS, 1)
gemv_w4a16_tc_kernel(const uint32_t *__restrict__ wt, const __grid_constant__ CUtensorMap xmap,
                     __nv_bfloat16 *y, const __nv_bfloat16 *resid, int N, int K, int M, float *partials,
                     int *counters, int *status) {
    constexpr int B_BYTES = NTOK * 128;
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) | ((128u >> 4) << 24);
    constexpr uint32_t TMEM_COLS = NTOK == 16 ? 64u : 128u;  // DG_ACC accumulators of NTOK columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_st = smem;                                   // [DG_STAGES][DG_A_BYTES]
    uint8_t *b_st = a_st + DG_STAGES * DG_A_BYTES;          // [DG_XSTAGES][B_BYTES]
    uint8_t *w_ring = b_st + DG_XSTAGES * B_BYTES;           // [4][DG_WSLOTS][DG_WSLOT_BYTES]
    DgShared *sh = (DgShared *)(w_ring + 4 * DG_WSLOTS * DG_WSLOT_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = K >> 7, tiles16 = (N + 15) >> 4, n_tiles = (N + 127) >> 7;
    const DgRange rg = dg_range(n_tiles * G, (int)gridDim.x, (int)blockIdx.x);
    volatile int *failed = &sh->failed;

    if (threadIdx.x == 0) {
        for (int q = 0; q < 4; ++q)
            for (int i = 0; i < DG_WSLOTS; ++i) { bar_init(&sh->wfull[q][i], 1); bar_init(&sh->wempty[q][i], 2); }
        for (int i = 0; i < DG_STAGES; ++i) { bar_init(&sh->afull[i], 4); bar_init(&sh->sempty[i], 1); }
        for (int i = 0; i < DG_XSTAGES; ++i) { bar_init(&sh->xfull[i], 1); bar_init(&sh->xempty[i], 1); }
        for (int i = 0; i < DG_ACC; ++i) { bar_init(&sh->accfull[i], 1); bar_init(&sh->accempty[i], 4); }
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {  // tensor-memory allocation is a whole-warp operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sptr(&sh->tmem_base)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = sh->tmem_base;
    pdl_launch_dependents();  // the next kernel may start fetching its constant weights

    if (warp == 0) {
        // ---------------------------------------------------------- producer of the activation tiles
        if (lane == 0) {
            pdl_wait();  // the activations come from the preceding kernel
            uint32_t use = 0;
            for (int u = rg.u0; u < rg.u1 && !*failed; ++u, ++use) {
                const int g = u % G;
                for (int half = 0; half < 2; ++half) {
                    const uint32_t xuse = 2 * use + half;
                    const int xs = xuse % DG_XSTAGES;
                    if (!bar_wait(&sh->xempty[xs], ((xuse / DG_XSTAGES) & 1) ^ 1, failed)) break;
                    bar_expect_tx(&sh->xfull[xs], B_BYTES);
                    tma_load_2d(b_st + xs * B_BYTES, &xmap, g * 128 + half * 64, 0, &sh->xfull[xs]);
                }
            }
        }
    } else if (warp == DG_THREADS / 32 - 1) {
        // ---------------------------------------------------------- producer of the packed weights
        // Lane b fetches block b of a unit (blocks 2q and 2q + 1 go to ring q); issuing a copy occupies a
        // warp for a few hundred cycles, which the unpack warps used to pay once per unit each.
        const int n_units = rg.u1 - rg.u0;
        for (int use = 0; use < n_units && !*failed; ++use) {
            const int u = rg.u0 + use, nt = u / G, g = u - nt * G, ws = use % DG_WSLOTS;
            int ok = 1;
            if (use >= DG_WSLOTS && lane < 4) ok = bar_wait(&sh->wempty[lane][ws], ((use / DG_WSLOTS) & 1) ^ 1, failed) ? 1 : 0;
            if (!__all_sync(0xffffffffu, ok)) break;
            if (lane < 8) {
                const int q = lane >> 1, blk = nt * 8 + lane;
                if ((lane & 1) == 0) {
                    const int have = (blk < tiles16 ? 1 : 0) + (blk + 1 < tiles16 ? 1 : 0);
                    if (have) bar_expect_tx(&sh->wfull[q][ws], (uint32_t)have * W4_BLOCK_WORDS * 4);
                    else bar_arrive(&sh->wfull[q][ws]);  // a channel tile past the last row has fewer blocks
                }
            }
            __syncwarp();
            if (lane < 8 && nt * 8 + lane < tiles16)
                bulk_copy(w_ring + (lane >> 1) * DG_WSLOTS * DG_WSLOT_BYTES + ws * DG_WSLOT_BYTES + (lane & 1) * W4_BLOCK_WORDS * 4,
                          wt + ((size_t)(nt * 8 + lane) * G + g) * W4_BLOCK_WORDS, W4_BLOCK_WORDS * 4, &sh->wfull[lane >> 1][ws]);
        }
    } else if (warp == 1 || warp >= 14) {
        // ---------------------------------------------------------- MMA issue (alternate units per warp)
        const uint32_t my_id = warp == 1 ? 0u : (uint32_t)(warp - 13);
        uint32_t use = 0;
        for (int u = rg.u0; u < rg.u1 && !*failed; ++u, ++use) {
            if (use % DG_MMA_WARPS != my_id) continue;
            const int ab = use % DG_ACC;
            if (!bar_wait(&sh->accempty[ab], ((use / DG_ACC) & 1) ^ 1, failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t td = tmem + (uint32_t)(ab * NTOK);
            for (int half = 0; half < 2 && !*failed; ++half) {
                const uint32_t suse = 2 * use + half;
                const int s = suse % DG_STAGES, xs = suse % DG_XSTAGES;
                if (!bar_wait(&sh->xfull[xs], (suse / DG_XSTAGES) & 1, failed)) break;
                if (!bar_wait(&sh->afull[s], (suse / DG_STAGES) & 1, failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (lane == 0) {
                    const uint32_t a0 = sptr(a_st + s * DG_A_BYTES), b0 = sptr(b_st + xs * B_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(td, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), IDESC, (half | k) != 0);
                    umma_commit(&sh->sempty[s]);  // the operand stages are free when the MMAs retire
                    umma_commit(&sh->xempty[xs]);
                }
                __syncwarp();
            }
            if (lane == 0) umma_commit(&sh->accfull[ab]);
            __syncwarp();
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------- unpack: codes -> bf16 128 + q
        // The two warps that share 32 channels (one per half of the group) read those channels'
        // two packed blocks from a ring of their own, filled by the producer warp.
        const int t = (threadIdx.x - 64) & 127;   // channel within the 128-channel tile
        const int half = (threadIdx.x - 64) >> 7;  // which 64 of the group's 128 K-elements
        const int q = t >> 5;                      // ring: channels 32q .. 32q+31 = blocks 2q, 2q+1
        const int blk = t >> 4, r = t & 15;
        uint8_t *ring = w_ring + q * DG_WSLOTS * DG_WSLOT_BYTES;
        uint32_t k_mask = 0x000F000Fu, k_magic = 0x43004300u;
        asm volatile("" : "+r"(k_mask), "+r"(k_magic));
        uint32_t use = 0;
        for (int u = rg.u0; u < rg.u1 && !*failed; ++u, ++use) {
            const int ws = use % DG_WSLOTS;
            if (!bar_wait(&sh->wfull[q][ws], (use / DG_WSLOTS) & 1, failed)) break;
            const uint32_t *bw = (const uint32_t *)(ring + ws * DG_WSLOT_BYTES) + (blk & 1) * W4_BLOCK_WORDS;
            const uint4 p0 = *reinterpret_cast<const uint4 *>(bw + r * 16 + half * 8);
            const uint4 p1 = *reinterpret_cast<const uint4 *>(bw + r * 16 + half * 8 + 4);
            const uint32_t pr = bw[256 + r];
            if (half == 0) sh->params[use % DG_PARAM_BUFS][t] = pr;
            const uint32_t nz2 = __byte_perm(pr, pr, 0x3232);  // bf16x2 -(128 + zero) of this channel
            // one arrival per warp: arrivals on one mbarrier serialise on its word
            __syncwarp();
            if (lane == 0) bar_arrive_after(&sh->wempty[q][ws], p0.x ^ p1.x ^ pr, (uint32_t)K & 1u);
            const uint32_t suse = 2 * use + half;
            const int s = suse % DG_STAGES;
            if (!bar_wait(&sh->sempty[s], ((suse / DG_STAGES) & 1) ^ 1, failed)) break;
            uint8_t *arow = a_st + s * DG_A_BYTES + t * 128;
            const uint32_t words[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {  // chunk c = 8 consecutive k = one code word
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = bf16x2_add(w4_pair_bf16(words[c], j, k_mask, k_magic), nz2);  // q - zero, exact
                *reinterpret_cast<uint4 *>(arow + ((c ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(&sh->afull[s]);
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int quad = warp & 3;              // warps 10..13 -> TMEM lane quarters 2,3,0,1
        const int row = quad * 32 + lane;       // channel within the tile
        const int et = threadIdx.x - 320;       // 0..127 among the epilogue threads
        float acc[NTOK];
#pragma unroll
        for (int j = 0; j < NTOK; ++j) acc[j] = 0.f;
        uint32_t use = 0;
        for (int u = rg.u0; u < rg.u1 && !*failed; ++u, ++use) {
            const int nt = u / G, g = u - nt * G;
            const int ab = use % DG_ACC;
            if (!bar_wait(&sh->accfull[ab], (use / DG_ACC) & 1, failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t d[NTOK];
            tmem_ld<NTOK>(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ab * NTOK), d);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            const uint32_t pr = sh->params[use % DG_PARAM_BUFS][row];
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(&sh->accempty[ab]);
            const float sc = __uint_as_float(pr << 16);
#pragma unroll
            for (int j = 0; j < NTOK; ++j) acc[j] = fmaf(sc, __uint_as_float(d[j]), acc[j]);

            if (g != G - 1 && u + 1 != rg.u1) continue;
            // ---- end of this CTA's share of channel tile nt
            const int first_u = nt * G, last_u = first_u + G - 1;
            const bool whole = rg.u0 <= first_u && last_u < rg.u1;
            bool finish = whole;
            if (!whole) {
                const int c_first = dg_owner(rg, first_u), c_last = dg_owner(rg, last_u);
                const int which = (int)blockIdx.x == c_first ? 1 : 0;  // slot 1: the tile my range ends inside
                float *mine = partials + ((size_t)blockIdx.x * 2 + which) * (NTOK * 128);
#pragma unroll
                for (int j = 0; j < NTOK; ++j) mine[j * 128 + row] = acc[j];
                __threadfence();
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (et == 0) sh->last_flag = atomicAdd(&counters[nt], 1) == c_last - c_first;
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                finish = sh->last_flag != 0;
                if (finish) {
                    __threadfence();
#pragma unroll
                    for (int j = 0; j < NTOK; ++j) acc[j] = 0.f;
                    for (int c = c_first; c <= c_last; ++c) {
                        const float *p = partials + ((size_t)c * 2 + (c == c_first ? 1 : 0)) * (NTOK * 128);
#pragma unroll
                        for (int j = 0; j < NTOK; ++j) acc[j] += __ldcg(p + j * 128 + row);
                    }
                    if (et == 0) counters[nt] = 0;
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");  // last_flag is reused by the next cut tile
            }
            if (finish) {
                const int n = nt * 128 + row;
                // the residual may alias the output: its values are all read before the first store
                float rv[EPI == W4_EPI_ADD ? NTOK : 1];
                if (EPI == W4_EPI_ADD) {
#pragma unroll
                    for (int j = 0; j < NTOK; ++j)
                        rv[j] = (j < M && n < N) ? __bfloat162float(resid[(size_t)j * N + n]) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < NTOK; ++j) {
                    if (EPI == W4_EPI_SWIGLU) {
                        // channels come in 16s: 8 gate rows, then the 8 matching up rows (8 lanes further)
                        const float g_ = __bfloat162float(__float2bfloat16_rn(acc[j]));
                        const float u_ = __bfloat162float(__float2bfloat16_rn(__shfl_xor_sync(0xffffffffu, acc[j], 8)));
                        const int col = (n >> 4) * 8 + (n & 7), half_n = N >> 1;
                        if ((n & 8) == 0 && j < M && col < half_n)
                            y[(size_t)j * half_n + col] = __float2bfloat16_rn(swiglu_value(g_, u_));
                    } else if (j < M && n < N) {
                        const size_t o = (size_t)j * N + n;
                        float v = acc[j];
                        if (EPI == W4_EPI_F32) {
                            reinterpret_cast<float *>(y)[o] = v;
                        } else {
                            if (EPI == W4_EPI_ADD) v = rv[EPI == W4_EPI_ADD ? j : 0] + __bfloat162float(__float2bfloat16_rn(v));
                            y[o] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < NTOK; ++j) acc[j] = 0.f;
        }
    }

    // ---- teardown: every warp arrives here (all waits are bounded)
    if (!(warp == 0 && lane == 0)) pdl_wait();  // every thread passes the wait before the grid counts as finished
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && sh->failed) atomicExch(status, (int)AB2_ERR_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

template <int NTOK>
constexpr size_t dg_smem_bytes() {
    return 1024 + DG_STAGES * DG_A_BYTES + DG_XSTAGES * NTOK * 128 + 4 * DG_WSLOTS * DG_WSLOT_BYTES + sizeof(DgShared);
}

template <int NTOK, int EPI>
int launch_dg(const ab2_qweight *w, const void *x, int M, void *y, const void *resid, float *partials, int *counters,
              int max_ctas, cudaStream_t s) {
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    CUtensorMap map;
    rc = make_x_map(&map, x, M, w->K, NTOK);
    if (rc != AB2_OK) return rc;
    const size_t smem = dg_smem_bytes<NTOK>();
    static bool configured[64] = {false};  // the attribute is per device
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!configured[dev]) {
        AB2_CUDA(cudaFuncSetAttribute(gemv_w4a16_tc_kernel<NTOK, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = true;
    }
    const int units = ((w->N + 127) / 128) * (w->K / 128);
    const int grid = std::max(1, std::min(std::min(max_ctas, device_sm_count()), units / 2));
    cudaError_t e = launch_kernel(gemv_w4a16_tc_kernel<NTOK, EPI>, dim3(grid), dim3(DG_THREADS), smem, s,
                                  (const uint32_t *)w->codes, map, (__nv_bfloat16 *)y, (const __nv_bfloat16 *)resid, w->N,
                                  w->K, M, partials, counters, status);
    if (e != cudaSuccess) return fail(AB2_ERR_CUDA, "decode GEMM launch failed: %s", cudaGetErrorString(e));
    return AB2_OK;
}

}  // namespace

// Scratch the kernel needs per CTA: two slots of [32 tokens][128 channels] f32.
size_t gemv_w4a16_tc_partial_floats_per_cta() { return 2 * 32 * 128; }

// Y = epilogue(X[M][K] . W^T) for 2..32 tokens; partials / counters are the caller's
// scratch (zeroed counters, one per 128-channel tile; partials for max_ctas CTAs).
int qlinear_w4a16_tc_decode(const ab2_qweight *w, const void *x, int M, void *y, const void *resid, int epi,
                            float *partials, int *counters, int max_ctas, cudaStream_t s) {
    AB2_REQUIRE(M >= 1 && M <= 32, AB2_ERR_BAD_SHAPE, "the decode GEMM serves 1..32 tokens, got %d", M);
    AB2_REQUIRE(((uintptr_t)x & 15) == 0 && (w->K * 2) % 16 == 0, AB2_ERR_BAD_ALIGN, "activations must be 16-byte aligned");
#define AB2_DG(NT)                                                                                              \
    switch (epi) {                                                                                              \
    case W4_EPI_STORE: return launch_dg<NT, W4_EPI_STORE>(w, x, M, y, resid, partials, counters, max_ctas, s);   \
    case W4_EPI_ADD: return launch_dg<NT, W4_EPI_ADD>(w, x, M, y, resid, partials, counters, max_ctas, s);       \
    case W4_EPI_SWIGLU: return launch_dg<NT, W4_EPI_SWIGLU>(w, x, M, y, resid, partials, counters, max_ctas, s); \
    case W4_EPI_F32: return launch_dg<NT, W4_EPI_F32>(w, x, M, y, resid, partials, counters, max_ctas, s);       \
    default: return fail(AB2_ERR_BAD_ARG, "unsupported epilogue %d", epi);                                       \
    }
    if (M <= 16) { AB2_DG(16) }
    AB2_DG(32)
#undef AB2_DG
}

}  // namespace ab2
