// W4A16 (group 128, bf16) GEMM for many tokens (prefill, batched decode) on the
// 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
//   Y[M, N] = X[M, K] . W^T,  W packed 4-bit in tile-major blocks (w4a16_layout.cuh)
//
// The product is formed transposed: the 128 output channels of a tile are the M
// dimension of the MMA (operand A = dequantised weights), the tokens its N
// dimension (operand B = activations), so any token count is a legal N and the
// weights are dequantised once per (channel tile, token tile).  One CTA per SM,
// persistent over tiles, warp-specialised:
//   warp 0      producer of the packed weights: one ring slot per quantisation
//               group, lane b issues the bulk copy of 16-channel block b
//   warp 10     producer of the activations: TMA tile loads of X (128-byte
//               swizzle) into the operand-B stages
//   warp 1      allocates tensor memory, issues tcgen05.mma (K = 16 per
//               instruction, 64 per stage), commits stage / accumulator barriers.
//               A tcgen05 instruction costs the issuing thread on the order of a
//               hundred cycles, about what a 128 x 256 x 16 MMA takes to execute:
//               tiles are 256 tokens wide where the token count allows, and the
//               operand rings of that tile size have equal depth so that one
//               commit per stage frees both operands
//   warps 2-5   dequantise: thread = output channel; nibbles -> bf16 (128 + q by
//               one logic op, minus (128 + z) exactly, times the bf16 scale, i.e.
//               the round-to-nearest bf16 of (q - z) * s) written into the
//               operand-A stage in the canonical K-major 128-byte-swizzle layout
//   warps 6-9   epilogue: tcgen05.ld of the accumulator, bf16 stores of Y
// Every wait on an mbarrier is bounded; on a time-out the CTA records
// AB2_ERR_TIMEOUT, stops issuing work, still frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "tcgen05_util.cuh"
#include "w4a16_layout.cuh"

using namespace ab2;
using namespace ab2::tc;

namespace ab2 {
int device_status_word(int **out);
int device_sm_count();
namespace {

constexpr int TC_STAGES = 4;          // operand-A (unpacked weight) stages of 64 K-elements
constexpr int TC_MAX_XSTAGES = 8;     // operand-B (activation) stages: a ring of its own, 128 KB deep, because an
                                      // activation tile takes about three stage times to arrive from L2
constexpr int TC_WSLOTS = 3;          // packed-weight ring slots (one quantisation group each)
constexpr int TC_BLOCK_WORDS = 272;   // 16 rows x 16 code words + 16 parameter words
constexpr int TC_WSLOT_BYTES = 8 * TC_BLOCK_WORDS * 4;  // 8 row tiles of 16 = 128 channels
constexpr int TC_A_BYTES = 128 * 128;  // 128 channels x 64 bf16
constexpr int TC_THREADS = 352;

struct TcShared {
    uint64_t wfull[TC_WSLOTS], wempty[TC_WSLOTS];
    uint64_t xfull[TC_MAX_XSTAGES], xempty[TC_MAX_XSTAGES], afull[TC_STAGES], sempty[TC_STAGES];
    uint64_t accfull[2], accempty[2];  // two accumulators: the epilogue of a tile overlaps the next tile's MMAs
    uint32_t tmem_base;
    int failed;
};

template <int NTOK>
__host__ __device__ constexpr int tc_xstages() {
    return NTOK > 128 ? TC_STAGES : TC_MAX_XSTAGES;
}

template <int NTOK>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_w4a16_tc_kernel(const uint32_t *__restrict__ wt, const __grid_constant__ CUtensorMap xmap,
                     __nv_bfloat16 *__restrict__ y, int N, int K, int M, int *status, int ksplit, float *part) {
    constexpr int B_BYTES = NTOK * 128;
    constexpr int XST = tc_xstages<NTOK>();
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) | ((128u >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *a_st = smem;                                   // [TC_STAGES][TC_A_BYTES]
    uint8_t *b_st = a_st + TC_STAGES * TC_A_BYTES;          // [XST][B_BYTES]
    uint8_t *w_ring = b_st + XST * B_BYTES;                 // [TC_WSLOTS][TC_WSLOT_BYTES]
    TcShared *sh = (TcShared *)(w_ring + TC_WSLOTS * TC_WSLOT_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = K >> 7, tiles16 = (N + 15) >> 4;
    const int n_tiles = (N + 127) >> 7, m_tiles = (M + NTOK - 1) / NTOK;
    // an item is (channel tile, token tile, K split): with fewer tiles than SMs the groups of a tile are
    // divided over `ksplit` CTAs, which leave f32 partial sums in `part` [ksplit][M][N] for a reduce pass
    const int items = n_tiles * m_tiles * ksplit;
#define TC_ITEM(it)                                                                    \
    const int ksp = (it) % ksplit, tile_ = (it) / ksplit;                              \
    const int nt = tile_ / m_tiles, mt = tile_ % m_tiles;                              \
    const int g0 = (int)((long long)ksp * G / ksplit), g1 = (int)((long long)(ksp + 1) * G / ksplit); \
    (void)ksp; (void)nt; (void)mt; (void)g0; (void)g1;
    volatile int *failed = &sh->failed;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_WSLOTS; ++i) { bar_init(&sh->wfull[i], 1); bar_init(&sh->wempty[i], 128); }
        for (int i = 0; i < TC_STAGES; ++i) { bar_init(&sh->afull[i], 128); bar_init(&sh->sempty[i], 1); }
        for (int i = 0; i < XST; ++i) { bar_init(&sh->xfull[i], 1); bar_init(&sh->xempty[i], 1); }
        for (int i = 0; i < 2; ++i) { bar_init(&sh->accfull[i], 1); bar_init(&sh->accempty[i], 4); }
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {  // tensor-memory allocation is a whole-warp operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(sptr(&sh->tmem_base)), "r"((uint32_t)(2 * NTOK)));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------- producer of the packed weights
        // One slot per quantisation group; lane b issues the bulk copy of block b, so the eight
        // copies of a group leave in parallel instead of one after the other from a single thread.
        uint32_t wuse = 0;
        for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x) {
            TC_ITEM(it)
            const int nblk = min(8, tiles16 - nt * 8);
            for (int g = g0; g < g1 && !*failed; ++g, ++wuse) {
                const int ws = wuse % TC_WSLOTS;
                int ok = 1;
                if (lane == 0) {
                    ok = bar_wait(&sh->wempty[ws], ((wuse / TC_WSLOTS) & 1) ^ 1, failed) ? 1 : 0;
                    if (ok) bar_expect_tx(&sh->wfull[ws], (uint32_t)nblk * TC_BLOCK_WORDS * 4);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < nblk)
                    bulk_copy(w_ring + ws * TC_WSLOT_BYTES + lane * TC_BLOCK_WORDS * 4,
                              wt + ((size_t)(nt * 8 + lane) * G + g) * TC_BLOCK_WORDS, TC_BLOCK_WORDS * 4, &sh->wfull[ws]);
            }
        }
    } else if (warp == TC_THREADS / 32 - 1) {
        // ---------------------------------------------------------- producer of the activation tiles
        if (lane == 0) {
            uint32_t suse = 0;
            for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x) {
                TC_ITEM(it)
                for (int ks = 2 * g0; ks < 2 * g1 && !*failed; ++ks, ++suse) {
                    const int xs = suse % XST;
                    // rings of equal depth share one "stage free" barrier (one commit per stage instead of two)
                    if (!bar_wait(XST == TC_STAGES ? &sh->sempty[xs] : &sh->xempty[xs], ((suse / XST) & 1) ^ 1, failed)) break;
                    bar_expect_tx(&sh->xfull[xs], B_BYTES);
                    tma_load_2d(b_st + xs * B_BYTES, &xmap, ks * 64, mt * NTOK, &sh->xfull[xs]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issue
        uint32_t suse = 0, tuse = 0;
        for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x, ++tuse) {
            const int ab = tuse & 1;
            if (!bar_wait(&sh->accempty[ab], ((tuse >> 1) & 1) ^ 1, failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t tacc = tmem + (uint32_t)(ab * NTOK);
            TC_ITEM(it)
            for (int ks = 2 * g0; ks < 2 * g1 && !*failed; ++ks, ++suse) {
                const int s = suse % TC_STAGES, xs = suse % XST;
                if (!bar_wait(&sh->xfull[xs], (suse / XST) & 1, failed)) break;
                if (!bar_wait(&sh->afull[s], (suse / TC_STAGES) & 1, failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (lane == 0) {
                    const uint32_t a0 = sptr(a_st + s * TC_A_BYTES), b0 = sptr(b_st + xs * B_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tacc, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), IDESC, ((ks - 2 * g0) | k) != 0);
                    umma_commit(&sh->sempty[s]);  // the operand stages are free when the MMAs retire
                    if (XST != TC_STAGES) umma_commit(&sh->xempty[xs]);
                }
                __syncwarp();
            }
            if (lane == 0) umma_commit(&sh->accfull[ab]);
            __syncwarp();
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------- dequantise
        const int t = threadIdx.x - 64;  // output channel within the 128-channel tile
        const int blk = t >> 4, r = t & 15;
        uint32_t wuse = 0, suse = 0;
        uint32_t k_mask = 0x000F000Fu, k_magic = 0x43004300u;
        asm volatile("" : "+r"(k_mask), "+r"(k_magic));
        for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x) {
            TC_ITEM(it)
            for (int g = g0; g < g1 && !*failed; ++g, ++wuse) {
                const int ws = wuse % TC_WSLOTS;
                if (!bar_wait(&sh->wfull[ws], (wuse / TC_WSLOTS) & 1, failed)) break;
                const uint32_t *bw = (const uint32_t *)(w_ring + ws * TC_WSLOT_BYTES) + blk * TC_BLOCK_WORDS;
                uint4 pw[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) pw[i] = *reinterpret_cast<const uint4 *>(bw + r * 16 + i * 4);
                const uint32_t pr = bw[256 + r];
                bar_arrive_after(&sh->wempty[ws], pw[0].x ^ pw[1].x ^ pw[2].x ^ pw[3].x ^ pr, (uint32_t)K & 1u);
                const uint32_t sc2 = __byte_perm(pr, pr, 0x1010);  // bf16x2 (scale, scale)
                const uint32_t nz2 = __byte_perm(pr, pr, 0x3232);  // bf16x2 -(128 + z)
#pragma unroll
                for (int half = 0; half < 2; ++half, ++suse) {
                    const int s = suse % TC_STAGES;
                    if (!bar_wait(&sh->sempty[s], ((suse / TC_STAGES) & 1) ^ 1, failed)) break;
                    uint8_t *arow = a_st + s * TC_A_BYTES + t * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {  // chunk c = 8 consecutive k = one code word
                        const uint4 q4 = pw[half * 2 + (c >> 2)];
                        const uint32_t word = (c & 3) == 0 ? q4.x : (c & 3) == 1 ? q4.y : (c & 3) == 2 ? q4.z : q4.w;
                        uint32_t o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t v;
                            const uint32_t shv = j ? (word >> (4 * j)) : word;
                            asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(v) : "r"(shv), "r"(k_mask), "r"(k_magic));
                            o[j] = bf16x2_mul_(bf16x2_add_(v, nz2), sc2);
                        }
                        *reinterpret_cast<uint4 *>(arow + ((c ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    bar_arrive(&sh->afull[s]);
                }
            }
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------- epilogue
        const int quad = warp & 3;
        uint32_t tuse = 0;
        for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x, ++tuse) {
            TC_ITEM(it)
            const int ab = tuse & 1;
            if (!bar_wait(&sh->accfull[ab], (tuse >> 1) & 1, failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int n = nt * 128 + quad * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < NTOK / 32; ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ab * NTOK + c * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (n < N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int tok = mt * NTOK + c * 32 + j;
                        if (tok < M) {
                            if (ksplit > 1) part[((size_t)ksp * M + tok) * N + n] = __uint_as_float(v[j]);
                            else y[(size_t)tok * N + n] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(&sh->accempty[ab]);
        }
    }

    // ---- teardown: every warp arrives here (all waits are bounded)
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && sh->failed) atomicExch(status, (int)AB2_ERR_TIMEOUT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((uint32_t)(2 * NTOK)));
    }
}

// y[i] = bf16(sum over splits of part[s][i]): eight elements per thread
__global__ void splitk_reduce_kernel(const float *__restrict__ part, __nv_bfloat16 *__restrict__ y, size_t n8, size_t stride, int ksplit) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < ksplit; ++s) {
        const float4 a = reinterpret_cast<const float4 *>(part + s * stride)[2 * i];
        const float4 b = reinterpret_cast<const float4 *>(part + s * stride)[2 * i + 1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        o[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * j])) |
               ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * j + 1])) << 16);
    reinterpret_cast<uint4 *>(y)[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// Workspace of the K split, one per device, grown on demand (prefill passes are not captured in graphs;
// a capture in progress simply runs without the split).
constexpr size_t TC_SPLIT_MAX_BYTES = (size_t)128 << 20;
static float *g_split_ws[64] = {nullptr};
static size_t g_split_bytes[64] = {0};
static float *split_workspace(int dev, size_t bytes, cudaStream_t s) {
    if (g_split_bytes[dev] >= bytes) return g_split_ws[dev];
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    if (cudaDeviceSynchronize() != cudaSuccess) return nullptr;
    if (g_split_ws[dev]) cudaFree(g_split_ws[dev]);
    g_split_ws[dev] = nullptr;
    g_split_bytes[dev] = 0;
    if (cudaMalloc((void **)&g_split_ws[dev], bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    g_split_bytes[dev] = bytes;
    return g_split_ws[dev];
}

template <int NTOK>
int launch_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    CUtensorMap map;
    rc = make_x_map(&map, x, M, w->K, NTOK);
    if (rc != AB2_OK) return rc;
    const size_t smem = 1024 + TC_STAGES * TC_A_BYTES + tc_xstages<NTOK>() * NTOK * 128 + TC_WSLOTS * TC_WSLOT_BYTES + sizeof(TcShared);
    static bool configured[64] = {false};  // the attribute is per device
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!configured[dev]) {
        AB2_CUDA(cudaFuncSetAttribute(gemm_w4a16_tc_kernel<NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = true;
    }
    const int tiles = ((w->N + 127) / 128) * ((M + NTOK - 1) / NTOK);
    // Fewer tiles than about half the SMs: split K so that the machine is busy (512 tokens on the
    // 14336 x 4096 weight are 64 tiles of 256 tokens).  The sums of the splits are f32; one rounding.
    const int sms = device_sm_count(), G = w->K / 128;
    int ksplit = 1;
    float *part = nullptr;
    static const bool no_split = getenv("AB2_GEMM_NO_SPLITK") != nullptr;
    if (!no_split && tiles * 2 <= sms + sms / 4 && G >= 8 && w->N % 8 == 0) {
        ksplit = std::max(1, std::min(4, std::min(G / 4, sms / tiles)));  // all items in one wave
        const size_t bytes = (size_t)ksplit * M * w->N * sizeof(float);
        part = ksplit > 1 && bytes <= TC_SPLIT_MAX_BYTES ? split_workspace(dev, bytes, s) : nullptr;
        if (!part) ksplit = 1;
    }
    const int items = tiles * ksplit;
    const int grid = std::min(items, sms);
    gemm_w4a16_tc_kernel<NTOK><<<grid, TC_THREADS, smem, s>>>((const uint32_t *)w->codes, map, (__nv_bfloat16 *)y, w->N, w->K, M, status, ksplit, part);
    AB2_LAUNCH_CHECK();
    if (ksplit > 1) {
        const size_t n8 = (size_t)M * w->N / 8;
        splitk_reduce_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, s>>>(part, (__nv_bfloat16 *)y, n8, (size_t)M * w->N, ksplit);
        AB2_LAUNCH_CHECK();
    }
    return AB2_OK;
}

}  // namespace

// Y[M][N] = X[M][K] . W^T on the tcgen05 path (W4A16, group 128, bf16).
int qlinear_w4a16_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    AB2_REQUIRE(((uintptr_t)x & 15) == 0 && (w->K * 2) % 16 == 0, AB2_ERR_BAD_ALIGN, "activations must be 16-byte aligned");
    if (M <= 48) return launch_tc<32>(w, x, M, y, s);
    // From 257 tokens on, 256-token tiles: an unpacked weight stage then feeds twice the MMA work, which
    // is what bounds the kernel at 128 (512 tokens on the 4096 x 28672 weight: 139 against 228 us), even
    // where fewer tiles than SMs remain (4096 x 4096 at 512 tokens: 45 against 43 us).
    if (M <= 256) return launch_tc<128>(w, x, M, y, s);
    return launch_tc<256>(w, x, M, y, s);
}

}  // namespace ab2
