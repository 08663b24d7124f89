// W8A16 GEMM for many tokens (prefill) on the 5th-generation tensor cores: INT8 symmetric
// weights with one f32 scale per output channel (per-output-channel absmax,
// crates/aarambh-studio-quant/src/qat.rs:140-169; a per-tensor scale, absmax.rs:7-24, is the same
// with the scale replicated; the reference dequantises such weights at load,
// crates/aarambh-studio-weights/src/gguf.rs:187-212, and multiplies dense), bf16 activations.
//
//   Y[M, N] = X[M, K] . W^T,   W = codes[N][K] (int8, row-major) * scale[N]
//
// Same skeleton as the W4A16 kernel (gemm_w4a16_tc.cu): the 128 output channels of a tile are the
// M dimension of tcgen05.mma, the tokens its N dimension, one persistent CTA per SM with
// specialised warps.  What differs:
//   warp 0      one lane loads a 128-channel x 128-K tile of codes per ring slot with one TMA
//               tile copy (128-byte swizzle, so that the row-per-thread reads below do not
//               collide on shared-memory banks)
//   warps 2-9   two threads per channel turn 32 codes each into bf16 per stage: a byte b is
//               b + 128 after one XOR, PRMT puts it under the exponent of 2^23, one subtract
//               gives float(b) exactly, and since |b| <= 127 needs at most 7 significant bits the
//               bf16 is the upper half of that float (one PRMT per pair).  The codes enter the
//               MMA unscaled and exact;
//   warps 10-13 the epilogue multiplies the f32 accumulator by the channel's f32 scale - the
//               product is rounded once, where the reference rounds q * scale to the model
//               dtype before its matmul.
// Every wait on an mbarrier is bounded; on a time-out the CTA records AB2_ERR_TIMEOUT, stops
// issuing work, still frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "tcgen05_util.cuh"

using namespace ab2;
using namespace ab2::tc;

namespace ab2 {
int device_status_word(int **out);
int device_sm_count();
namespace {

constexpr int TC_STAGES = 4;          // operand-A (unpacked weight) stages of 64 K-elements
constexpr int TC_MAX_XSTAGES = 6;     // operand-B (activation) stages: a ring of its own, 128 KB deep, because an
                                      // activation tile takes about three stage times to arrive from L2
constexpr int TC_WSLOTS = 2;          // code ring slots (128 channels x 128 K, 16 KB each)
constexpr int TC_WSLOT_BYTES = 128 * 128;  // 128 channels x 128 codes
constexpr int TC_A_BYTES = 128 * 128;  // 128 channels x 64 bf16
constexpr int TC_THREADS = 480;  // 1 weight producer, 1 MMA, 8 convert, 4 epilogue, 1 activation producer

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
gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap wmap, const float *__restrict__ scales,
                  const __grid_constant__ CUtensorMap xmap, __nv_bfloat16 *__restrict__ y, int N, int K, int M, int *status) {
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
    const int G = K >> 7;
    const int n_tiles = (N + 127) >> 7, m_tiles = (M + NTOK - 1) / NTOK;
    const int items = n_tiles * m_tiles;
    volatile int *failed = &sh->failed;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_WSLOTS; ++i) { bar_init(&sh->wfull[i], 1); bar_init(&sh->wempty[i], 256); }
        for (int i = 0; i < TC_STAGES; ++i) { bar_init(&sh->afull[i], 256); bar_init(&sh->sempty[i], 1); }
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
        // ---------------------------------------------------------- producer of the codes
        if (lane == 0) {
            uint32_t wuse = 0;
            for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x) {
                const int nt = it / m_tiles;
                for (int g = 0; g < G && !*failed; ++g, ++wuse) {
                    const int ws = wuse % TC_WSLOTS;
                    if (!bar_wait(&sh->wempty[ws], ((wuse / TC_WSLOTS) & 1) ^ 1, failed)) break;
                    bar_expect_tx(&sh->wfull[ws], TC_WSLOT_BYTES);  // rows past N arrive as zeros and count
                    tma_load_2d(w_ring + ws * TC_WSLOT_BYTES, &wmap, g * 128, nt * 128, &sh->wfull[ws]);
                }
            }
        }
    } else if (warp == TC_THREADS / 32 - 1) {
        // ---------------------------------------------------------- producer of the activation tiles
        if (lane == 0) {
            uint32_t suse = 0;
            for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x) {
                const int mt = it % m_tiles;
                for (int ks = 0; ks < 2 * G && !*failed; ++ks, ++suse) {
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
            for (int ks = 0; ks < 2 * G && !*failed; ++ks, ++suse) {
                const int s = suse % TC_STAGES, xs = suse % XST;
                if (!bar_wait(&sh->xfull[xs], (suse / XST) & 1, failed)) break;
                if (!bar_wait(&sh->afull[s], (suse / TC_STAGES) & 1, failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (lane == 0) {
                    const uint32_t a0 = sptr(a_st + s * TC_A_BYTES), b0 = sptr(b_st + xs * B_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tacc, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), IDESC, (ks | k) != 0);
                    umma_commit(&sh->sempty[s]);  // the operand stages are free when the MMAs retire
                    if (XST != TC_STAGES) umma_commit(&sh->xempty[xs]);
                }
                __syncwarp();
            }
            if (lane == 0) umma_commit(&sh->accfull[ab]);
            __syncwarp();
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------- codes -> bf16
        const int u = threadIdx.x - 64;    // 0..255
        const int t = u & 127;             // output channel within the 128-channel tile
        const int hsel = u >> 7;           // which 32 of a stage's 64 K-elements this thread converts
        uint32_t wuse = 0, suse = 0;
        for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x) {
            for (int g = 0; g < G && !*failed; ++g, ++wuse) {
                const int ws = wuse % TC_WSLOTS;
                if (!bar_wait(&sh->wfull[ws], (wuse / TC_WSLOTS) & 1, failed)) break;
                // row t of the slot: 128 codes in eight 16-byte chunks, chunk c stored at c ^ (t & 7)
                const uint8_t *wrow = w_ring + ws * TC_WSLOT_BYTES + t * 128;
                uint4 raw[2][2];
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        raw[half][i] = *reinterpret_cast<const uint4 *>(wrow + (((4 * half + 2 * hsel + i) ^ (t & 7)) << 4));
                bar_arrive_after(&sh->wempty[ws], raw[0][0].x ^ raw[0][1].x ^ raw[1][0].x ^ raw[1][1].x, (uint32_t)K & 1u);
#pragma unroll
                for (int half = 0; half < 2; ++half, ++suse) {
                    const int s = suse % TC_STAGES;
                    if (!bar_wait(&sh->sempty[s], ((suse / TC_STAGES) & 1) ^ 1, failed)) break;
                    uint8_t *arow = a_st + s * TC_A_BYTES + t * 128;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {  // 16 codes -> two chunks of 8 bf16
                        const uint32_t w4[4] = {raw[half][i].x, raw[half][i].y, raw[half][i].z, raw[half][i].w};
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t ub = w4[j] ^ 0x80808080u;  // b + 128 as unsigned bytes
                            const float f0 = __uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7540)) - 8388736.0f;
                            const float f1 = __uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7541)) - 8388736.0f;
                            const float f2 = __uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7542)) - 8388736.0f;
                            const float f3 = __uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7543)) - 8388736.0f;
                            // exact small integers: the bf16 is the upper half of the float
                            o[2 * j] = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
                            o[2 * j + 1] = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
                        }
                        const int oc = 4 * hsel + 2 * i;  // chunk = 8 consecutive k of the stage row
                        *reinterpret_cast<uint4 *>(arow + ((oc ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4 *>(arow + (((oc + 1) ^ (t & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    bar_arrive(&sh->afull[s]);
                }
            }
        }
    } else if (warp < 14) {
        // ---------------------------------------------------------- epilogue
        const int quad = warp & 3;
        uint32_t tuse = 0;
        for (int it = blockIdx.x; it < items && !*failed; it += gridDim.x, ++tuse) {
            const int nt = it / m_tiles, mt = it % m_tiles;
            const int ab = tuse & 1;
            if (!bar_wait(&sh->accfull[ab], (tuse >> 1) & 1, failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int n = nt * 128 + quad * 32 + lane;
            const float sc = n < N ? __ldg(scales + n) : 0.f;
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
                        if (tok < M) y[(size_t)tok * N + n] = __float2bfloat16_rn(__uint_as_float(v[j]) * sc);
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

// Tensor map of the codes: [N][K] bytes, tiles of 128 K x 128 channels, 128-byte swizzle.
static int make_w8_map(CUtensorMap *map, const void *codes, int N, int K) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        AB2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        AB2_REQUIRE(fn != nullptr && qres == cudaDriverEntryPointSuccess, AB2_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is unavailable");
        encode = (EncodeTiledFn)fn;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(codes), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    AB2_REQUIRE(r == CUDA_SUCCESS, AB2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return AB2_OK;
}

template <int NTOK>
int launch_i8_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    int *status = nullptr;
    int rc = device_status_word(&status);
    if (rc != AB2_OK) return rc;
    CUtensorMap xmap, wmap;
    rc = make_x_map(&xmap, x, M, w->K, NTOK);
    if (rc != AB2_OK) return rc;
    rc = make_w8_map(&wmap, w->codes, w->N, w->K);
    if (rc != AB2_OK) return rc;
    const size_t smem = 1024 + TC_STAGES * TC_A_BYTES + tc_xstages<NTOK>() * NTOK * 128 + TC_WSLOTS * TC_WSLOT_BYTES + sizeof(TcShared);
    static bool configured[64] = {false};  // the attribute is per device
    int dev = 0;
    AB2_CUDA(cudaGetDevice(&dev));
    AB2_REQUIRE(dev >= 0 && dev < 64, AB2_ERR_BAD_ARG, "device index %d out of range", dev);
    if (!configured[dev]) {
        AB2_CUDA(cudaFuncSetAttribute(gemm_i8_tc_kernel<NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = true;
    }
    const int items = ((w->N + 127) / 128) * ((M + NTOK - 1) / NTOK);
    const int grid = std::min(items, device_sm_count());
    gemm_i8_tc_kernel<NTOK><<<grid, TC_THREADS, smem, s>>>(wmap, (const float *)w->scales, xmap, (__nv_bfloat16 *)y, w->N, w->K, M, status);
    AB2_LAUNCH_CHECK();
    return AB2_OK;
}

}  // namespace

// Whether the tensor-core path serves this weight and token count: INT8 codes whose rows start on
// 16-byte boundaries, K in whole 128-element slots.
bool qlinear_i8_tc_eligible(const ab2_qweight *w, ab2_dtype dtype, int M) {
    return w->fmt == FMT_I8 && dtype == AB2_BF16 && M > 8 && w->K % 128 == 0 && ((uintptr_t)w->codes & 15) == 0;
}

// Y[M][N] = X[M][K] . W^T on the tcgen05 path (INT8 codes, f32 scale per channel, bf16 activations).
int qlinear_i8_tc(const ab2_qweight *w, const void *x, int M, void *y, cudaStream_t s) {
    AB2_REQUIRE(((uintptr_t)x & 15) == 0, AB2_ERR_BAD_ALIGN, "activations must be 16-byte aligned");
    if (M <= 256) return launch_i8_tc<128>(w, x, M, y, s);  // as for the W4A16 GEMM: 256-token tiles from 257 tokens on
    return launch_i8_tc<256>(w, x, M, y, s);
}

}  // namespace ab2
