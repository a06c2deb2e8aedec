// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05, accumulators in TMEM):
//     C[M,N] = A[M,K] * W[N,K]^T,   float32 accumulation, C bfloat16 or float32
// (a linear layer y = x W^T with the weight stored [out, in], no bias), for the many rows of a
// prompt portion.  Few rows (decoding) go to csrc/gemm_bf16.cu, which is built around the weight
// stream instead.
//
// A block computes 128 x BN tiles of C, one after the other (one block per SM).  Roles:
//   warp 0, one thread   TMA producer: tiled bulk tensor copies (cp.async.bulk.tensor.2d, 128-byte
//                        swizzle) of a 128 x 64 tile of A and a BN x 64 tile of W per stage into a
//                        ring of shared-memory stages, completion on an mbarrier per stage;
//   warp 1, one thread   issues tcgen05.mma (cta_group::1, kind::f16, M 128, N BN, K 16) on shared
//                        memory descriptors, 4 per stage; tcgen05.commit hands the stage back to
//                        the producer and, after the last one, signals the epilogue;
//                        the warp also allocates and frees 2 x BN columns of TMEM: two accumulators,
//                        so that the products of the next tile run during the epilogue of this one;
//   warps 2..5           epilogue: tcgen05.ld of the accumulator (a warp reads the 32 TMEM lanes
//                        of its quarter), conversion, stores of the rows that exist.
// Rows beyond M or N and columns beyond K are zero-filled by the TMA unit, so any M and N are
// taken; K must be a multiple of 8 (16-byte rows).  With swiglu != 0, W holds blocks of 8 gate rows
// followed by their 8 up rows and the epilogue writes C[m, 8b + i] = silu(y[m, 16b + i]) * y[m, 16b + 8 + i]
// into a [M, N/2] matrix.  Every wait on an mbarrier is bounded: when one
// expires the block records VL_DEV_WAIT_EXPIRED, stops, and still frees its TMEM.
#include "tc5.cuh"

namespace {
constexpr int BM = 128;
constexpr int BK = 64;                       // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;

}  // namespace
using namespace tc5;

// Tile number -> corner of the tile.  Blocks that run at the same time should share tiles of W
// (and of A) in L2: consecutive numbers walk down a band of up to 16 tiles of M before they move on
// to the next tile of N.
template <int BN>
__device__ __forceinline__ void tile_corner(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
    constexpr int BAND = 16;
    const int band = tile / (BAND * tiles_n), in_band = tile - band * BAND * tiles_n;
    const int band_rows = min(BAND, tiles_m - band * BAND);
    m0 = (band * BAND + in_band % band_rows) * BM;
    n0 = (in_band / band_rows) * BN;
}

// Persistent: a block takes the tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The ring of stages
// runs on across tiles, and TMEM holds two accumulators, so the epilogue of one tile overlaps the
// products of the next.
template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                TO* __restrict__ C, int M, int N, int K, int ldc, unsigned* err, int tiles_m, int tiles_n, int swiglu) {
    constexpr unsigned A_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    extern __shared__ unsigned char tc5_smem_raw[];
    // tiles of the 128-byte swizzle must start on 1024-byte boundaries
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc5_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BK - 1) / BK;
    const int total_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full_bar[i], 1); mbar_init(&acc_empty_bar[i], 128); }
        mbar_fence_init();
        failed = 0;
    }
    // Tensor memory is taken only after the kernels before this one have completed: a block started as a
    // programmatic dependent then holds nothing of the SM that an earlier kernel may still be waiting for.
    pdl_launch_dependents();
    pdl_wait();                                              // A is written by the kernel before
    if (warp == 1) tc5_alloc(&tmem_base_slot, 2 * BN);       // two accumulators; 2 * BN is a power of two >= 32
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                     // ---- TMA producer ----
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int m0, n0;
                tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait_bounded(&empty_bar[s], (unsigned)((it / STAGES - 1) & 1))) {
                        atomicOr(&failed, 1);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
                    unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    tma_load_2d(st, &map_a, kb * BK, m0, &full_bar[s]);
                    tma_load_2d(st + A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                     // ---- MMA issuer ----
            constexpr unsigned idesc = make_idesc(BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                if (local >= 2 && !mbar_wait_bounded(&acc_empty_bar[acc], (unsigned)((local / 2 - 1) & 1))) {
                    atomicOr(&failed, 2);
                    break;
                }
                tc5_fence_after();
                const unsigned tmem_c = tmem_base + (unsigned)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(&full_bar[s], (unsigned)((it / STAGES) & 1))) {
                        atomicOr(&failed, 4);
                        ok = false;
                        break;
                    }
                    tc5_fence_after();
                    const unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    const unsigned long long adesc = make_smem_desc(st), bdesc = make_smem_desc(st + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 columns of K further on: 32 bytes inside the swizzled row, i.e. +2 in the address field
                        tc5_mma(tmem_c, adesc + (unsigned long long)(k * 2), bdesc + (unsigned long long)(k * 2), idesc,
                                (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc5_commit(&empty_bar[s]);               // the stage is free once these MMAs have read it
                }
                if (ok) tc5_commit(&acc_full_bar[acc]);      // this accumulator is complete
            }
        }
    } else {                                                 // ---- epilogue: warps 2..5 ----
        const int quarter = warp & 3;                        // the TMEM lanes this warp may read
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            if (!mbar_wait_bounded(&acc_full_bar[acc], (unsigned)((local / 2) & 1))) {
                atomicOr(&failed, 8);
                break;
            }
            tc5_fence_after();
            int m0, n0;
            tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
            const int row = m0 + quarter * 32 + lane;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned v[32];
                tc5_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), v);
                if (row < M) store_chunk32<TO>(v, C + (size_t)row * ldc, n0 + c0, N, swiglu);
            }
            tc5_fence_before();
            mbar_arrive(&acc_empty_bar[acc]);                // 128 arrivals hand the accumulator back
        }
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    if (warp == 1) tc5_dealloc(tmem_base, 2 * BN);
    if (threadIdx.x == 0 && failed && err)
        atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_GEMM_TC5 | ((unsigned)failed << VL_DEV_ROLE_SHIFT));
}

// ---- host side -------------------------------------------------------------------------------
template <int BN, int STAGES, typename TO>
static int launch_tc5(const void* A, const void* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                      unsigned* err, int swiglu, cudaStream_t s) {
    CUtensorMap map_a, map_w;
    int rc = tc5_make_map(&map_a, A, M, K, lda, BM);
    if (rc) return rc;
    rc = tc5_make_map(&map_w, W, N, K, ldw, BN);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (BM + BN) * BK * 2 + 1024;
    auto kern = gemm_tc5_kernel<BN, STAGES, TO>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    const int total = tiles_m * tiles_n;
    dim3 grid(total < num_sms ? total : num_sms);             // one block per SM; blocks walk the tiles
    return vl_launch(kern, grid, dim3(NUM_THREADS), smem, s, map_a, map_w, C, M, N, K, ldc, err, tiles_m, tiles_n, swiglu);
}

// Width of the tiles: 256, or 128 when N is no wider.  (Narrower tiles spread few rows over more SMs
// but re-read A once per tile of N; measured slower, so products of few hundred rows are not this
// kernel's business.)
template <typename TO>
static int dispatch_tc5(const void* A, const void* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                        unsigned* err, int swiglu, cudaStream_t s) {
    if (N > 128) return launch_tc5<256, 4, TO>(A, W, C, M, N, K, lda, ldw, ldc, err, swiglu, s);
    return launch_tc5<128, 6, TO>(A, W, C, M, N, K, lda, ldw, ldc, err, swiglu, s);
}

extern "C" int vl_gemm_bf16_tc5(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K,
                                int lda, int ldw, int ldc, unsigned* err, int swiglu, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) return VL_ERR_UNSUPPORTED;
    if (swiglu ? (N % 16 || ldc < N / 2) : ldc < N) return VL_ERR_ARGUMENT;
    if (lda < K || ldw < K) return VL_ERR_ARGUMENT;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return VL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == VL_BF16) return dispatch_tc5<bf16>(A, W, (bf16*)C, M, N, K, lda, ldw, ldc, err, swiglu, s);
    if (out_dtype == VL_F32) return dispatch_tc5<float>(A, W, (float*)C, M, N, K, lda, ldw, ldc, err, swiglu, s);
    return VL_ERR_UNSUPPORTED;
}
