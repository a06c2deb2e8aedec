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
#include "common.cuh"
#include <cuda.h>

namespace {
constexpr int BM = 128;
constexpr int BK = 64;                       // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int SPIN_LIMIT = 1 << 22;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    for (int i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// x = element index along K (a multiple of 8: the copy starts on a 16-byte boundary), y = row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc5_alloc(unsigned* smem_result, unsigned ncols) {          // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc5_dealloc(unsigned taddr, unsigned ncols) {              // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc5_mma(unsigned tmem_c, unsigned long long adesc, unsigned long long bdesc,
                                        unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the mbarrier once every tcgen05 operation this thread issued before has completed
__device__ __forceinline__ void tc5_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc5_ld32(unsigned taddr, unsigned (&r)[32]) {              // 32 lanes x 32 columns
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16) with the
// 128-byte swizzle: 8 rows make one 1024-byte swizzle atom, atoms follow each other along M/N.
//   bits  0-13  start address >> 4          bits 16-29  leading byte offset >> 4 (unused here)
//   bits 32-45  stride byte offset >> 4 = 1024 >> 4 (from one 8-row atom to the next)
//   bits 46-47  descriptor version 1        bits 61-63  swizzle mode, 2 = 128 bytes
__device__ __forceinline__ unsigned long long make_smem_desc(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3ffff) >> 4);
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// Instruction descriptor of kind::f16: float32 accumulator (bits 4-5 = 1), bfloat16 A and B
// (bits 7-9 and 10-12 = 1), both K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in 24-28.
__host__ __device__ constexpr unsigned make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
}  // namespace

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
    if (warp == 1) tc5_alloc(&tmem_base_slot, 2 * BN);       // two accumulators; 2 * BN is a power of two >= 32
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const unsigned tmem_base = tmem_base_slot;
    pdl_launch_dependents();
    pdl_wait();                                              // A is written by the kernel before

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
                        atomicExch(&failed, 1);
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
                    atomicExch(&failed, 1);
                    break;
                }
                tc5_fence_after();
                const unsigned tmem_c = tmem_base + (unsigned)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(&full_bar[s], (unsigned)((it / STAGES) & 1))) {
                        atomicExch(&failed, 1);
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
                atomicExch(&failed, 1);
                break;
            }
            tc5_fence_after();
            int m0, n0;
            tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
            const int row = m0 + quarter * 32 + lane;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned v[32];
                tc5_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), v);
                if (row < M && swiglu) {
                    // 32 columns = two blocks of 8 gate and 8 up columns -> 16 columns of C at (n0 + c0) / 2
                    TO* dst = C + (size_t)row * ldc + (n0 + c0) / 2;
#pragma unroll
                    for (int blk = 0; blk < 2; ++blk) {
                        if (n0 + c0 + 16 * blk + 16 <= N) {
                            float o[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float gt = __uint_as_float(v[16 * blk + i]), up = __uint_as_float(v[16 * blk + 8 + i]);
                                o[i] = gt / (1.0f + __expf(-gt)) * up;
                            }
                            if constexpr (sizeof(TO) == 2) {
                                uint4 q;
                                unsigned* w = reinterpret_cast<unsigned*>(&q);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    __nv_bfloat162 p = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
                                    w[i] = *reinterpret_cast<unsigned*>(&p);
                                }
                                if ((((uintptr_t)(dst + 8 * blk)) & 15) == 0) {
                                    *reinterpret_cast<uint4*>(dst + 8 * blk) = q;
                                } else {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) dst[8 * blk + i] = from_f32<TO>(o[i]);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i) dst[8 * blk + i] = from_f32<TO>(o[i]);
                            }
                        }
                    }
                } else if (row < M) {
                    TO* dst = C + (size_t)row * ldc + n0 + c0;
                    if (n0 + c0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
                        if constexpr (sizeof(TO) == 2) {
                            uint4 q[4];
                            unsigned* w = reinterpret_cast<unsigned*>(q);
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                                w[i] = *reinterpret_cast<unsigned*>(&p);
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst)[i] = q[i];
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                        }
                    } else {
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c0 + i < N) dst[i] = from_f32<TO>(__uint_as_float(v[i]));
                    }
                }
            }
            tc5_fence_before();
            mbar_arrive(&acc_empty_bar[acc]);                // 128 arrivals hand the accumulator back
        }
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    if (warp == 1) tc5_dealloc(tmem_base, 2 * BN);
    if (threadIdx.x == 0 && failed && err) atomicOr(err, VL_DEV_WAIT_EXPIRED);
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld elements; boxes of box_rows x 64 elements, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return VL_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VL_ERR_ARGUMENT;
}

template <int BN, int STAGES, typename TO>
static int launch_tc5(const void* A, const void* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                      unsigned* err, int swiglu, cudaStream_t s) {
    CUtensorMap map_a, map_w;
    int rc = make_map(&map_a, A, M, K, lda, BM);
    if (rc) return rc;
    rc = make_map(&map_w, W, N, K, ldw, BN);
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
