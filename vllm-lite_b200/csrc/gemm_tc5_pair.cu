// bfloat16 matrix product on the 5th-generation tensor cores with two SMs on one tile
// (tcgen05.mma.cta_group::2):   C[M,N] = A[M,K] * W[N,K]^T,  float32 accumulation.
//
// csrc/gemm_tc5.cu computes a 128 x 256 tile per SM and has to bring 128 rows of A and 256 rows of
// W into shared memory for it: 48 KB per 64 columns of K, and that traffic, not the tensor cores,
// bounds it.  Here a cluster of two blocks (one SM each) computes a 256 x 256 tile together: each
// block brings its own 128 rows of A and only its half of the 256 rows of W (32 KB per 64 columns
// of K), the tensor cores of both SMs read W from both halves, and each block keeps the 128 rows of
// the accumulator that belong to its rows of A in its own TMEM.
//
// Roles in each block of the pair:
//   warp 0, one thread   TMA producer: its rows of A and its half of W, stage by stage
//                        (cp.async.bulk.tensor.2d, 128-byte swizzle; the copies of both blocks
//                        complete on the mbarrier of the pair's first block);
//   warp 1, one thread   first block only: waits for a stage of both blocks, issues the pair's
//                        MMAs (M 256, N 256, K 16, four per stage); tcgen05.commit with multicast
//                        hands the stage back to both producers and, after a tile's last product,
//                        tells both epilogues; the warp of either block allocates and frees TMEM
//                        (512 columns: two accumulators, so that a tile's products run during the
//                        epilogue of the tile before);
//   warps 2..5           epilogue of the block's 128 rows, as in csrc/gemm_tc5.cu; when done they
//                        arrive on the first block's mbarrier (256 arrivals free an accumulator).
// Any M and N (the TMA unit fills what lies outside with zeros), K a multiple of 8.  Every wait on
// an mbarrier is bounded: when one expires the block records VL_DEV_WAIT_EXPIRED, stops, and
// still joins the pair's last barrier and frees its TMEM.
#include "tc5.cuh"

using namespace tc5;

namespace {
constexpr int BM_CTA = 128, BM = 256, BK = 64, UMMA_K = 16;
constexpr int BN_MMA = 256, BN_CTA = 128;    // one product: 256 columns of the tile, 128 rows of W from each block
constexpr int NUM_THREADS = 192;
constexpr unsigned A_BYTES = BM_CTA * BK * 2, W_BYTES = BN_CTA * BK * 2;
constexpr unsigned TMEM_COLS = 512;

// The tile's width.  256: two accumulators in TMEM, 6 stages of 32 KB; a stage feeds 512 cycles of the tensor
// core with 32 KB, more than an SM takes in (about 52 bytes a cycle), so the tensor pipe is busy 74 to 83 % of
// a tile's time.  512: one accumulator of all 512 columns, 4 stages of 48 KB (A once for two products per 16
// columns of K): 48 KB per 1,024 cycles, the tensor pipe no longer waits, but the epilogue of a tile no
// longer runs beside the products of the next.  The launcher picks by the rounds of tiles either needs.
template <int BN> struct Shape {
    static constexpr int HALVES = BN / BN_MMA;                                 // products per 16 columns of K
    static constexpr int STAGES = BN == 256 ? 6 : 4;
    static constexpr int ACCS = BN == 256 ? 2 : 1;                              // accumulators in TMEM
    static constexpr unsigned STAGE_BYTES = A_BYTES + HALVES * W_BYTES;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of the same variable in block `rank` of the cluster
__device__ __forceinline__ unsigned map_to_rank(unsigned local_addr, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// a copy into this block's shared memory that completes on an mbarrier of the pair (cluster address)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void alloc_pair(unsigned* smem_result, unsigned ncols) {            // a warp of either block
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void dealloc_pair(unsigned taddr, unsigned ncols) {                 // a warp of either block
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_pair(unsigned tmem_c, unsigned long long adesc, unsigned long long bdesc,
                                         unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once every MMA issued so far has completed, on the mbarrier at this address in both blocks
__device__ __forceinline__ void commit_pair(unsigned long long* bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int BN>
__device__ __forceinline__ void tile_corner(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
    constexpr int BAND = 8;                                  // pairs that run together share tiles of W in L2
    const int band = tile / (BAND * tiles_n), in_band = tile - band * BAND * tiles_n;
    const int band_rows = min(BAND, tiles_m - band * BAND);
    m0 = (band * BAND + in_band % band_rows) * BM;
    n0 = (in_band / band_rows) * BN;
}
}  // namespace

template <typename TO, int BN>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc5_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     TO* __restrict__ C, int M, int N, int K, int ldc, unsigned* err, int tiles_m, int tiles_n, int swiglu) {
    constexpr int STAGES = Shape<BN>::STAGES, ACCS = Shape<BN>::ACCS, HALVES = Shape<BN>::HALVES;
    constexpr unsigned STAGE_BYTES = Shape<BN>::STAGE_BYTES;
    extern __shared__ unsigned char pair_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)pair_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();                    // 0: the block that issues the pair's products
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int k_blocks = (K + BK - 1) / BK;
    const int total_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        for (int i = 0; i < ACCS; ++i) { mbar_init(&acc_full_bar[i], 1); mbar_init(&acc_empty_bar[i], 2 * 128); }
        mbar_fence_init();
        failed = 0;
    }
    // This kernel is never launched as a programmatic dependent (see launch_pair), so both calls below do
    // nothing today.  They stay ahead of everything that takes a shared resource of the SM pair (tensor
    // memory, the cluster's barrier): were the attribute ever given, nothing would be held while earlier
    // kernels of the stream still run.
    pdl_wait();                                              // A is written by the kernel before
    pdl_launch_dependents();
    if (warp == 1) alloc_pair(&tmem_base_slot, TMEM_COLS);
    tc5_fence_before();
    __syncthreads();
    cluster_sync();                                          // the other block's mbarriers exist before anything arrives there
    tc5_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                     // ---- TMA producer ----
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
                int m0, n0;
                tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait_bounded(&empty_bar[s], (unsigned)((it / STAGES - 1) & 1))) {
                        atomicOr(&failed, 1);
                        ok = false;
                        break;
                    }
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);       // the bytes of both blocks
                    const unsigned bar = map_to_rank(smem_u32(&full_bar[s]), 0);
                    unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    tma_load_2d_pair(st, &map_a, kb * BK, m0 + (int)rank * BM_CTA, bar);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)     // this block's 128 rows of W for each product of 256 columns
                        tma_load_2d_pair(st + A_BYTES + h * W_BYTES, &map_w, kb * BK, n0 + h * BN_MMA + (int)rank * BN_CTA, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                        // ---- MMA issuer of the pair ----
            constexpr unsigned idesc = make_idesc(BM, BN_MMA);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++local) {
                const int acc = local % ACCS;
                if (local >= ACCS && !mbar_wait_bounded(&acc_empty_bar[acc], (unsigned)((local / ACCS - 1) & 1))) {
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
                    const unsigned long long adesc = make_smem_desc(st);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        const unsigned long long bdesc = make_smem_desc(st + A_BYTES + h * W_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            mma_pair(tmem_c + (unsigned)(h * BN_MMA), adesc + (unsigned long long)(k * 2),
                                     bdesc + (unsigned long long)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    commit_pair(&empty_bar[s]);              // both blocks' stages are free once these MMAs have read them
                }
                if (ok) commit_pair(&acc_full_bar[acc]);     // both halves of this accumulator are complete
            }
        }
    } else {                                                 // ---- epilogue: warps 2..5 ----
        const int quarter = warp & 3;                        // the TMEM lanes this warp may read
        const unsigned freed = map_to_rank(smem_u32(&acc_empty_bar[0]), 0);
        int local = 0;
        for (int tile = pair; tile < total_tiles; tile += num_pairs, ++local) {
            const int acc = local % ACCS;
            if (!mbar_wait_bounded(&acc_full_bar[acc], (unsigned)((local / ACCS) & 1))) {
                atomicOr(&failed, 8);
                break;
            }
            tc5_fence_after();
            int m0, n0;
            tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
            const int row = m0 + (int)rank * BM_CTA + quarter * 32 + lane;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned v[32];
                tc5_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), v);
                if (row < M) store_chunk32<TO>(v, C + (size_t)row * ldc, n0 + c0, N, swiglu);
            }
            tc5_fence_before();
            mbar_arrive_remote(freed + (unsigned)(acc * sizeof(unsigned long long)));
        }
    }
    tc5_fence_before();
    __syncthreads();
    cluster_sync();                                          // neither block frees or leaves while the other may still read it
    tc5_fence_after();
    if (warp == 1) dealloc_pair(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0 && failed && err)
        atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_GEMM_TC5_PAIR | ((unsigned)failed << VL_DEV_ROLE_SHIFT));
}

template <typename TO, int BN>
static int launch_pair(const void* A, const void* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                       unsigned* err, int swiglu, cudaStream_t s) {
    constexpr int STAGES = Shape<BN>::STAGES;
    constexpr unsigned STAGE_BYTES = Shape<BN>::STAGE_BYTES;
    CUtensorMap map_a, map_w;
    int rc = tc5_make_map(&map_a, A, M, K, lda, BM_CTA);
    if (rc) return rc;
    rc = tc5_make_map(&map_w, W, N, K, ldw, BN_CTA);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    auto kern = gemm_tc5_pair_kernel<TO, BN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    const int total = tiles_m * tiles_n, pairs = num_sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (total < pairs ? total : pairs));   // a pair per two SMs; pairs walk the tiles
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    // The cluster attribute and no other.  Started as a programmatic dependent (its clusters brought onto
    // the SM pairs, their tensor memory allocated and their barrier passed while earlier kernels, other
    // paired products among them, still ran) this kernel stood still on the device now and then; launched
    // the plain way it never did.  So it is always launched the plain way, whatever vl_set_pdl says.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, map_a, map_w, C, M, N, K, ldc, err, tiles_m, tiles_n, swiglu);
}

extern "C" int vl_gemm_bf16_tc5_pair(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K,
                                     int lda, int ldw, int ldc, unsigned* err, int swiglu, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (K <= 0 || K % 8 || lda % 8 || ldw % 8) return VL_ERR_UNSUPPORTED;
    if (swiglu ? (N % 16 || ldc < N / 2) : ldc < N) return VL_ERR_ARGUMENT;
    if (lda < K || ldw < K) return VL_ERR_ARGUMENT;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return VL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    // Which width.  A tile of 512 columns costs about 1.8 tiles of 256 (measured: neither keeps the tensor pipe
    // busier than about 80 %, what the shared memory of an SM moves bounds both) plus an epilogue that nothing
    // hides, and loses more when a pair walks many tiles (4,096 x 24,576 x 4,096: 560 us against 624).  It wins
    // where it saves a round of the pairs of SMs and the rounds are few: at 2,048 rows of Qwen3-8B o 53.9 ->
    // 50.1 us and down 155.5 -> 142.0 (one round of 64 tiles instead of two of 128), at 4,096 rows down 341 ->
    // 320; q/k/v and gate/up stay at 256 (80.2 against 100.5, 295.8 against 312.7).
    static int pairs = 0;
    if (!pairs) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        pairs = sms / 2;
    }
    const long long kb = (K + BK - 1) / BK, tm = (M + BM - 1) / BM;
    const long long r256 = (tm * ((N + 255) / 256) + pairs - 1) / pairs, r512 = (tm * ((N + 511) / 512) + pairs - 1) / pairs;
    int wide = N > 256 && r512 <= 2 && r512 * (18 * kb + 60) < r256 * 10 * kb;
    if (const char* v = getenv("VLLM_LITE_B200_PAIR_WIDTH")) {      // 256 or 512: for tests and measurements
        const int w = atoi(v);
        if (w == 256 || w == 512) wide = w == 512;
    }
    if (out_dtype == VL_BF16)
        return wide ? launch_pair<bf16, 512>(A, W, (bf16*)C, M, N, K, lda, ldw, ldc, err, swiglu, s)
                    : launch_pair<bf16, 256>(A, W, (bf16*)C, M, N, K, lda, ldw, ldc, err, swiglu, s);
    if (out_dtype == VL_F32)
        return wide ? launch_pair<float, 512>(A, W, (float*)C, M, N, K, lda, ldw, ldc, err, swiglu, s)
                    : launch_pair<float, 256>(A, W, (float*)C, M, N, K, lda, ldw, ldc, err, swiglu, s);
    return VL_ERR_UNSUPPORTED;
}
