// bfloat16 matrix product for the 9 to 64 rows of a decode step with many requests, on the
// 5th-generation tensor cores:
//     C[M,N] = A[M,K] * W[N,K]^T,   float32 accumulation, C bfloat16 or float32,  M <= 64
// Like csrc/gemm_bf16.cu (up to 8 rows) the product is bound by one read of W, and the kernel is
// built around that stream; unlike it the arithmetic no longer fits mma.sync beside the stream
// (every block would read all rows of A once per 16 rows of W), so the roles of the operands are
// turned round for tcgen05: a tile is 128 rows of W (the M side of the instruction) by BT = 16, 32 or
// 64 rows of A (its N side), the accumulator [128 x BT] lives in TMEM, and a thread of the epilogue
// owns one column n of C and sees all rows m.
//
//   warp 0, one thread   TMA producer: per stage a 128 x 64 tile of W and a BT x 64 tile of A
//                        (cp.async.bulk.tensor.2d, 128-byte swizzle) into a ring of stages.  W is a
//                        constant of the step: the copies of its first stages are issued before the
//                        kernel waits for the kernels before it;
//   warp 1, one thread   tcgen05.mma (cta_group::1, kind::f16, M 128, N BT, K 16), 4 per stage; the
//                        warp allocates and frees the accumulator's columns of TMEM;
//   warps 2..5           epilogue.
// Few tiles (a hidden size of 4,096 gives 32) cannot keep memory busy: then K is cut among the 2, 4
// or 8 blocks of a cluster, each block leaves its [BT x 128] partial sums in its shared memory, and
// after a cluster barrier every block adds, for its share of the tile's columns, the partial sums
// of all blocks in the order of their ranks (ld.shared::cluster) and finishes them: the result does
// not depend on the launch.  With tiles for every SM a block walks several tiles instead.
//
// The epilogue can, as in gemm_bf16.cu: scale row m by an RMS norm's factor (ss_in: partial sums of
// squares left by the producer of A); apply SwiGLU (W holds blocks of 8 gate rows and their 8 up
// rows); add the result into the float32 stream and leave the next norm's unnormalised input and the
// partial sums of squares of the stream (vectors of SS_STRIDE floats, one per group of up to 32
// columns' worth of threads, written in full by exactly one group each).
// Rows beyond M or N and columns beyond K are zero-filled by the TMA unit.  Every wait on an
// mbarrier is bounded (tc5.cuh); the cluster's barriers are reached by every thread whatever happened.
#include "tc5.cuh"

namespace {
constexpr int BW = 128;                      // rows of W per tile
constexpr int BK = 64;                       // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int SS_STRIDE = 64;                // floats between two vectors of partial sums
constexpr int MAX_SPLIT = 8;

struct StreamFusion {
    const float* ss_in; int ss_count; float eps; int hidden;
    float* res; int ldres; const float* next_w; float* ss_out;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned cluster_size() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of the same place in block `rank` of the cluster
__device__ __forceinline__ unsigned cluster_map(unsigned local_addr, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ float ld_cluster_f32(unsigned cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void tc5_ld16(unsigned taddr, unsigned* r) {                  // 32 lanes x 16 columns
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
}  // namespace
using namespace tc5;

// What the epilogue does with one element of the product: `val` is y[m, n] summed over all of K.
// Called by all lanes of a warp together (it shuffles); `live` says whether (m, n) exists.
// Returns the element's square of the new stream (0 where there is none) for the sums of squares.
template <typename TO>
__device__ __forceinline__ float finish_element(float val, int m, int n, bool live, int N, TO* __restrict__ C, int ldc,
                                                int swiglu, const StreamFusion& nf, const float* s_inv) {
    if (nf.ss_in) val *= s_inv[m];
    if (swiglu) {
        // n = 16 b + i (gate, i < 8) or 16 b + 8 + i (up): the partner sits 8 lanes further on
        const float up = __shfl_down_sync(0xffffffffu, val, 8);
        if (live && (n & 8) == 0 && n + 8 < N)
            C[(size_t)m * ldc + (n >> 4) * 8 + (n & 7)] = from_f32<TO>(val / (1.0f + expf(-val)) * up);
        return 0.f;
    }
    if (!live) return 0.f;
    if (nf.res) {
        float* rp = nf.res + (size_t)m * nf.ldres + n;
        const float r = *rp + val;
        *rp = r;
        C[(size_t)m * ldc + n] = from_f32<TO>(r * nf.next_w[n]);
        return r * r;
    }
    C[(size_t)m * ldc + n] = from_f32<TO>(val);
    return 0.f;
}

// Grid: clusters of `split` blocks (1: no cluster); cluster c takes the tiles c, c + clusters, ...
// (with split > 1 the launcher gives every cluster exactly one tile).
template <int BT, int STAGES, typename TO>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc5_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                       TO* __restrict__ C, int M, int N, int K, int ldc, unsigned* err, int tiles, int swiglu,
                       StreamFusion nf) {
    constexpr unsigned W_BYTES = BW * BK * 2, A_BYTES = BT * BK * 2, STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr unsigned TMEM_COLS = BT < 32 ? 32 : BT;        // a power of two >= 32
    static_assert(STAGES * STAGE_BYTES >= BT * BW * 4, "the partial sums of a tile reuse the ring");
    extern __shared__ unsigned char tc5_smem_raw[];
    // tiles of the 128-byte swizzle must start on 1024-byte boundaries
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc5_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full_bar, acc_empty_bar;
    __shared__ unsigned tmem_base_slot;
    __shared__ int failed;
    __shared__ float s_inv[SS_STRIDE];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = (int)cluster_size(), rank = (int)cluster_rank();
    const int cluster_id = blockIdx.x / split, clusters = gridDim.x / split;
    const int k_blocks = (K + BK - 1) / BK;
    const int kb0 = (int)((long long)rank * k_blocks / split), kb1 = (int)((long long)(rank + 1) * k_blocks / split);
    const int kcount = kb1 - kb0;                            // this block's share of K, in stages

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        mbar_init(&acc_full_bar, 1);
        mbar_init(&acc_empty_bar, 128);
        mbar_fence_init();
        failed = 0;
    }
    pdl_launch_dependents();
    __syncthreads();
    // The weight stream starts at once: the first stages' tiles of W are on their way while the kernels
    // before this one finish (they never write a weight).
    const int early = (cluster_id < tiles) ? min(STAGES, kcount) : 0;
    if (threadIdx.x == 0) {
        for (int j = 0; j < early; ++j) {
            mbar_arrive_expect_tx(&full_bar[j], STAGE_BYTES);
            tma_load_2d(smem + (size_t)j * STAGE_BYTES, &map_w, (kb0 + j) * BK, cluster_id * BW, &full_bar[j]);
        }
    }
    pdl_wait();                                              // A, the stream and the partial sums come from the kernels before
    // Tensor memory is taken only now: a block started as a programmatic dependent holds none of it while
    // an earlier kernel still runs.
    if (warp == 1) tc5_alloc(&tmem_base_slot, TMEM_COLS);
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    float v[BT];                                             // (epilogue) column n of the tile, all rows m
    const int e = (warp & 3) * 32 + lane;                    // (epilogue) this thread's TMEM lane = row of W in the tile

    if (warp == 0) {
        if (lane == 0) {                                     // ---- TMA producer ----
            int it = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < tiles && ok; tile += clusters) {
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    if (it >= early) {
                        if (it >= STAGES && !mbar_wait_bounded(&empty_bar[s], (unsigned)((it / STAGES - 1) & 1))) {
                            atomicOr(&failed, 1);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
                        tma_load_2d(st, &map_w, kb * BK, tile * BW, &full_bar[s]);
                    }
                    tma_load_2d(st + W_BYTES, &map_a, kb * BK, 0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                     // ---- MMA issuer ----
            constexpr unsigned idesc = make_idesc(BW, BT);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < tiles && ok; tile += clusters, ++local) {
                if (local >= 1 && !mbar_wait_bounded(&acc_empty_bar, (unsigned)((local - 1) & 1))) {
                    atomicOr(&failed, 2);
                    break;
                }
                tc5_fence_after();
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(&full_bar[s], (unsigned)((it / STAGES) & 1))) {
                        atomicOr(&failed, 4);
                        ok = false;
                        break;
                    }
                    tc5_fence_after();
                    const unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    const unsigned long long wdesc = make_smem_desc(st), adesc = make_smem_desc(st + W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)    // 16 columns of K further on: +32 bytes, +2 in the address field
                        tc5_mma(tmem_base, wdesc + (unsigned long long)(k * 2), adesc + (unsigned long long)(k * 2), idesc,
                                (kb > kb0 || k > 0) ? 1u : 0u);
                    tc5_commit(&empty_bar[s]);               // the stage is free once these MMAs have read it
                }
                if (ok) tc5_commit(&acc_full_bar);           // the accumulator is complete
            }
        }
    } else {                                                 // ---- epilogue: warps 2..5 ----
        if (nf.ss_in) {
            // 128 / BT threads per row add the producer's partial sums, each its share in a fixed order
            constexpr int P = 128 / BT;
            const int t = (warp - 2) * 32 + lane, m = t / P, part = t % P;
            float ss = 0.f;
            for (int b = part; b < nf.ss_count; b += P) ss += nf.ss_in[(size_t)b * SS_STRIDE + m];
#pragma unroll
            for (int o = 1; o < P; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (part == 0) s_inv[m] = 1.0f / sqrtf(ss / (float)nf.hidden + nf.eps);
            epilogue_barrier();
        }
        int local = 0;
        for (int tile = cluster_id; tile < tiles; tile += clusters, ++local) {
            if (!mbar_wait_bounded(&acc_full_bar, (unsigned)(local & 1))) {
                atomicOr(&failed, 8);
                break;
            }
            tc5_fence_after();
            unsigned* vu = reinterpret_cast<unsigned*>(v);
            const unsigned taddr = tmem_base + ((unsigned)((warp & 3) * 32) << 16);
            if constexpr (BT == 16) {
                tc5_ld16(taddr, vu);
            } else {
#pragma unroll
                for (int c = 0; c < BT; c += 32) tc5_ld32_nowait(taddr + (unsigned)c, vu + c);
            }
            tc5_wait_ld();
            if (kcount == 0) {                               // (never with the launcher's choice of split) nothing was added
#pragma unroll
                for (int m = 0; m < BT; ++m) v[m] = 0.f;
            }
            if (split > 1) break;                            // one tile; it is finished by the whole cluster below
            tc5_fence_before();
            mbar_arrive(&acc_empty_bar);                     // 128 arrivals hand the accumulator back
            const int n = tile * BW + e;
#pragma unroll
            for (int m = 0; m < BT; ++m) {
                float sq = finish_element<TO>(v[m], m, n, m < M && n < N, N, C, ldc, swiglu, nf, s_inv);
                if (nf.ss_out) {                             // (uniform) the warp's 32 columns
#pragma unroll
                    for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    if (lane == 0) nf.ss_out[(size_t)(tile * 4 + (e >> 5)) * SS_STRIDE + m] = sq;
                }
            }
        }
    }
    __syncwarp();
    if (split > 1) {
        // ---- K was cut among the blocks of the cluster: everybody's partial sums, then everybody's share ----
        float* part = reinterpret_cast<float*>(smem);        // [BT][128]; the ring is idle: every stage was multiplied
        const bool mine = warp >= 2 && cluster_id < tiles && !failed;
        if (warp >= 2) {
#pragma unroll
            for (int m = 0; m < BT; ++m) part[m * BW + e] = mine ? v[m] : 0.f;
        }
        cluster_sync();
        if (warp >= 2 && cluster_id < tiles) {
            const int Wd = BW / split;                       // columns of the tile that this block finishes
            const int n_sub = e % Wd, mg = e / Wd;           // split groups of threads share out the rows
            const int n_local = rank * Wd + n_sub, n = cluster_id * BW + n_local;
            const int per = BT / split;                      // rows per group (BT and split are powers of two, split <= 8 <= BT / 2)
            const unsigned base = smem_u32(part);
            const int unit = Wd < 32 ? Wd : 32;              // threads that hold the columns of one vector's entry
            const int vec = (cluster_id * split + rank) * (Wd > 32 ? Wd / 32 : 1) + (n_sub >> 5);
            for (int mi = 0; mi < per; ++mi) {
                const int m = mg * per + mi;
                const unsigned off = base + (unsigned)(m * BW + n_local) * 4u;
                float val = 0.f;
                for (int s = 0; s < split; ++s) val += ld_cluster_f32(cluster_map(off, (unsigned)s));
                float sq = finish_element<TO>(val, m, n, m < M && n < N, N, C, ldc, swiglu, nf, s_inv);
                if (nf.ss_out) {
                    for (int o = unit >> 1; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    if ((lane & (unit - 1)) == 0) nf.ss_out[(size_t)vec * SS_STRIDE + m] = sq;
                }
            }
        }
        cluster_sync();                                      // nobody leaves while another block may still read its sums
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    if (warp == 1) tc5_dealloc(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0 && failed && err)
        atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_GEMM_TC5 | ((unsigned)failed << VL_DEV_ROLE_SHIFT));
}

// ---- host side -------------------------------------------------------------------------------
// How K is cut: the fewest blocks per tile (1, 2, 4 or 8) that give every SM a block, each block keeping
// at least two stages of K.
static int stream_split(int tiles, int k_blocks, int num_sms) {
    int split = 1;
    while (split < MAX_SPLIT && tiles * split < num_sms && k_blocks / (split * 2) >= 2) split *= 2;
    return split;
}

template <int BT, int STAGES, typename TO>
static int launch_stream(const void* A, const void* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                         unsigned* err, int swiglu, StreamFusion nf, int* vectors_out, cudaStream_t s) {
    CUtensorMap map_w, map_a;
    int rc = tc5_make_map(&map_w, W, N, K, ldw, BW);
    if (rc) return rc;
    rc = tc5_make_map(&map_a, A, M, K, lda, BT);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (BW + BT) * BK * 2 + 1024;
    auto kern = gemm_tc5_stream_kernel<BT, STAGES, TO>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    static int per_sm = 0;
    if (!per_sm && (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NUM_THREADS, smem) != cudaSuccess || per_sm < 1))
        per_sm = 1;
    const int tiles = (N + BW - 1) / BW, k_blocks = (K + BK - 1) / BK;
    const int split = stream_split(tiles, k_blocks, num_sms);
    const int vectors = tiles * (split > 4 ? split : 4);
    if (vectors_out) *vectors_out = vectors;
    cudaLaunchConfig_t cfg = {};
    // one tile per cluster when K is cut; else as many blocks as are resident at once walk the tiles
    cfg.gridDim = dim3(split > 1 ? tiles * split : (tiles < num_sms * per_sm ? tiles : num_sms * per_sm));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = split; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (vl_pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, kern, map_w, map_a, C, M, N, K, ldc, err, tiles, swiglu, nf);
}

template <typename TO>
static int dispatch_stream(const void* A, const void* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                           unsigned* err, int swiglu, StreamFusion nf, int* vectors_out, cudaStream_t s) {
    // stages: about 100 KB of ring, so that two blocks share an SM
    if (M <= 16) return launch_stream<16, 6, TO>(A, W, C, M, N, K, lda, ldw, ldc, err, swiglu, nf, vectors_out, s);
    if (M <= 32) return launch_stream<32, 5, TO>(A, W, C, M, N, K, lda, ldw, ldc, err, swiglu, nf, vectors_out, s);
    return launch_stream<64, 4, TO>(A, W, C, M, N, K, lda, ldw, ldc, err, swiglu, nf, vectors_out, s);
}

// The most rows the kernel takes, the stride of a vector of partial sums, and the number of vectors
// that a product of N columns over K leaves (what `partial_out` must hold).
extern "C" int vl_gemm_bf16_stream_max_rows() { return 64; }
extern "C" int vl_gemm_bf16_stream_ss_stride() { return SS_STRIDE; }

// C = A W^T for M <= 64 with the optional fusions of vl_gemm_bf16_small_m_fused (csrc/gemm_bf16.cu):
//   ss_in (ss_count vectors of SS_STRIDE floats), eps, hidden: an RMS norm on the input side;
//   res [M, ldres] float32, next_w [N], ss_out: the result is added into res, C receives
//   bf16(res * next_w) and ss_out the partial sums of squares of res; *vectors_out their number.
extern "C" int vl_gemm_bf16_stream_tc5(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K,
                                       int lda, int ldw, int ldc, unsigned* err, int swiglu,
                                       const float* ss_in, int ss_count, float eps, int hidden,
                                       float* res, int ldres, const float* next_w, float* ss_out, int* vectors_out,
                                       void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (M > 64 || K <= 0 || K % 8 || lda % 8 || ldw % 8) return VL_ERR_UNSUPPORTED;
    if (swiglu ? (N % 16 || ldc < N / 2) : ldc < N) return VL_ERR_ARGUMENT;
    if (lda < K || ldw < K) return VL_ERR_ARGUMENT;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return VL_ERR_UNSUPPORTED;
    if (ss_in && (ss_count <= 0 || hidden <= 0)) return VL_ERR_ARGUMENT;
    if (res && (swiglu || !next_w || !ss_out || ldres < N)) return VL_ERR_ARGUMENT;
    StreamFusion nf = {ss_in, ss_count, eps, hidden, res, ldres, next_w, res ? ss_out : nullptr};
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == VL_BF16)
        return dispatch_stream<bf16>(A, W, (bf16*)C, M, N, K, lda, ldw, ldc, err, swiglu, nf, vectors_out, s);
    if (out_dtype == VL_F32)
        return dispatch_stream<float>(A, W, (float*)C, M, N, K, lda, ldw, ldc, err, swiglu, nf, vectors_out, s);
    return VL_ERR_UNSUPPORTED;
}
