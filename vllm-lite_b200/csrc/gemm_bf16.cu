// bfloat16 matrix products with float32 accumulation:  C[M,N] = A[M,K] * W[N,K]^T
// (a linear layer, y = x W^T, weight stored [out, in], no bias).
//
// vl_gemm_bf16_small_m: for the few rows of a decode step (M <= 16).  The product is bound by
// reading W once from HBM, so the kernel is built around that stream: a block owns 16 rows of W,
// a producer warp brings them in by bulk copies (TMA) through a ring of shared-memory stages, and
// four consumer warps multiply on the tensor cores (mma.sync m16n8k16, W as the 16-row operand,
// 8 rows of A as the other); every lane reads 16 contiguous bytes of two rows of W and of one row
// of A per 32-wide slice of K.  The instruction pairs
// operand elements by their index along K and never mixes rows, so the 8 values a lane holds may
// stand for any 8 of the 16 positions of a slice as long as both operands use the same
// assignment; that is what lets each lane load whole 16-byte pieces.  The 4 warps' partial sums
// are added in warp order, so the result does not depend on the launch.
// K must be a multiple of 8 (16-byte rows); any M <= 16 and any N.
#include "common.cuh"

#define GS_ROWS 16

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- mbarrier / bulk-copy helpers ------------------------------------------------------------
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
// A wait gives up after a bounded number of polls and of cycles (common.cuh) instead of hanging the device.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 0; i < VL_WAIT_POLL_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (vl_wait_gave_up(i, t0)) return false;
    }
    return false;
}
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

#define GS_CONSUMERS 4                     // consumer warps; warp 4 is the producer

// Optional fusion of an RMS norm on either side of the product (both sides null: a plain product).
//   Input side (ss_in): the rows of A are not yet normalised, A[m, k] = x[m, k] * w_norm[k]; row m of
//   the result is scaled by 1 / sqrt(sum_b ss_in[b * 16 + m] / hidden + eps), where the ss_count
//   vectors are the partial sums of squares that the producer of x left, block by block.
//   Output side (res): the result is added into the float32 stream res[m, n] (each block owns its
//   columns), C receives the next norm's unnormalised input bf16(res[m, n] * next_w[n]), and the
//   block's partial sums of squares of its columns of res go to ss_out[block * 16 + m].
struct NormFusion {
    const float* ss_in; int ss_count; float eps; int hidden;
    float* res; int ldres; const float* next_w; float* ss_out;
};

// Block = 16 rows of W.  The producer warp streams them through a ring of GS_STAGES stages of
// GS_KC columns (a multiple of 128) with one bulk copy (TMA) per row and stage; four consumer warps
// each take a quarter of every stage, read their tensor-core operands from shared memory (W) and
// from global memory (A, small and cached), and hand the stage back.  Sums are added in warp order
// at the end.  Stage size and count decide how many blocks share an SM and how many bytes each
// keeps in flight; the launcher picks them by the shape.
template <int MT, typename TO, int GS_KC, int GS_STAGES>
__global__ void __launch_bounds__(160)
gemm_bf16_small_m_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, TO* __restrict__ C,
                         int M, int N, int K, int lda, int ldw, int ldc, unsigned* err, int swiglu, int gran,
                         NormFusion nf) {
    static_assert(GS_KC % (32 * GS_CONSUMERS) == 0, "a stage is shared out in 32-wide slices among the consumer warps");
    constexpr int GS_ROWB = GS_KC * 2 + 16;    // bytes of a padded row of a stage: rows 16 bytes apart modulo 128
    extern __shared__ __align__(128) unsigned char gs_smem[];               // [GS_STAGES][16][GS_ROWB]
    __shared__ float red[GS_CONSUMERS][MT][GS_ROWS][8];
    __shared__ float s_inv[16];                                             // row scales of a fused input norm
    __shared__ __align__(8) unsigned long long full_bar[GS_STAGES], empty_bar[GS_STAGES];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // rows of W of this block: an even share of N, in units of `gran` rows, walked in tiles of 16
    const int units = (N + gran - 1) / gran;
    const int r0 = (int)((long long)blockIdx.x * units / gridDim.x) * gran;
    const int r1 = min(N, (int)((long long)(blockIdx.x + 1) * units / gridDim.x) * gran);
    const int iters = (K + GS_KC - 1) / GS_KC;
    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < GS_STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], GS_CONSUMERS); }
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == GS_CONSUMERS) {                                            // ---- producer ----
        // W is a constant of the step: its stream starts while earlier kernels are still running
        if (lane < GS_ROWS) {
            int git = 0;                                                 // stages issued so far, over all tiles
            for (int n0 = r0; n0 < r1; n0 += GS_ROWS) {
                const int valid = min(GS_ROWS, r1 - n0);                   // rows of this tile; the others are not copied
                const bf16* src_row = W + (size_t)min(n0 + lane, N - 1) * ldw;
                bool stop = false;
                for (int it = 0; it < iters; ++it, ++git) {
                    const int s = git % GS_STAGES;
                    if (git >= GS_STAGES) {                              // lane 0 waits for the consumers, all 16 follow it
                        int ok = 1;
                        if (lane == 0) ok = mbar_wait_bounded(&empty_bar[s], (unsigned)((git / GS_STAGES - 1) & 1)) ? 1 : 0;
                        ok = __shfl_sync(0x0000ffffu, ok, 0);
                        if (!ok) {
                            if (lane == 0 && err) atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_GEMM_SMALL_M);
                            stop = true;
                            break;
                        }
                    }
                    const int k0 = it * GS_KC;
                    const unsigned bytes = (unsigned)(min(GS_KC, K - k0) * 2);
                    if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], bytes * (unsigned)valid);
                    __syncwarp(0x0000ffffu);
                    if (lane < valid)
                        bulk_copy_g2s(gs_smem + ((size_t)s * GS_ROWS + lane) * GS_ROWB, src_row + k0, bytes, &full_bar[s]);
                }
                if (stop) break;
            }
        }
        return;
    }
    // ---- consumers ----
    pdl_wait();                                                            // A comes from the kernel before
    const int g = lane >> 2, t = lane & 3;
    if (nf.ss_in) {
        // 8 threads per row add the producer's partial sums, each its share in a fixed order
        const int m = tid >> 3, part = tid & 7;
        float ss = 0.f;
        for (int b = part; b < nf.ss_count; b += 8) ss += nf.ss_in[(size_t)b * 16 + m];
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (part == 0) s_inv[m] = 1.0f / sqrtf(ss / (float)nf.hidden + nf.eps);
        consumer_barrier();
    }
    float ss_run[MT];                                                      // (threads with n = 0) sums of squares of this block's columns
#pragma unroll
    for (int j = 0; j < MT; ++j) ss_run[j] = 0.f;
    const bf16* a_row[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) a_row[j] = A + (size_t)min(8 * j + g, M - 1) * lda + 8 * t;
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    constexpr int STEPS = GS_KC / 32 / GS_CONSUMERS;                        // 32-wide slices per warp and stage
    // A is small and cached, but a miss in L1 costs about a microsecond under load: the rows of A for
    // stage it + 1 are requested before stage it is multiplied, so that latency hides behind the wait
    // for W and the tensor-core work.
    uint4 av[2][STEPS][MT];
    auto load_a = [&](int it, uint4 (&dst)[STEPS][MT]) {
        const int kbase = it * GS_KC + warp * (GS_KC / GS_CONSUMERS);
#pragma unroll
        for (int u = 0; u < STEPS; ++u) {
            const int k = kbase + 32 * u;
#pragma unroll
            for (int j = 0; j < MT; ++j)
                dst[u][j] = (it < iters && k + 8 * t < K) ? __ldg(reinterpret_cast<const uint4*>(a_row[j] + k)) : zero;
        }
    };
    int git = 0;                                                           // stages consumed so far, over all tiles
    auto multiply = [&](int it, const uint4 (&a)[STEPS][MT]) -> bool {
        const int s = git % GS_STAGES;
        const int kbase = it * GS_KC + warp * (GS_KC / GS_CONSUMERS);
        if (!mbar_wait_bounded(&full_bar[s], (unsigned)((git / GS_STAGES) & 1))) {
            if (lane == 0 && err) atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_GEMM_SMALL_M);
            return false;
        }
        const unsigned char* stage = gs_smem + (size_t)s * GS_ROWS * GS_ROWB + (size_t)warp * (GS_KC / GS_CONSUMERS) * 2;
#pragma unroll
        for (int u = 0; u < STEPS; ++u) {
            // columns beyond K of the last stage were not copied; A is zero there, but stale bytes could
            // be NaN patterns, so W is zeroed as well
            const bool in = kbase + 32 * u + 8 * t < K;
            const uint4 wl = in ? *reinterpret_cast<const uint4*>(stage + (size_t)g * GS_ROWB + (32 * u + 8 * t) * 2) : zero;
            const uint4 wh = in ? *reinterpret_cast<const uint4*>(stage + (size_t)(g + 8) * GS_ROWB + (32 * u + 8 * t) * 2) : zero;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                mma_bf16_16816(acc[j], wl.x, wh.x, wl.y, wh.y, a[u][j].x, a[u][j].y);
                mma_bf16_16816(acc[j], wl.z, wh.z, wl.w, wh.w, a[u][j].z, a[u][j].w);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
        ++git;
        return true;
    };
    for (int n0 = r0; n0 < r1; n0 += GS_ROWS) {
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    bool ok = true;
    load_a(0, av[0]);
    for (int it = 0; it < iters; it += 2) {                                 // two stages per round: the buffers swap roles
        load_a(it + 1, av[1]);
        if (!multiply(it, av[0])) { ok = false; break; }
        if (it + 1 >= iters) break;
        load_a(it + 2, av[0]);
        if (!multiply(it + 1, av[1])) { ok = false; break; }
    }
    // acc[j] = {(row g, m 2t), (row g, m 2t+1), (row g+8, m 2t), (row g+8, m 2t+1)} of m-tile j
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        red[warp][j][g][2 * t] = acc[j][0];
        red[warp][j][g][2 * t + 1] = acc[j][1];
        red[warp][j][g + 8][2 * t] = acc[j][2];
        red[warp][j][g + 8][2 * t + 1] = acc[j][3];
    }
    consumer_barrier();
    if (swiglu) {
        // the tile's 16 rows of W are 8 gate rows and their 8 up rows: C[m, n0/2 + i] = silu(gate_i) * up_i
        for (int idx = tid; idx < MT * 8 * 8; idx += 32 * GS_CONSUMERS) {
            const int i = idx & 7, m = idx >> 3;
            const int j = m >> 3, mm = m & 7;
            if (ok && m < M && n0 + 8 + i < r1) {
                float gt = red[0][j][i][mm], up = red[0][j][i + 8][mm];
#pragma unroll
                for (int w = 1; w < GS_CONSUMERS; ++w) { gt += red[w][j][i][mm]; up += red[w][j][i + 8][mm]; }
                if (nf.ss_in) { gt *= s_inv[m]; up *= s_inv[m]; }
                C[(size_t)m * ldc + n0 / 2 + i] = from_f32<TO>(gt / (1.0f + expf(-gt)) * up);
            }
        }
    } else {
#pragma unroll
        for (int p = 0; p < MT; ++p) {                                     // 128 threads x MT passes = MT * 8 rows x 16 columns
            const int idx = tid + p * 32 * GS_CONSUMERS;
            const int n = idx % GS_ROWS, m = idx / GS_ROWS;                // n fastest: 16 neighbours of a row of C
            const int j = m >> 3, mm = m & 7;
            const bool valid = ok && m < M && n0 + n < r1;
            float sq = 0.f;
            if (valid) {
                float v = red[0][j][n][mm];
#pragma unroll
                for (int w = 1; w < GS_CONSUMERS; ++w) v += red[w][j][n][mm];
                if (nf.ss_in) v *= s_inv[m];
                if (nf.res) {
                    float* rp = nf.res + (size_t)m * nf.ldres + n0 + n;
                    const float r = *rp + v;
                    *rp = r;
                    sq = r * r;
                    v = r * nf.next_w[n0 + n];
                }
                C[(size_t)m * ldc + n0 + n] = from_f32<TO>(v);
            }
            if (nf.res) {                                                  // (uniform) the 16 threads of a row add their squares
                sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                ss_run[p] += sq;
            }
        }
    }
    consumer_barrier();                                                    // `red` is free for the next tile
    if (!ok) break;                                                        // a wait ran out: the error word says so
    }
    if (nf.ss_out && (tid & 15) == 0) {
#pragma unroll
        for (int p = 0; p < MT; ++p) {
            const int m = (tid + p * 32 * GS_CONSUMERS) / GS_ROWS;
            if (m < 16) nf.ss_out[(size_t)blockIdx.x * 16 + m] = m < M ? ss_run[p] : 0.f;
        }
    }
}

// One shape of the ring (columns a stage, stages) of the kernel for MT * 8 rows: its shared memory, how
// many of its blocks share an SM, and the grid for a product of `tiles` tiles of 16 rows.
// A block per tile, or, when that gives more blocks than fit on the device at once, the fewest blocks that
// need no more tiles each than that many would (1,536 tiles for 444 places: 384 blocks of 4 tiles, not
// 444 blocks of 3 or 4), each with an even share of the rows (for the fused activation: of the 16-row
// groups): all blocks end together, and the stream is bound by memory, not by the blocks' number (a decode
// step at batch 8: 3.99 -> 3.92 ms).
template <int MT, typename TO, int KC, int STAGES>
struct RingShape {
    static constexpr size_t smem = (size_t)STAGES * GS_ROWS * (KC * 2 + 16);
    static constexpr long long in_flight = (long long)STAGES * GS_ROWS * KC * 2;     // bytes of W a block keeps on their way
    static int per_sm() {
        static int v = 0;
        if (!v) {
            auto kern = gemm_bf16_small_m_kernel<MT, TO, KC, STAGES>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
                cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, kern, 160, smem) != cudaSuccess || v < 1)
                v = 1;
        }
        return v;
    }
    static int blocks(int tiles, int num_sms) {
        const int fit = num_sms * per_sm();
        const int rounds = (tiles + fit - 1) / fit;               // tiles of the busiest block
        return tiles < fit ? tiles : (tiles + rounds - 1) / rounds;
    }
    static int launch(const bf16* A, const bf16* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc, unsigned* err,
                      int swiglu, NormFusion nf, int* grid_out, int num_sms, cudaStream_t s) {
        auto kern = gemm_bf16_small_m_kernel<MT, TO, KC, STAGES>;
        const int grid = blocks((N + GS_ROWS - 1) / GS_ROWS, num_sms);
        if (grid_out) *grid_out = grid;
        return vl_launch(kern, dim3(grid), dim3(160), smem, s, A, W, C, M, N, K, lda, ldw, ldc, err, swiglu,
                         swiglu ? GS_ROWS : 1, nf);
    }
};

template <typename TO>
static int launch_small_m(const bf16* A, const bf16* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                          unsigned* err, int swiglu, NormFusion nf, int* grid_out, cudaStream_t s) {
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
#define GS_ARGS A, W, C, M, N, K, lda, ldw, ldc, err, swiglu, nf, grid_out, num_sms, s
    if (M > 8) return RingShape<2, TO, 512, 4>::launch(GS_ARGS);   // more rows need the registers
    // Up to 8 rows.  What decides is how many bytes of W the launch keeps on their way: memory answers after
    // 3 to 5 us under load, so about 23 MB must be in flight for its full bandwidth (measured inside a decode
    // step's graph, 8 rows, over the layer shapes of Qwen3-8B, 14B and 32B).  The shapes, finest stages first:
    // 4 x 512 columns (three blocks per SM), 3 x 768 (three), 2 x 1,024 (three), 3 x 1,024 (two per SM).  The
    // first whose blocks, all resident, hold 22.5 MB is taken, else the one that holds most.  For instance
    // (us): q/k/v of 8B, 384 tiles: 9.8 with 4 x 512 against 10.1 and 11.1 with 3 x 768 and 3 x 1,024; o of 8B,
    // 256 tiles: 7.7 with 3 x 1,024 against 8.5; q/k/v of 14B, 448 tiles (one more than 444 places: 224 blocks of
    // two tiles): 13.7 with 3 x 1,024 against 18.7 with 4 x 512; down of 32B, 320 tiles, K = 25,600: 42.6 with
    // 3 x 768 against 46.6 and 50.3.  Less than about 200 KB in flight per SM loses outright (two blocks of
    // 50 KB: 16.2 / 48.2 / 24.8 us for q/k/v, gate/up, down of 8B against 10.6 / 34.0 / 18.2).
    using S0 = RingShape<1, TO, 512, 4>;
    using S1 = RingShape<1, TO, 768, 3>;
    using S2 = RingShape<1, TO, 1024, 2>;
    using S3 = RingShape<1, TO, 1024, 3>;
    const int tiles = (N + GS_ROWS - 1) / GS_ROWS;
    const long long held[4] = {S0::blocks(tiles, num_sms) * S0::in_flight, S1::blocks(tiles, num_sms) * S1::in_flight,
                               S2::blocks(tiles, num_sms) * S2::in_flight, S3::blocks(tiles, num_sms) * S3::in_flight};
    int pick = -1;
    for (int i = 0; i < 4 && pick < 0; ++i)
        if (held[i] >= 22500000ll) pick = i;
    if (pick < 0) {
        pick = 0;
        for (int i = 1; i < 4; ++i)
            if (held[i] > held[pick]) pick = i;
    }
    switch (pick) {
        case 0: return S0::launch(GS_ARGS);
        case 1: return S1::launch(GS_ARGS);
        case 2: return S2::launch(GS_ARGS);
        default: return S3::launch(GS_ARGS);
    }
#undef GS_ARGS
}

// The product with an RMS norm fused on its input side (ss_in != null), on its output side
// (res != null), on both, or on neither; see NormFusion.  Fusion takes up to 16 rows, no fused
// activation on the output side, and bfloat16 C there.  grid_out (host, may be null) receives the
// number of blocks launched = the number of partial-sum vectors written to ss_out.
extern "C" int vl_gemm_bf16_small_m_fused(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K,
                                          int lda, int ldw, int ldc, unsigned* err, int swiglu,
                                          const float* ss_in, int ss_count, float eps, int hidden,
                                          float* res, int ldres, const float* next_w, float* ss_out,
                                          int* grid_out, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (swiglu && (N % 16 || ldc < N / 2)) return VL_ERR_ARGUMENT;
    if (M > 16 || K <= 0 || K % 8 || lda % 8 || ldw % 8) return VL_ERR_UNSUPPORTED;
    if (lda < K || ldw < K || (!swiglu && ldc < N)) return VL_ERR_ARGUMENT;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return VL_ERR_UNSUPPORTED;
    NormFusion nf = {};
    if (ss_in) {
        if (ss_count <= 0 || hidden <= 0) return VL_ERR_ARGUMENT;
        nf.ss_in = ss_in; nf.ss_count = ss_count; nf.eps = eps; nf.hidden = hidden;
    }
    if (res) {
        if (swiglu || out_dtype != VL_BF16) return VL_ERR_UNSUPPORTED;
        if (!next_w || !ss_out || ldres < N) return VL_ERR_ARGUMENT;
        nf.res = res; nf.ldres = ldres; nf.next_w = next_w; nf.ss_out = ss_out;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == VL_BF16) return launch_small_m<bf16>((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, ldw, ldc, err, swiglu, nf, grid_out, s);
    if (out_dtype == VL_F32) return launch_small_m<float>((const bf16*)A, (const bf16*)W, (float*)C, M, N, K, lda, ldw, ldc, err, swiglu, nf, grid_out, s);
    return VL_ERR_UNSUPPORTED;
}

extern "C" int vl_gemm_bf16_small_m(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K,
                                    int lda, int ldw, int ldc, unsigned* err, int swiglu, void* stream) {
    return vl_gemm_bf16_small_m_fused(A, W, C, out_dtype, M, N, K, lda, ldw, ldc, err, swiglu,
                                      nullptr, 0, 0.f, 0, nullptr, 0, nullptr, nullptr, nullptr, stream);
}
