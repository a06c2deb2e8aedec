// bfloat16 matrix products with float32 accumulation:  C[M,N] = A[M,K] * W[N,K]^T
// (a linear layer, y = x W^T, weight stored [out, in], no bias).
//
// vl_gemm_bf16_small_m: for the few rows of a decode step (M <= 64).  The product is bound by
// reading W once from HBM, so the kernel is built around that stream: a block owns 16 rows of W,
// its 8 warps take the 32-wide slices of K in turn, every lane reads 16 contiguous bytes of two
// rows of W and of one row of A per slice, and the tensor cores multiply them
// (mma.sync m16n8k16, W as the 16-row operand, 8 rows of A as the other).  The instruction pairs
// operand elements by their index along K and never mixes rows, so the 8 values a lane holds may
// stand for any 8 of the 16 positions of a slice as long as both operands use the same
// assignment; that is what lets each lane load whole 16-byte pieces.  The 8 warps' partial sums
// are added in warp order, so the result does not depend on the launch.
// K must be a multiple of 8 (16-byte rows); any M <= 64 and any N.
#include "common.cuh"

#define GS_THREADS 256
#define GS_WARPS (GS_THREADS / 32)
#define GS_ROWS 16

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, typename TO>
__global__ void __launch_bounds__(GS_THREADS)
gemm_bf16_small_m_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, TO* __restrict__ C,
                         int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float red[GS_THREADS / 32][MT][GS_ROWS][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GS_ROWS;
    const int r_lo = n0 + g, r_hi = n0 + g + 8;
    const bf16* w_lo = W + (size_t)min(r_lo, N - 1) * ldw;
    const bf16* w_hi = W + (size_t)min(r_hi, N - 1) * ldw;
    const bool ok_lo = r_lo < N, ok_hi = r_hi < N;
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int steps = (K + 31) / 32;
    constexpr int UNROLL = MT == 1 ? 8 : (MT == 2 ? 4 : 2);
    for (int s0 = warp; s0 < steps; s0 += GS_WARPS * UNROLL) {
        uint4 wl[UNROLL], wh[UNROLL], av[UNROLL][MT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (s0 + GS_WARPS * u) * 32 + 8 * t;
            const bool in = (s0 + GS_WARPS * u) < steps && k < K;
            wl[u] = (in && ok_lo) ? ldg_stream16(w_lo + k) : zero;
            wh[u] = (in && ok_hi) ? ldg_stream16(w_hi + k) : zero;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const int m = 8 * j + g;
                av[u][j] = (in && m < M) ? __ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda + k)) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                mma_bf16_16816(acc[j], wl[u].x, wh[u].x, wl[u].y, wh[u].y, av[u][j].x, av[u][j].y);
                mma_bf16_16816(acc[j], wl[u].z, wh[u].z, wl[u].w, wh[u].w, av[u][j].z, av[u][j].w);
            }
    }
    // acc[j] = {(row g, m 2t), (row g, m 2t+1), (row g+8, m 2t), (row g+8, m 2t+1)} of m-tile j
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        red[warp][j][g][2 * t] = acc[j][0];
        red[warp][j][g][2 * t + 1] = acc[j][1];
        red[warp][j][g + 8][2 * t] = acc[j][2];
        red[warp][j][g + 8][2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    for (int idx = tid; idx < MT * 8 * GS_ROWS; idx += GS_THREADS) {
        const int n = idx % GS_ROWS, m = idx / GS_ROWS;          // n fastest: 16 neighbours of a row of C
        const int j = m >> 3, mm = m & 7;
        if (m < M && n0 + n < N) {
            float v = red[0][j][n][mm];
#pragma unroll
            for (int w = 1; w < GS_THREADS / 32; ++w) v += red[w][j][n][mm];
            C[(size_t)m * ldc + n0 + n] = from_f32<TO>(v);
        }
    }
}

template <typename TO>
static int launch_small_m(const bf16* A, const bf16* W, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                          cudaStream_t s) {
    dim3 grid((N + GS_ROWS - 1) / GS_ROWS);
    if (M <= 8) gemm_bf16_small_m_kernel<1, TO><<<grid, GS_THREADS, 0, s>>>(A, W, C, M, N, K, lda, ldw, ldc);
    else if (M <= 16) gemm_bf16_small_m_kernel<2, TO><<<grid, GS_THREADS, 0, s>>>(A, W, C, M, N, K, lda, ldw, ldc);
    else if (M <= 32) gemm_bf16_small_m_kernel<4, TO><<<grid, GS_THREADS, 0, s>>>(A, W, C, M, N, K, lda, ldw, ldc);
    else gemm_bf16_small_m_kernel<8, TO><<<grid, GS_THREADS, 0, s>>>(A, W, C, M, N, K, lda, ldw, ldc);
    return vl_launch_status();
}

extern "C" int vl_gemm_bf16_small_m(const void* A, const void* W, void* C, int out_dtype, int M, int N, int K,
                                    int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (M > 64 || K <= 0 || K % 8 || lda % 8 || ldw % 8) return VL_ERR_UNSUPPORTED;
    if (lda < K || ldw < K || ldc < N) return VL_ERR_ARGUMENT;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return VL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == VL_BF16) return launch_small_m<bf16>((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, ldw, ldc, s);
    if (out_dtype == VL_F32) return launch_small_m<float>((const bf16*)A, (const bf16*)W, (float*)C, M, N, K, lda, ldw, ldc, s);
    return VL_ERR_UNSUPPORTED;
}
