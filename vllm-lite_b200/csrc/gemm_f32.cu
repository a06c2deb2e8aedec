// True float32 matrix product for the 32-bit path:  C[M,N] = A[M,K] * W[N,K]^T
// (a linear layer, y = x W^T with the weight stored [out, in]; no bias:
//  crates/model/src/components/attention/gqa/norm.rs:21-26 of the reference).
//
// Plain FFMA on CUDA cores: no tensor cores, no TF32, no split of K.  Every
// output element is the sum over k = 0..K-1 in that order, whatever M is and
// wherever the element lies in its tile, so a row's result is bit-for-bit the
// same whether it is computed alone or among thousands.
// Tiles of 64x64x16, 256 threads, 4x4 outputs per thread; any M, N, K.
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                   int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[GF_BK][GF_BM + 4];
    __shared__ float Ws[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            const int m = m0 + r, n = n0 + r;
            As[kk][r] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
            Ws[kk][r] = (n < N && k < K) ? W[(size_t)n * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

extern "C" int vl_gemm_f32_nt(const float* A, const float* W, float* C, int M, int N, int K,
                              int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return VL_ERR_ARGUMENT;
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    if (grid.y > 65535) return VL_ERR_UNSUPPORTED;
    gemm_f32_nt_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
    return vl_launch_status();
}
