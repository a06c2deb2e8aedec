// Attention of a ragged batch over the paged key/value cache.
//
// Every query token t of the step belongs to a request req[t] and sits at the
// absolute position pos[t]; it reads the keys lo..pos[t] of its request from
// the request's pages, lo = 0 or pos[t] - window + 1.  The new keys of this
// step are already in the cache (the rotary kernel wrote them), so a prompt
// portion, a continuation and a single decoded token are one case:
//     s_j = (q . k_j) * scale;  p = softmax_j(s);  o = sum_j p_j v_j
// (crates/model/src/components/attention/util.rs:150-176 of the reference;
//  query head h reads KV head h / (nq / nkv), util.rs:55-87).
// Scores, the running maximum, the sum and the output are float32.
//
// vl_paged_attention: one block per (token, query head), 16 groups of 8 lanes.
// Group g owns the keys whose position is g modulo 16 and keeps a running
// softmax of its own; the 16 partial results are merged in group order.  Which
// keys a group sees and the order of every sum depend on positions alone, so a
// token's output does not depend on how the batch was cut.
// head_dim: multiples of 16 up to 256.
#include "common.cuh"

#define ATT_THREADS 128
#define ATT_GROUPS 16
#define ATT_MAX_HD 256

template <typename T> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair<bf16> {
    static __device__ __forceinline__ float2 load(const bf16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
};

template <typename T, int R>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                       const T* __restrict__ kcache, const T* __restrict__ vcache,
                       const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ req_index, const int* __restrict__ positions,
                       int nq, int nkv, int page_size, int num_pages, float scale, int window,
                       unsigned* err) {
    constexpr int HD = R * 16;
    __shared__ float s_acc[ATT_GROUPS][HD];
    __shared__ float s_m[ATT_GROUPS], s_l[ATT_GROUPS];
    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (nq / nkv);
    const int g = threadIdx.x >> 3, l = threadIdx.x & 7;
    const int req = req_index[t];
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (size_t)req * max_blocks;

    float qr[R][2], acc[R][2];
    const T* qp = q + (size_t)t * q_stride + (size_t)h * HD;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float2 v = Pair<T>::load(qp + 16 * r + 2 * l);
        qr[r][0] = v.x; qr[r][1] = v.y;
        acc[r][0] = 0.f; acc[r][1] = 0.f;
    }
    float m = -INFINITY, lsum = 0.f;

    for (int jb = (lo / ATT_GROUPS) * ATT_GROUPS; jb <= pos; jb += ATT_GROUPS) {
        const int j = jb + g;
        bool valid = (j >= lo) && (j <= pos);
        size_t base = 0;
        if (valid) {
            const int blk = j / page_size;
            const int page = blk < max_blocks ? table[blk] : -1;
            if (page < 0 || page >= num_pages) {
                if (l == 0) atomicOr(err, VL_DEV_BAD_PAGE);
                valid = false;
            } else {
                base = (((size_t)page * nkv + kvh) * page_size + (j - blk * page_size)) * HD;
            }
        }
        float dot = 0.f;
        if (valid) {
            const T* kp = kcache + base;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float2 kv = Pair<T>::load(kp + 16 * r + 2 * l);
                dot += qr[r][0] * kv.x;
                dot += qr[r][1] * kv.y;
            }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        if (valid) {
            const float s = dot * scale;
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn);
            const float p = expf(s - mn);
            lsum = lsum * corr + p;
            const T* vp = vcache + base;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float2 vv = Pair<T>::load(vp + 16 * r + 2 * l);
                acc[r][0] = acc[r][0] * corr + p * vv.x;
                acc[r][1] = acc[r][1] * corr + p * vv.y;
            }
            m = mn;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        s_acc[g][16 * r + 2 * l] = acc[r][0];
        s_acc[g][16 * r + 2 * l + 1] = acc[r][1];
    }
    if (l == 0) { s_m[g] = m; s_l[g] = lsum; }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < ATT_GROUPS; ++i) M = fmaxf(M, s_m[i]);
    T* op = out + ((size_t)t * nq + h) * HD;
    for (int e = threadIdx.x; e < HD; e += ATT_THREADS) {
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int i = 0; i < ATT_GROUPS; ++i) {
            const float wgt = (s_m[i] == -INFINITY) ? 0.f : expf(s_m[i] - M);
            L += s_l[i] * wgt;
            o += s_acc[i][e] * wgt;
        }
        op[e] = from_f32<T>(L > 0.f ? o / L : 0.f);
    }
}

template <typename T>
static int launch_paged_attention(int R, dim3 grid, cudaStream_t s, const T* q, int q_stride, T* out,
                                  const T* kc, const T* vc, const int* bt, int max_blocks,
                                  const int* req, const int* pos, int nq, int nkv, int page_size,
                                  int num_pages, float scale, int window, unsigned* err) {
#define ATT_CASE(RR)                                                                              \
    case RR:                                                                                      \
        paged_attention_kernel<T, RR><<<grid, ATT_THREADS, 0, s>>>(                               \
            q, q_stride, out, kc, vc, bt, max_blocks, req, pos, nq, nkv, page_size, num_pages,    \
            scale, window, err);                                                                  \
        break;
    switch (R) {
        ATT_CASE(1) ATT_CASE(2) ATT_CASE(3) ATT_CASE(4) ATT_CASE(5) ATT_CASE(6) ATT_CASE(7) ATT_CASE(8)
        ATT_CASE(9) ATT_CASE(10) ATT_CASE(11) ATT_CASE(12) ATT_CASE(13) ATT_CASE(14) ATT_CASE(15) ATT_CASE(16)
        default: return VL_ERR_UNSUPPORTED;
    }
#undef ATT_CASE
    return vl_launch_status();
}

extern "C" int vl_paged_attention(const void* q, int q_stride, void* out, int dtype,
                                  const void* kcache, const void* vcache,
                                  const int* block_table, int max_blocks,
                                  const int* req_index, const int* positions,
                                  int T, int nq, int nkv, int hd, int page_size, int num_pages,
                                  float scale, int window, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd <= 0 || hd % 16 || hd > ATT_MAX_HD) return VL_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0) return VL_ERR_ARGUMENT;
    if (nq > 65535) return VL_ERR_UNSUPPORTED;
    dim3 grid(T, nq);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return launch_paged_attention<float>(hd / 16, grid, s, (const float*)q, q_stride, (float*)out,
                                             (const float*)kcache, (const float*)vcache, block_table,
                                             max_blocks, req_index, positions, nq, nkv, page_size,
                                             num_pages, scale, window, err);
    if (dtype == VL_BF16)
        return launch_paged_attention<bf16>(hd / 16, grid, s, (const bf16*)q, q_stride, (bf16*)out,
                                            (const bf16*)kcache, (const bf16*)vcache, block_table,
                                            max_blocks, req_index, positions, nq, nkv, page_size,
                                            num_pages, scale, window, err);
    return VL_ERR_UNSUPPORTED;
}
