// Embedding gather and RMS norm with the residual sum folded in.
//
// The residual stream `x` is float32 in every mode.  A block hands the next
// norm a pending `delta` (the previous mixer's or feed-forward's output, in the
// activation dtype); the norm kernel adds it into `x` in float32, then norms:
//     x <- x + delta;   h = x / sqrt(mean(x^2) + eps) * w
// (formula: crates/model/src/components/norm/rms_norm.rs:26-49 of the reference).
// One block of 256 threads per row; the order of the additions of the mean is a
// function of the row length alone.
#include "common.cuh"

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ x, int H, int V, unsigned* err) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* row = x + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = to_f32(src[i]);
}

// rows == nullptr: row r of the output is row r of x (and x is updated in place
// when delta is given).  rows != nullptr: output row r is made from x[rows[r]]
// (+ delta[rows[r]]) and x is left untouched.
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ w,
                                   TA* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * H;
    const TA* dr = delta ? delta + (size_t)src * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = xr[i];
        if (dr) {
            v += to_f32(dr[i]);
            if (!rows) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum<256>(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = xr[i];
        if (dr && rows) v += to_f32(dr[i]);
        o[i] = from_f32<TA>(v * inv * w[i]);
    }
}

// x += delta, for the residual that is still pending after the last block when
// someone wants the stream itself.
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ x, const TA* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_f32(delta[i]);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<TO>(to_f32(in[i]));
}

extern "C" int vl_embed(const int* ids, const void* table, int table_dtype, float* x,
                        int T, int H, int V, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == VL_F32)
        embed_kernel<float><<<T, 256, 0, s>>>(ids, (const float*)table, x, H, V, err);
    else if (table_dtype == VL_BF16)
        embed_kernel<bf16><<<T, 256, 0, s>>>(ids, (const bf16*)table, x, H, V, err);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

extern "C" int vl_add_rmsnorm(float* x, const void* delta, const int* rows, const float* w, void* out,
                              int act_dtype, int R, int H, float eps, void* stream) {
    if (R <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == VL_F32)
        add_rmsnorm_kernel<float><<<R, 256, 0, s>>>(x, (const float*)delta, rows, w, (float*)out, H, eps);
    else if (act_dtype == VL_BF16)
        add_rmsnorm_kernel<bf16><<<R, 256, 0, s>>>(x, (const bf16*)delta, rows, w, (bf16*)out, H, eps);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

extern "C" int vl_residual_add(float* x, const void* delta, int act_dtype, long long n, void* stream) {
    if (n <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_dtype == VL_F32)
        residual_add_kernel<float><<<blocks, 256, 0, s>>>(x, (const float*)delta, (size_t)n);
    else if (act_dtype == VL_BF16)
        residual_add_kernel<bf16><<<blocks, 256, 0, s>>>(x, (const bf16*)delta, (size_t)n);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

extern "C" int vl_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream) {
    if (n <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == VL_F32 && out_dtype == VL_BF16)
        cast_kernel<float, bf16><<<blocks, 256, 0, s>>>((const float*)in, (bf16*)out, (size_t)n);
    else if (in_dtype == VL_BF16 && out_dtype == VL_F32)
        cast_kernel<bf16, float><<<blocks, 256, 0, s>>>((const bf16*)in, (float*)out, (size_t)n);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}
