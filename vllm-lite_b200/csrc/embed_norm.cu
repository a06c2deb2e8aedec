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
    pdl_launch_dependents();
    pdl_wait();
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

// The same function with a row kept in registers: 16-byte loads, one pass over memory.
// Thread i holds the float4 pieces i, i + 256, ... of the row (H a multiple of 4, at most
// 256 * 4 * VPT values).  The sum of squares is taken piece by piece in that fixed order.
template <typename TA> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                           __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<unsigned*>(&lo);
        r.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename TA, int VPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ delta, const int* __restrict__ rows,
                       const float* __restrict__ w, TA* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * H;
    const TA* dr = delta ? delta + (size_t)src * H : nullptr;
    const int H4 = H >> 2;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            v[i] = Quad<float>::load(xr + 4 * c);
            if (dr) {
                const float4 d = Quad<TA>::load(dr + 4 * c);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                if (!rows) Quad<float>::store(xr + 4 * c, v[i]);
            }
            ss += v[i].x * v[i].x; ss += v[i].y * v[i].y; ss += v[i].z * v[i].z; ss += v[i].w * v[i].w;
        }
    }
    ss = block_sum<256>(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            const float4 g = Quad<float>::load(w + 4 * c);
            Quad<TA>::store(o + 4 * c, make_float4(v[i].x * inv * g.x, v[i].y * inv * g.y, v[i].z * inv * g.z, v[i].w * inv * g.w));
        }
    }
}

template <typename TA>
static bool launch_rmsnorm_vec(float* x, const TA* delta, const int* rows, const float* w, TA* out, int R, int H,
                               float eps, cudaStream_t s) {
    if (H % 4) return false;
    const int pieces = (H / 4 + 255) / 256;
    if (pieces <= 1) vl_launch(add_rmsnorm_vec_kernel<TA, 1>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else if (pieces <= 2) vl_launch(add_rmsnorm_vec_kernel<TA, 2>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else if (pieces <= 4) vl_launch(add_rmsnorm_vec_kernel<TA, 4>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else if (pieces <= 8) vl_launch(add_rmsnorm_vec_kernel<TA, 8>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else return false;
    return true;
}

// y[r, c] += bias[c] for a linear layer with a bias vector: the product's result is widened, the float32
// bias added and the sum rounded once.
template <typename TA>
__global__ void add_bias_kernel(TA* __restrict__ y, const float* __restrict__ bias, size_t n, int cols) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = from_f32<TA>(to_f32(y[i]) + bias[i % (size_t)cols]);
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
        vl_launch(embed_kernel<float>, dim3(T), dim3(256), 0, s, ids, (const float*)table, x, H, V, err);
    else if (table_dtype == VL_BF16)
        vl_launch(embed_kernel<bf16>, dim3(T), dim3(256), 0, s, ids, (const bf16*)table, x, H, V, err);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

extern "C" int vl_add_rmsnorm(float* x, const void* delta, const int* rows, const float* w, void* out,
                              int act_dtype, int R, int H, float eps, void* stream) {
    if (R <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == VL_F32) {
        if (!launch_rmsnorm_vec<float>(x, (const float*)delta, rows, w, (float*)out, R, H, eps, s))
            add_rmsnorm_kernel<float><<<R, 256, 0, s>>>(x, (const float*)delta, rows, w, (float*)out, H, eps);
    } else if (act_dtype == VL_BF16) {
        if (!launch_rmsnorm_vec<bf16>(x, (const bf16*)delta, rows, w, (bf16*)out, R, H, eps, s))
            add_rmsnorm_kernel<bf16><<<R, 256, 0, s>>>(x, (const bf16*)delta, rows, w, (bf16*)out, H, eps);
    } else {
        return VL_ERR_UNSUPPORTED;
    }
    return vl_launch_status();
}

extern "C" int vl_add_bias(void* y, int act_dtype, const float* bias, long long rows, int cols, void* stream) {
    if (rows <= 0 || cols <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * (size_t)cols;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_dtype == VL_F32)
        add_bias_kernel<float><<<blocks, 256, 0, s>>>((float*)y, bias, n, cols);
    else if (act_dtype == VL_BF16)
        add_bias_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)y, bias, n, cols);
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
