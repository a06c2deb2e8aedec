// SwiGLU activation on the fused gate|up projection:
//     out[t, i] = silu(gu[t, i]) * gu[t, I + i],   silu(z) = z / (1 + exp(-z))
// (crates/model/src/components/mlp/swiglu.rs:18-31 of the reference).
// The arithmetic is float32; input and output are in the activation dtype.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * (size_t)I + i]);
    const float u = to_f32(gu[t * 2 * (size_t)I + I + i]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

extern "C" int vl_silu_mul(const void* gu, void* out, int dtype, int T, int I, void* stream) {
    if (T <= 0 || I <= 0) return VL_OK;
    const size_t total = (size_t)T * I;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, total);
    else if (dtype == VL_BF16)
        return vl_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, total);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}
