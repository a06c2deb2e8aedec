// SwiGLU activation on the fused gate|up projection:
//     out[t, i] = silu(gate_i) * up_i,   silu(z) = z / (1 + exp(-z))
// (crates/model/src/components/mlp/swiglu.rs:18-31 of the reference).
// Two layouts of the [T, 2I] input: group = 0, the gate columns then the up columns
// (gate_i = gu[t, i], up_i = gu[t, I + i]); group = g > 0, blocks of g gate columns followed by
// their g up columns (gate_i = gu[t, 2g*(i/g) + i%g], up_i = that + g), which is what lets a
// matrix-product kernel apply the activation to the tile it holds.
// The arithmetic is float32; input and output are in the activation dtype.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int group) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const size_t gi = group > 0 ? (size_t)2 * group * (i / group) + i % group : (size_t)i;
    const float g = to_f32(gu[t * 2 * (size_t)I + gi]);
    const float u = to_f32(gu[t * 2 * (size_t)I + gi + (group > 0 ? group : I)]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

extern "C" int vl_silu_mul(const void* gu, void* out, int dtype, int T, int I, int group, void* stream) {
    if (T <= 0 || I <= 0) return VL_OK;
    if (group < 0 || (group > 0 && I % group)) return VL_ERR_ARGUMENT;
    const size_t total = (size_t)T * I;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, total, group);
    else if (dtype == VL_BF16)
        return vl_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, total, group);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}
