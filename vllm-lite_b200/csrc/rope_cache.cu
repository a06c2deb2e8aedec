// Per-head norm of q and k, rotary position encoding, and the write of the new
// keys and values into the paged cache, in one pass over the fused q|k|v rows.
//
//   q_head, k_head <- head / sqrt(mean(head^2) + eps) * w        (optional)
//   angle = (float)pos * inv_freq[i];  pairs (x[i], x[i + rot/2]) of the first
//   `rot` features:  x1' = x1 cos - x2 sin,  x2' = x2 cos + x1 sin   (optional)
// (crates/model/src/components/attention/rope_gqa.rs:214-248 and
//  crates/model/src/components/positional/rope.rs:507-558 of the reference).
// q is rewritten in place; k and v go to the cache slot of their token:
//   page = slot / page_size, offset = slot % page_size,
//   cache[page][kv_head][offset][:]  with cache = [pages, nkv, page_size, hd].
// A token whose slot is negative writes no cache (a call that reads another
// call's cache).  Norm, angles, sine and cosine are float32 in every mode.
//
// One warp per (token, head); head_dim up to 512, any even value.
#include "common.cuh"

#define ROPE_WARPS 4
#define ROPE_MAX_HD 512

template <typename T>
__global__ void qk_norm_rope_write_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ inv_freq, int rot,
    T* __restrict__ kcache, T* __restrict__ vcache,
    int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err) {
    __shared__ float buf[ROPE_WARPS][ROPE_MAX_HD];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * ROPE_WARPS + warp;
    const int nheads = nq + 2 * nkv;
    if (head >= nheads) return;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nq : head - nq - nkv);
    const int slot = slots ? slots[t] : -1;

    T* dst = nullptr;
    if (!is_q) {
        if (slot < 0) return;                 // nothing to write for this token
        if ((long long)slot >= num_slots) {
            if (lane == 0) atomicOr(err, VL_DEV_BAD_SLOT);
            return;
        }
        const int page = slot / page_size, off = slot - page * page_size;
        T* cache = is_k ? kcache : vcache;
        dst = cache + (((size_t)page * nkv + kvh) * page_size + off) * hd;
    }
    if (!is_q && !is_k) {                     // v: plain copy
        for (int e = lane; e < hd; e += 32) dst[e] = src[e];
        return;
    }
    float* b = buf[warp];
    float ss = 0.f;
    for (int e = lane; e < hd; e += 32) {
        const float v = to_f32(src[e]);
        b[e] = v;
        ss += v * v;
    }
    const float* w = is_q ? qw : kw;
    if (w) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
        for (int e = lane; e < hd; e += 32) b[e] = b[e] * inv * w[e];
    }
    __syncwarp();
    T* out = is_q ? src : dst;
    const int half = rot / 2;
    if (inv_freq && half > 0) {
        const float pos = (float)positions[t];
        for (int i = lane; i < half; i += 32) {
            const float angle = pos * inv_freq[i];
            float sn, cs;
            sincosf(angle, &sn, &cs);
            const float x1 = b[i], x2 = b[i + half];
            out[i] = from_f32<T>(x1 * cs - x2 * sn);
            out[i + half] = from_f32<T>(x2 * cs + x1 * sn);
        }
        for (int e = rot + lane; e < hd; e += 32) out[e] = from_f32<T>(b[e]);
    } else {
        for (int e = lane; e < hd; e += 32) out[e] = from_f32<T>(b[e]);
    }
}

extern "C" int vl_qk_norm_rope_write(
    void* qkv, int dtype, const int* positions, const int* slots,
    const float* qw, const float* kw, float eps, const float* inv_freq, int rot,
    void* kcache, void* vcache, int T, int nq, int nkv, int hd, int page_size,
    long long num_slots, int row_stride, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd <= 0 || hd > ROPE_MAX_HD || rot < 0 || rot > hd || (rot & 1)) return VL_ERR_UNSUPPORTED;
    if (page_size <= 0 || row_stride < (nq + 2 * nkv) * hd) return VL_ERR_ARGUMENT;
    const int nheads = nq + 2 * nkv;
    dim3 grid(T, (nheads + ROPE_WARPS - 1) / ROPE_WARPS);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(qk_norm_rope_write_kernel<float>, grid, dim3(ROPE_WARPS * 32), 0, s,
            (float*)qkv, positions, slots, qw, kw, eps, inv_freq, rot, (float*)kcache, (float*)vcache,
            nq, nkv, hd, page_size, num_slots, row_stride, err);
    else if (dtype == VL_BF16)
        return vl_launch(qk_norm_rope_write_kernel<bf16>, grid, dim3(ROPE_WARPS * 32), 0, s,
            (bf16*)qkv, positions, slots, qw, kw, eps, inv_freq, rot, (bf16*)kcache, (bf16*)vcache,
            nq, nkv, hd, page_size, num_slots, row_stride, err);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}
