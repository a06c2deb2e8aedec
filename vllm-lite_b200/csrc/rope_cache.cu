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
// head_dim up to 512, any even value.
#include "common.cuh"

#define ROPE_MAX_HD 512

// A block serves one token and `heads_per_block` of its heads: its 4 warps share the token's
// sine/cosine table and walk those heads (many tokens: all heads, so the table is computed once per
// token; few tokens: 4 heads, so that a decode step still fills the SMs); a lane handles pairs of neighbouring features (4-byte accesses for
// bfloat16, 8-byte for float32).
#define ROPE_THREADS 128

template <typename T> struct Two;
template <> struct Two<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Two<bf16> {
    static __device__ __forceinline__ float2 load(const bf16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
    static __device__ __forceinline__ void store(bf16* p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    }
};

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_write_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ inv_freq, int rot,
    T* __restrict__ kcache, T* __restrict__ vcache,
    int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err,
    int heads_per_block) {
    __shared__ float buf[ROPE_THREADS / 32][ROPE_MAX_HD];
    __shared__ float s_cos[ROPE_MAX_HD / 2], s_sin[ROPE_MAX_HD / 2];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head_lo = blockIdx.y * heads_per_block;
    const int head_hi = min(nq + 2 * nkv, head_lo + heads_per_block);
    const int half = rot / 2;
    pdl_wait();
    if (inv_freq) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += ROPE_THREADS) sincosf(pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    __syncthreads();
    const int slot = slots ? slots[t] : -1;
    bool slot_ok = slot >= 0;
    if (slot_ok && (long long)slot >= num_slots) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        slot_ok = false;
    }
    const int page = slot_ok ? slot / page_size : 0, off = slot_ok ? slot - page * page_size : 0;
    float* b = buf[warp];
    for (int head = head_lo + warp; head < head_hi; head += ROPE_THREADS / 32) {
        T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
        const bool is_q = head < nq;
        const bool is_k = !is_q && head < nq + nkv;
        const int kvh = is_q ? 0 : (is_k ? head - nq : head - nq - nkv);
        T* dst = nullptr;
        if (!is_q) {
            if (!slot_ok) continue;                       // nothing to write for this token
            dst = (is_k ? kcache : vcache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
        }
        if (!is_q && !is_k) {                             // v: plain copy
            for (int e = 2 * lane; e < hd; e += 64) {
                const float2 v = Two<T>::load(src + e);
                Two<T>::store(dst + e, v.x, v.y);
            }
            continue;
        }
        float ss = 0.f;
        for (int e = 2 * lane; e < hd; e += 64) {
            const float2 v = Two<T>::load(src + e);
            b[e] = v.x; b[e + 1] = v.y;
            ss += v.x * v.x; ss += v.y * v.y;
        }
        const float* w = is_q ? qw : kw;
        if (w) {
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
            for (int e = 2 * lane; e < hd; e += 64) {
                b[e] = b[e] * inv * w[e];
                b[e + 1] = b[e + 1] * inv * w[e + 1];
            }
        }
        __syncwarp();
        T* out = is_q ? src : dst;
        if (inv_freq && half > 0) {
            // a lane takes features (i, i+1) of the first half and their partners in the second half
            for (int i = 2 * lane; i < half; i += 64) {
                const float c0 = s_cos[i], s0 = s_sin[i], x1 = b[i], x2 = b[i + half];
                float y1b = 0.f, y2b = 0.f;
                const float y1a = x1 * c0 - x2 * s0, y2a = x2 * c0 + x1 * s0;
                if (i + 1 < half) {
                    const float c1 = s_cos[i + 1], s1 = s_sin[i + 1], u1 = b[i + 1], u2 = b[i + 1 + half];
                    y1b = u1 * c1 - u2 * s1; y2b = u2 * c1 + u1 * s1;
                }
                if ((half & 1) == 0) {
                    Two<T>::store(out + i, y1a, y1b);
                    Two<T>::store(out + i + half, y2a, y2b);
                } else {                                  // an odd half breaks the pairing of the second half
                    out[i] = from_f32<T>(y1a); out[i + half] = from_f32<T>(y2a);
                    if (i + 1 < half) { out[i + 1] = from_f32<T>(y1b); out[i + 1 + half] = from_f32<T>(y2b); }
                }
            }
            for (int e = rot + 2 * lane; e < hd; e += 64) Two<T>::store(out + e, b[e], b[e + 1]);
        } else {
            for (int e = 2 * lane; e < hd; e += 64) Two<T>::store(out + e, b[e], b[e + 1]);
        }
        __syncwarp();                                     // the buffer is reused for the next head
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
    if (hd & 1) return VL_ERR_UNSUPPORTED;
    const int nheads = nq + 2 * nkv;
    const int heads_per_block = T >= 256 ? nheads : ROPE_THREADS / 32;
    dim3 grid(T, (nheads + heads_per_block - 1) / heads_per_block);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(qk_norm_rope_write_kernel<float>, grid, dim3(ROPE_THREADS), 0, s,
            (float*)qkv, positions, slots, qw, kw, eps, inv_freq, rot, (float*)kcache, (float*)vcache,
            nq, nkv, hd, page_size, num_slots, row_stride, err, heads_per_block);
    else if (dtype == VL_BF16)
        return vl_launch(qk_norm_rope_write_kernel<bf16>, grid, dim3(ROPE_THREADS), 0, s,
            (bf16*)qkv, positions, slots, qw, kw, eps, inv_freq, rot, (bf16*)kcache, (bf16*)vcache,
            nq, nkv, hd, page_size, num_slots, row_stride, err, heads_per_block);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}
