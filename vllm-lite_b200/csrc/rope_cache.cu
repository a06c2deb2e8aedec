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
#include "rope_head.cuh"

#define ROPE_MAX_HD 512

// A block serves one token and `heads_per_block` of its heads: its 4 warps share the token's
// sine/cosine table and walk those heads (many tokens: all heads, so the table is computed once per
// token; few tokens: 4 heads, so that a decode step still fills the SMs).  A warp keeps a head in
// registers: a lane holds pairs of neighbouring features (4-byte accesses for bfloat16, 8-byte for
// float32) of the first rotated half together with their partners in the second half, and pairs of
// the features behind the rotated part.  A warp works on two heads at a time, so that the loads of
// one overlap the arithmetic of the other.
#define ROPE_THREADS 128
// The kernel is compiled for head sizes up to MAXHD = 128 and up to ROPE_MAX_HD: per lane at most
// MAXHD / 128 pairs of the first half and MAXHD / 64 pairs behind the rotated part.

template <typename T, int MAXHD>
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_write_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ inv_freq, int rot,
    T* __restrict__ kcache, T* __restrict__ vcache,
    int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err,
    int heads_per_block) {
    __shared__ float s_cos[MAXHD / 2], s_sin[MAXHD / 2];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head_lo = blockIdx.y * heads_per_block;
    const int head_hi = min(nq + 2 * nkv, head_lo + heads_per_block);
    const int half = rot / 2;
    if (inv_freq) {                                  // positions are part of the step's description: no wait needed
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += ROPE_THREADS) sincosf(pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    pdl_wait();                                      // qkv comes from the kernel before
    __syncthreads();
    const int slot = slots ? slots[t] : -1;
    bool slot_ok = slot >= 0;
    if (slot_ok && (long long)slot >= num_slots) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        slot_ok = false;
    }
    const int page = slot_ok ? slot / page_size : 0, off = slot_ok ? slot - page * page_size : 0;
    // where head `head` of this token is read and written, which norm weight it takes, whether it is rotated
    auto setup = [&](HeadRegs<T, MAXHD>& r, int head) {
        r.live = head < head_hi;
        r.src = qkv; r.out = qkv; r.w = nullptr; r.rot = 0;
        if (!r.live) return;
        r.src = qkv + (size_t)t * row_stride + (size_t)head * hd;
        const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
        if (is_q) {
            r.out = qkv + (size_t)t * row_stride + (size_t)head * hd;
        } else {
            if (!slot_ok) { r.live = false; return; }             // nothing to write for this token
            const int kvh = is_k ? head - nq : head - nq - nkv;
            r.out = (is_k ? kcache : vcache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
        }
        if (is_q || is_k) {
            r.w = is_q ? qw : kw;
            r.rot = inv_freq ? rot : 0;
        }
    };
    constexpr int WARPS = ROPE_THREADS / 32;
    for (int head = head_lo + warp; head < head_hi; head += 2 * WARPS) {
        HeadRegs<T, MAXHD> r0, r1;
        setup(r0, head);
        setup(r1, head + WARPS);
        r0.load(lane, hd);
        r1.load(lane, hd);
        r0.finish(lane, hd, eps, s_cos, s_sin);
        r1.finish(lane, hd, eps, s_cos, s_sin);
    }
}

// ---- many tokens, the whole head rotated (or none of it), head size 32 .. 512 a power of two ----
// The same function with 16-byte accesses: hd / 16 lanes share a head, a lane holds 8 neighbouring
// features of the first half and their 8 partners in the second half, so a warp works on 512 / hd
// heads at once and on two such groups in flight.  (The kernel above reads 4 bytes per lane and
// load, which leaves a prompt portion's traffic far below what the memory can deliver.)
template <typename T> struct Eight;
template <> struct Eight<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Eight<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = q;
    }
};

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_write_wide_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ inv_freq, T* __restrict__ kcache, T* __restrict__ vcache,
    int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err) {
    __shared__ float s_cos[ROPE_MAX_HD / 2], s_sin[ROPE_MAX_HD / 2];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = hd / 2;
    const int lph = hd / 16, hpw = 32 / lph;                      // lanes per head, heads per warp
    const int nheads = nq + 2 * nkv;
    if (inv_freq) {                                  // positions are part of the step's description: no wait needed
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += ROPE_THREADS) sincosf(pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    pdl_wait();                                      // qkv comes from the kernel before
    __syncthreads();
    const int slot = slots ? slots[t] : -1;
    bool slot_ok = slot >= 0;
    if (slot_ok && (long long)slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        slot_ok = false;
    }
    const int page = slot_ok ? slot / page_size : 0, off = slot_ok ? slot - page * page_size : 0;
    const int sub = lane / lph, i0 = 8 * (lane % lph);             // which head of the warp's group, first feature
    constexpr int WARPS = ROPE_THREADS / 32;
    const int per_pass = WARPS * hpw;
    for (int base = 0; base < nheads; base += 2 * per_pass) {
        float a[2][8], b[2][8];
        T* out[2];
        const float* w[2];
        bool live[2], rotate[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int head = base + u * per_pass + warp * hpw + sub;
            live[u] = head < nheads;
            out[u] = nullptr; w[u] = nullptr; rotate[u] = false;
            if (live[u]) {
                T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
                const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
                if (is_q) out[u] = src;
                else if (slot_ok) out[u] = (is_k ? kcache : vcache) + (((size_t)page * nkv + (is_k ? head - nq : head - nq - nkv)) * page_size + off) * hd;
                else live[u] = false;                              // nothing to write for this token
                if (live[u]) {
                    Eight<T>::load(src + i0, a[u]);
                    Eight<T>::load(src + i0 + half, b[u]);
                    if (is_q || is_k) { w[u] = is_q ? qw : kw; rotate[u] = inv_freq != nullptr; }
                }
            }
            if (!live[u]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { a[u][j] = 0.f; b[u][j] = 0.f; }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            // (every lane takes part in the shuffles; lanes of a head agree on w)
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += a[u][j] * a[u][j] + b[u][j] * b[u][j];
            for (int o = 1; o < lph; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (!live[u]) continue;
            if (w[u]) {
                const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
                for (int j = 0; j < 8; ++j) { a[u][j] *= inv * w[u][i0 + j]; b[u][j] *= inv * w[u][i0 + half + j]; }
            }
            if (rotate[u]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float c = s_cos[i0 + j], sn = s_sin[i0 + j], x1 = a[u][j], x2 = b[u][j];
                    a[u][j] = x1 * c - x2 * sn;
                    b[u][j] = x2 * c + x1 * sn;
                }
            }
            Eight<T>::store(out[u] + i0, a[u]);
            Eight<T>::store(out[u] + i0 + half, b[u]);
        }
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
    cudaStream_t s = (cudaStream_t)stream;
    const bool pow2 = (hd & (hd - 1)) == 0 && hd >= 32;
    const bool aligned = row_stride % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache) & 31) == 0;
    // (bfloat16 only: in float32 one kernel serves every step, so that a token's result does not depend,
    // not even in its last bit, on how many tokens share the step)
    if (T >= 256 && pow2 && aligned && (rot == hd || !inv_freq) && dtype == VL_BF16)
        return vl_launch(qk_norm_rope_write_wide_kernel<bf16>, dim3(T), dim3(ROPE_THREADS), 0, s, (bf16*)qkv, positions,
                         slots, qw, kw, eps, inv_freq, (bf16*)kcache, (bf16*)vcache, nq, nkv, hd, page_size,
                         num_slots, row_stride, err);
    const int heads_per_block = T >= 256 ? nheads : ROPE_THREADS / 32;
    dim3 grid(T, (nheads + heads_per_block - 1) / heads_per_block);
#define ROPE_LAUNCH(TYPE, MAXHD)                                                                           \
    return vl_launch(qk_norm_rope_write_kernel<TYPE, MAXHD>, grid, dim3(ROPE_THREADS), 0, s,               \
        (TYPE*)qkv, positions, slots, qw, kw, eps, inv_freq, rot, (TYPE*)kcache, (TYPE*)vcache,            \
        nq, nkv, hd, page_size, num_slots, row_stride, err, heads_per_block)
    if (dtype == VL_F32) {
        if (hd <= 128) ROPE_LAUNCH(float, 128);
        ROPE_LAUNCH(float, ROPE_MAX_HD);
    }
    if (dtype == VL_BF16) {
        if (hd <= 128) ROPE_LAUNCH(bf16, 128);
        ROPE_LAUNCH(bf16, ROPE_MAX_HD);
    }
#undef ROPE_LAUNCH
    return VL_ERR_UNSUPPORTED;
}
