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
// token; few tokens: 4 heads, so that a decode step still fills the SMs).  A warp keeps a head in
// registers: a lane holds pairs of neighbouring features (4-byte accesses for bfloat16, 8-byte for
// float32) of the first rotated half together with their partners in the second half, and pairs of
// the features behind the rotated part.  A warp works on two heads at a time, so that the loads of
// one overlap the arithmetic of the other.
#define ROPE_THREADS 128
// The kernel is compiled for head sizes up to MAXHD = 128 and up to ROPE_MAX_HD: per lane at most
// MAXHD / 128 pairs of the first half and MAXHD / 64 pairs behind the rotated part.

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

// One head in a warp's registers.
template <typename T, int MAXHD>
struct HeadRegs {
    static constexpr int ROPE_ROT_UNITS = MAXHD / 128, ROPE_TAIL_UNITS = MAXHD / 64;
    float2 a[ROPE_ROT_UNITS], b[ROPE_ROT_UNITS], t[ROPE_TAIL_UNITS];
    const T* src;
    T* out;
    const float* w;      // norm weight or null
    int rot;             // rotated features of this head (0: none)
    bool live;

    // `half_even`: the second half starts on a pair boundary, so partners are loaded as pairs too
    __device__ __forceinline__ void load(int lane, int hd) {
        const int half = rot / 2;
        const bool half_even = (half & 1) == 0;
#pragma unroll
        for (int k = 0; k < ROPE_ROT_UNITS; ++k) {
            const int i = 2 * (lane + 32 * k);
            a[k] = make_float2(0.f, 0.f); b[k] = make_float2(0.f, 0.f);
            if (live && i < half) {
                if (half_even) {
                    a[k] = Two<T>::load(src + i);
                    b[k] = Two<T>::load(src + i + half);
                } else {
                    a[k].x = to_f32(src[i]); b[k].x = to_f32(src[i + half]);
                    if (i + 1 < half) { a[k].y = to_f32(src[i + 1]); b[k].y = to_f32(src[i + 1 + half]); }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < ROPE_TAIL_UNITS; ++k) {
            const int e = rot + 2 * (lane + 32 * k);
            t[k] = (live && e < hd) ? Two<T>::load(src + e) : make_float2(0.f, 0.f);
        }
    }

    __device__ __forceinline__ void finish(int lane, int hd, float eps, const float* s_cos, const float* s_sin) {
        const int half = rot / 2;
        const bool half_even = (half & 1) == 0;
        if (w) {                                          // (warp-uniform)
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < ROPE_ROT_UNITS; ++k) ss += a[k].x * a[k].x + a[k].y * a[k].y + b[k].x * b[k].x + b[k].y * b[k].y;
#pragma unroll
            for (int k = 0; k < ROPE_TAIL_UNITS; ++k) ss += t[k].x * t[k].x + t[k].y * t[k].y;
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
            for (int k = 0; k < ROPE_ROT_UNITS; ++k) {
                const int i = 2 * (lane + 32 * k);
                if (i < half) {
                    a[k].x *= inv * w[i]; b[k].x *= inv * w[i + half];
                    if (i + 1 < half) { a[k].y *= inv * w[i + 1]; b[k].y *= inv * w[i + 1 + half]; }
                }
            }
#pragma unroll
            for (int k = 0; k < ROPE_TAIL_UNITS; ++k) {
                const int e = rot + 2 * (lane + 32 * k);
                if (e < hd) { t[k].x *= inv * w[e]; t[k].y *= inv * w[e + 1]; }
            }
        }
        if (!live) return;
#pragma unroll
        for (int k = 0; k < ROPE_ROT_UNITS; ++k) {
            const int i = 2 * (lane + 32 * k);
            if (i < half) {
                const float c0 = s_cos[i], s0 = s_sin[i];
                const float y1a = a[k].x * c0 - b[k].x * s0, y2a = b[k].x * c0 + a[k].x * s0;
                float y1b = 0.f, y2b = 0.f;
                if (i + 1 < half) {
                    const float c1 = s_cos[i + 1], s1 = s_sin[i + 1];
                    y1b = a[k].y * c1 - b[k].y * s1; y2b = b[k].y * c1 + a[k].y * s1;
                }
                if (half_even) {
                    Two<T>::store(out + i, y1a, y1b);
                    Two<T>::store(out + i + half, y2a, y2b);
                } else {
                    out[i] = from_f32<T>(y1a); out[i + half] = from_f32<T>(y2a);
                    if (i + 1 < half) { out[i + 1] = from_f32<T>(y1b); out[i + 1 + half] = from_f32<T>(y2b); }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < ROPE_TAIL_UNITS; ++k) {
            const int e = rot + 2 * (lane + 32 * k);
            if (e < hd) Two<T>::store(out + e, t[k].x, t[k].y);
        }
    }
};

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
