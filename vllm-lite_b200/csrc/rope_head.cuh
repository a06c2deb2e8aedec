// One head of q, k or v in a warp's registers: per-head RMS norm (optional), rotary position encoding of the
// first `rot` features (optional), store.  Shared by the kernel that does this for all heads of a step
// (csrc/rope_cache.cu) and by the decode attention, which does it for its own heads while it loads them
// (csrc/flash_attn.cu): the same code, so the same bits.
//   head <- head / sqrt(mean(head^2) + eps) * w;   pairs (x[i], x[i + rot/2]):
//   x1' = x1 cos - x2 sin,  x2' = x2 cos + x1 sin,  angle = (float)pos * inv_freq[i]
// A lane holds pairs of neighbouring features (4-byte accesses for bfloat16, 8-byte for float32) of the
// first rotated half together with their partners in the second half, and pairs of the features behind
// the rotated part: per lane at most MAXHD / 128 pairs of the first half and MAXHD / 64 pairs behind.
#pragma once
#include "common.cuh"

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

