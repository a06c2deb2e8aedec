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

// ---------------------------------------------------------------------------------------
// Decode attention with the key range split across blocks.
//
// vl_decode_attention: for steps in which every request brings few tokens (decoding).
// A block serves one token, up to GT query heads that share a KV head (so a key is read
// once for all of them) and one chunk of `chunk` key positions; chunk c covers the
// absolute positions [c*chunk, (c+1)*chunk), so which keys meet in a block depends on
// positions alone.  Inside, 16 groups of 8 lanes own the keys whose position is the
// group's number modulo 16; a lane holds 16-byte pieces of the rows.  The groups' running
// softmax states are merged by a fixed butterfly, the blocks' partial results by a second
// kernel in chunk order.  Partials are float32 scratch memory given by the caller:
//   part_acc [T, nq, S, hd] (unnormalised), part_ml [T, nq, S, 2] (maximum, sum).
// ---------------------------------------------------------------------------------------
#define DEC_THREADS 128

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    uint4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { raw = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ float get(int i) const {
        const unsigned w = i == 0 ? raw.x : i == 1 ? raw.y : i == 2 ? raw.z : raw.w;
        return __uint_as_float(w);
    }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { raw = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ float get(int i) const {
        const unsigned w = (i >> 1) == 0 ? raw.x : (i >> 1) == 1 ? raw.y : (i >> 1) == 2 ? raw.z : raw.w;
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));   // bfloat16 is the top half of a float
    }
};

template <typename T> __device__ __forceinline__ float att_exp(float x);
template <> __device__ __forceinline__ float att_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float att_exp<bf16>(float x) { return __expf(x); }

// ---- asynchronous bulk copies (TMA, untiled) with mbarrier completion -----------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// A wait gives up after a bounded number of polls and of cycles (common.cuh) instead of hanging the device.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 0; i < VL_WAIT_POLL_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (vl_wait_gave_up(i, t0)) return false;
    }
    return false;
}

#define DEC_STAGE_KEYS 32
#define DEC_MAX_STAGES 4

// Keys and values of DEC_STAGE_KEYS consecutive positions are one stage of a ring in shared
// memory, filled by bulk copies of the page pieces that cover them (a page piece of one KV head
// is contiguous: rows x head_dim).  Thread 0 issues the copies; everybody consumes.
template <typename T, int NPASS, int GT>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_split_kernel(const T* __restrict__ q, int q_stride,
                              const T* __restrict__ kcache, const T* __restrict__ vcache,
                              const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ req_index, const int* __restrict__ positions,
                              int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                              int chunk, int S, int nstages, float* __restrict__ part_acc,
                              float* __restrict__ part_ml, unsigned* err) {
    constexpr int EPV = Vec16<T>::N;
    extern __shared__ __align__(128) unsigned char dec_smem[];
    __shared__ float s_acc[DEC_THREADS / 32][GT][ATT_MAX_HD];
    __shared__ float s_m[DEC_THREADS / 32][GT], s_l[DEC_THREADS / 32][GT];
    __shared__ __align__(8) unsigned long long full_bar[DEC_MAX_STAGES];
    const int split = blockIdx.x, t = blockIdx.z;
    const int g = nq / nkv;
    const int tiles = (g + GT - 1) / GT;
    const int kvh = blockIdx.y / tiles, tile = blockIdx.y - kvh * tiles;
    const int h0 = kvh * g + tile * GT;
    const int nvalid = min(GT, g - tile * GT);
    const int pos = positions[t];
    if (pos < 0) return;
    if ((long long)pos >= (long long)S * chunk) {         // beyond what the scratch was sized for: flagged, and
        if (threadIdx.x == 0 && split == 0 && err) atomicOr(err, VL_DEV_BEYOND_BOUND);   // the merge writes zeros
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int c0 = max(split * chunk, lo);
    const int c1 = min((split + 1) * chunk, pos + 1);
    if (c0 >= c1) return;
    const int tid = threadIdx.x, gi = tid >> 3, l = tid & 7, warp = tid >> 5;
    const int nvec = hd / EPV;                           // 16-byte pieces per row
    const int* table = block_table + (size_t)req_index[t] * max_blocks;
    const size_t tile_elems = (size_t)DEC_STAGE_KEYS * hd;         // one of K or V of a stage
    T* ring = reinterpret_cast<T*>(dec_smem);

    const int st0 = c0 / DEC_STAGE_KEYS, st1 = (c1 - 1) / DEC_STAGE_KEYS;
    if (tid == 0) {
        for (int i = 0; i < nstages; ++i) mbar_init(&full_bar[i], 1);
        mbar_fence_init();
    }
    __syncthreads();

    // thread 0: fill ring slot `buf` with the keys/values of stage `st`
    auto issue = [&](int st, int buf) {
        const int first = st * DEC_STAGE_KEYS;
        const int last = min(first + DEC_STAGE_KEYS, pos + 1);           // positions beyond pos are never read
        const int need = (c0 / page_size) * page_size;                   // pages wholly below the range may be gone
        unsigned total = 0;
        for (int p0 = first; p0 < last;) {
            const int blk = p0 / page_size;
            const int end = min(last, (blk + 1) * page_size);
            const int page = blk < max_blocks ? table[blk] : -1;
            if (end > need && page >= 0 && page < num_pages) total += 2u * (unsigned)((end - p0) * hd * (int)sizeof(T));
            p0 = end;
        }
        mbar_arrive_expect_tx(&full_bar[buf], total);
        T* kdst = ring + (size_t)buf * 2 * tile_elems;
        T* vdst = kdst + tile_elems;
        for (int p0 = first; p0 < last;) {
            const int blk = p0 / page_size;
            const int end = min(last, (blk + 1) * page_size);
            const int page = blk < max_blocks ? table[blk] : -1;
            if (end <= need) {
                // below the range: nothing to fetch
            } else if (page >= 0 && page < num_pages) {
                const size_t src = (((size_t)page * nkv + kvh) * page_size + (p0 - blk * page_size)) * hd;
                const unsigned bytes = (unsigned)((end - p0) * hd * (int)sizeof(T));
                bulk_copy_g2s(kdst + (size_t)(p0 - first) * hd, kcache + src, bytes, &full_bar[buf]);
                bulk_copy_g2s(vdst + (size_t)(p0 - first) * hd, vcache + src, bytes, &full_bar[buf]);
            } else {
                atomicOr(err, VL_DEV_BAD_PAGE);
            }
            p0 = end;
        }
    };
    if (tid == 0)
        for (int i = 0; i < nstages && st0 + i <= st1; ++i) issue(st0 + i, i);

    float qv[GT][NPASS][EPV], acc[GT][NPASS][EPV], m[GT], lsum[GT];
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
        m[hh] = -INFINITY; lsum[hh] = 0.f;
#pragma unroll
        for (int p = 0; p < NPASS; ++p) {
            Vec16<T> v; v.zero();
            const int c = l + 8 * p;
            if (hh < nvalid && c < nvec) v.load(q + (size_t)t * q_stride + (size_t)(h0 + hh) * hd + c * EPV);
#pragma unroll
            for (int i = 0; i < EPV; ++i) { qv[hh][p][i] = v.get(i) * scale; acc[hh][p][i] = 0.f; }
        }
    }
    for (int st = st0; st <= st1; ++st) {
        const int it = st - st0;
        const int buf = it % nstages;
        const bool arrived = mbar_wait_bounded(&full_bar[buf], (unsigned)((it / nstages) & 1));
        if (__syncthreads_or(!arrived)) {                 // the copy never came: flag it and leave
            if (tid == 0) {
                atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_DECODE_ATTENTION);
                // give the copies that are still in flight a bounded time to land before the block's
                // shared memory is handed to another block
                for (int k = 1; k < nstages && st + k <= st1; ++k)
                    mbar_wait_bounded(&full_bar[(it + k) % nstages], (unsigned)(((it + k) / nstages) & 1));
            }
            return;
        }
        const T* kt = ring + (size_t)buf * 2 * tile_elems;
        const T* vt = kt + tile_elems;
#pragma unroll
        for (int half = 0; half < DEC_STAGE_KEYS / ATT_GROUPS; ++half) {
            const int r = half * ATT_GROUPS + gi;          // row of the stage
            const int j = st * DEC_STAGE_KEYS + r;
            const bool valid = (j >= c0) && (j < c1);
            Vec16<T> kr[NPASS], vr[NPASS];
#pragma unroll
            for (int p = 0; p < NPASS; ++p) {
                kr[p].zero(); vr[p].zero();
                const int c = l + 8 * p;
                if (valid && c < nvec) {
                    kr[p].load(kt + (size_t)r * hd + c * EPV);
                    vr[p].load(vt + (size_t)r * hd + c * EPV);
                }
            }
            float dot[GT];
#pragma unroll
            for (int hh = 0; hh < GT; ++hh) {
                float d = 0.f;
#pragma unroll
                for (int p = 0; p < NPASS; ++p)
#pragma unroll
                    for (int i = 0; i < EPV; ++i) d = fmaf(qv[hh][p][i], kr[p].get(i), d);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                dot[hh] = d;
            }
            if (valid) {
#pragma unroll
                for (int hh = 0; hh < GT; ++hh) {
                    const float sc = dot[hh];
                    const float mn = fmaxf(m[hh], sc);
                    const float corr = att_exp<T>(m[hh] - mn);
                    const float pr = att_exp<T>(sc - mn);
                    lsum[hh] = lsum[hh] * corr + pr;
                    m[hh] = mn;
#pragma unroll
                    for (int p = 0; p < NPASS; ++p)
#pragma unroll
                        for (int i = 0; i < EPV; ++i) acc[hh][p][i] = fmaf(pr, vr[p].get(i), acc[hh][p][i] * corr);
                }
            }
        }
        __syncthreads();                                   // everybody is done with this slot
        if (tid == 0 && st + nstages <= st1) issue(st + nstages, buf);
    }
    // merge the 4 groups of a warp (lanes l, l+8, l+16, l+24 hold the same pieces)
#pragma unroll
    for (int hh = 0; hh < GT; ++hh) {
#pragma unroll
        for (int o = 8; o <= 16; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[hh], o);
            const float lo_ = __shfl_xor_sync(0xffffffffu, lsum[hh], o);
            const float mn = fmaxf(m[hh], mo);
            const float wa = (m[hh] == -INFINITY) ? 0.f : att_exp<T>(m[hh] - mn);
            const float wb = (mo == -INFINITY) ? 0.f : att_exp<T>(mo - mn);
            lsum[hh] = lsum[hh] * wa + lo_ * wb;
#pragma unroll
            for (int p = 0; p < NPASS; ++p)
#pragma unroll
                for (int i = 0; i < EPV; ++i) {
                    const float ao = __shfl_xor_sync(0xffffffffu, acc[hh][p][i], o);
                    acc[hh][p][i] = acc[hh][p][i] * wa + ao * wb;
                }
            m[hh] = mn;
        }
        if (gi % 4 == 0) {
#pragma unroll
            for (int p = 0; p < NPASS; ++p) {
                const int c = l + 8 * p;
                if (c < nvec) {
#pragma unroll
                    for (int i = 0; i < EPV; ++i) s_acc[warp][hh][c * EPV + i] = acc[hh][p][i];
                }
            }
            if (l == 0) { s_m[warp][hh] = m[hh]; s_l[warp][hh] = lsum[hh]; }
        }
    }
    __syncthreads();
    // merge the warps in order and write the block's partial result
    for (int idx = tid; idx < nvalid * hd; idx += DEC_THREADS) {
        const int hh = idx / hd, e = idx - hh * hd;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_THREADS / 32; ++w) M = fmaxf(M, s_m[w][hh]);
        float o = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_THREADS / 32; ++w) {
            const float wgt = (s_m[w][hh] == -INFINITY) ? 0.f : att_exp<T>(s_m[w][hh] - M);
            o += s_acc[w][hh][e] * wgt;
            L += s_l[w][hh] * wgt;
        }
        const size_t row = ((size_t)t * nq + (h0 + hh)) * S + split;
        part_acc[row * hd + e] = o;
        if (e == 0) { part_ml[row * 2] = M; part_ml[row * 2 + 1] = L; }
    }
}

template <typename T>
__global__ void decode_attention_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                              const int* __restrict__ positions, T* __restrict__ out,
                                              int nq, int hd, int chunk, int S, int window,
                                              const int* __restrict__ token_index) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;                    // t numbers the tokens of the launch
    const int tok = token_index ? token_index[t] : t;            // ... tok those of the step
    const int pos = positions[tok];
    T* op = out + ((size_t)tok * nq + h) * hd;
    // a padded place of the batch, or a position beyond the S chunks that were computed (the split pass
    // has flagged that): zeros, never a read outside this row's partial results
    if (pos < 0 || (long long)pos >= (long long)S * chunk) {
        for (int e = threadIdx.x; e < hd; e += blockDim.x) op[e] = from_f32<T>(0.f);
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int s0 = lo / chunk, s1 = pos / chunk;
    const size_t row0 = ((size_t)t * nq + h) * S;
    float M = -INFINITY;
    for (int s = s0; s <= s1; ++s) M = fmaxf(M, part_ml[(row0 + s) * 2]);
    float L = 0.f;
    for (int s = s0; s <= s1; ++s) {
        const float ms = part_ml[(row0 + s) * 2];
        L += (ms == -INFINITY) ? 0.f : part_ml[(row0 + s) * 2 + 1] * att_exp<T>(ms - M);
    }
    const float invL = L > 0.f ? 1.0f / L : 0.f;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        float o = 0.f;
        for (int s = s0; s <= s1; ++s) {
            const float ms = part_ml[(row0 + s) * 2];
            if (ms != -INFINITY) o += part_acc[(row0 + s) * hd + e] * att_exp<T>(ms - M);
        }
        op[e] = from_f32<T>(o * invL);
    }
}

template <typename T, int NPASS>
static int launch_decode_split(int GT, dim3 grid, cudaStream_t s, const T* q, int q_stride, const T* kc, const T* vc,
                               const int* bt, int max_blocks, const int* req, const int* pos, int nq, int nkv, int hd,
                               int page_size, int num_pages, float scale, int window, int chunk, int S,
                               float* pacc, float* pml, unsigned* err) {
    const size_t stage_bytes = 2 * (size_t)DEC_STAGE_KEYS * hd * sizeof(T);
    int nstages = (int)((96 * 1024) / stage_bytes);
    nstages = nstages > DEC_MAX_STAGES ? DEC_MAX_STAGES : (nstages < 2 ? 2 : nstages);
    const size_t smem = stage_bytes * nstages;
#define DEC_CASE(G)                                                                                        \
    case G: {                                                                                              \
        auto kern = decode_attention_split_kernel<T, NPASS, G>;                                            \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e;                                                               \
        kern<<<grid, DEC_THREADS, smem, s>>>(q, q_stride, kc, vc, bt, max_blocks, req, pos, nq, nkv, hd,   \
                                             page_size, num_pages, scale, window, chunk, S, nstages, pacc, \
                                             pml, err);                                                    \
        break;                                                                                             \
    }
    switch (GT) { DEC_CASE(1) DEC_CASE(2) DEC_CASE(4) default: return VL_ERR_UNSUPPORTED; }
#undef DEC_CASE
    return vl_launch_status();
}

template <typename T>
static int decode_attention_typed(const T* q, int q_stride, T* out, const T* kc, const T* vc, const int* bt,
                                  int max_blocks, const int* req, const int* pos, int T_, int nq, int nkv, int hd,
                                  int page_size, int num_pages, float scale, int window, int chunk, int S,
                                  float* pacc, float* pml, unsigned* err, cudaStream_t s) {
    constexpr int EPV = Vec16<T>::N;
    const int g = nq / nkv;
    // heads per block: as many of the group as keep a lane's registers (hd / 8 values per head) in bounds
    int GT = g >= 4 ? 4 : (g >= 2 ? 2 : 1);
    while (GT > 1 && GT * (hd / 8) > 64) GT >>= 1;
    const int tiles = (g + GT - 1) / GT;
    const int npass = (hd / EPV + 7) / 8;
    dim3 grid(S, nkv * tiles, T_);
    int rc;
#define DEC_PASS(P)                                                                                         \
    case P:                                                                                                 \
        rc = launch_decode_split<T, P>(GT, grid, s, q, q_stride, kc, vc, bt, max_blocks, req, pos, nq, nkv, \
                                       hd, page_size, num_pages, scale, window, chunk, S, pacc, pml, err);  \
        break;
    if (npass * EPV > 32) return VL_ERR_UNSUPPORTED;      // head_dim beyond 256
    switch (npass) {
        DEC_PASS(1) DEC_PASS(2) DEC_PASS(3) DEC_PASS(4)
        default:
            if constexpr (EPV == 4) {
                switch (npass) { DEC_PASS(5) DEC_PASS(6) DEC_PASS(7) DEC_PASS(8) default: return VL_ERR_UNSUPPORTED; }
            } else {
                return VL_ERR_UNSUPPORTED;
            }
    }
#undef DEC_PASS
    if (rc != 0) return rc;
    decode_attention_merge_kernel<T><<<dim3(T_, nq), 128, 0, s>>>(pacc, pml, pos, out, nq, hd, chunk, S, window, nullptr);
    return vl_launch_status();
}

// Merges per-chunk partial results (of vl_decode_attention's first pass or of vl_flash_decode).
extern "C" int vl_decode_attention_merge(const float* part_acc, const float* part_ml, const int* positions, void* out,
                                         int dtype, int T, int nq, int hd, int chunk, int S, int window,
                                         const int* token_index, void* stream) {
    if (T <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(decode_attention_merge_kernel<float>, dim3(T, nq), dim3(128), 0, s, part_acc, part_ml, positions,
                         (float*)out, nq, hd, chunk, S, window, token_index);
    if (dtype == VL_BF16)
        return vl_launch(decode_attention_merge_kernel<bf16>, dim3(T, nq), dim3(128), 0, s, part_acc, part_ml, positions,
                         (bf16*)out, nq, hd, chunk, S, window, token_index);
    return VL_ERR_UNSUPPORTED;
}

// Scratch: part_acc holds T*nq*S*hd floats and part_ml T*nq*S*2 floats, S = ceil(max_context / chunk),
// where max_context bounds positions + 1 of every token of the step.
extern "C" int vl_decode_attention(const void* q, int q_stride, void* out, int dtype,
                                   const void* kcache, const void* vcache,
                                   const int* block_table, int max_blocks,
                                   const int* req_index, const int* positions,
                                   int T, int nq, int nkv, int hd, int page_size, int num_pages,
                                   float scale, int window, int chunk, int S,
                                   float* part_acc, float* part_ml, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd <= 0 || hd % 16 || hd > ATT_MAX_HD) return VL_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0) return VL_ERR_ARGUMENT;
    if (chunk <= 0 || chunk % ATT_GROUPS || S <= 0 || S > 65535 || T > 65535) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return decode_attention_typed<float>((const float*)q, q_stride, (float*)out, (const float*)kcache,
                                             (const float*)vcache, block_table, max_blocks, req_index, positions,
                                             T, nq, nkv, hd, page_size, num_pages, scale, window, chunk, S,
                                             part_acc, part_ml, err, s);
    if (dtype == VL_BF16)
        return decode_attention_typed<bf16>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)kcache,
                                            (const bf16*)vcache, block_table, max_blocks, req_index, positions,
                                            T, nq, nkv, hd, page_size, num_pages, scale, window, chunk, S,
                                            part_acc, part_ml, err, s);
    return VL_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// vl_decode_attention_no_alloc: vl_decode_attention with its scratch inside the library.
// See attention_no_alloc.h for who needs it and for the limits.
// ---------------------------------------------------------------------------------------------
#include "attention_no_alloc.h"

// Partial results of the split pass: first the accumulators, then the (maximum, sum) pairs.
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) float vl_no_alloc_scratch[VL_NO_ALLOC_SCRATCH_FLOATS];

// Device address of the array, per device, looked up on the first call there.
static float* vl_no_alloc_address[VL_NO_ALLOC_MAX_DEVICES];

extern "C" int vl_decode_attention_no_alloc(const void* q, int q_stride, void* out, int dtype,
                                            const void* kcache, const void* vcache,
                                            const int* block_table, int max_blocks,
                                            const int* req_index, const int* positions,
                                            int T, int nq, int nkv, int hd, int page_size, int num_pages,
                                            float scale, int window, int chunk, int S,
                                            unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (nq <= 0 || hd <= 0 || S <= 0) return VL_ERR_ARGUMENT;
    const unsigned long long acc_floats = (unsigned long long)T * nq * S * hd;
    const unsigned long long ml_floats = (unsigned long long)T * nq * S * 2;
    if (acc_floats + ml_floats > VL_NO_ALLOC_SCRATCH_FLOATS) return VL_ERR_SCRATCH;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= VL_NO_ALLOC_MAX_DEVICES) return VL_ERR_UNSUPPORTED;
    float* scratch = vl_no_alloc_address[device];
    if (scratch == nullptr) {                       // first call on this device (which is current)
        e = cudaGetSymbolAddress((void**)&scratch, vl_no_alloc_scratch);
        if (e != cudaSuccess) return (int)e;
        vl_no_alloc_address[device] = scratch;
    }
    return vl_decode_attention(q, q_stride, out, dtype, kcache, vcache, block_table, max_blocks, req_index,
                               positions, T, nq, nkv, hd, page_size, num_pages, scale, window, chunk, S,
                               scratch, scratch + acc_floats, err, stream);
}
