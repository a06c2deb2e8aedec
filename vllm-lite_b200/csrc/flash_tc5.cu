// bfloat16 attention of prompt portions over the paged cache on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in TMEM), compiled for one head size: -DFA_HD=64 or 128.
//
// The function is that of csrc/attention.cu and csrc/flash_attn.cu: a query at absolute position p
// of a request reads the keys lo..p of that request from its pages (lo = 0 or p - window + 1),
//     s_j = (q . k_j) * scale;  p = softmax_j(s);  o = sum_j p_j v_j,
// query head h reads KV head h / (nq / nkv).  Scores, maxima, sums and the output accumulate in
// float32; the probabilities are rounded to bfloat16 for the second product.
//
// A block owns up to 128 consecutive tokens of one request (a tile of the host's list) and one
// query head, and walks that request's keys in tiles of 64.  Roles:
//   warps 0..3 (a thread per query row)   read the scores S = Q K^T of a key tile from TMEM
//        (tcgen05.ld), scale and mask them, keep the running maximum and sum of their row, write
//        P = exp2(S - m) as bfloat16 into shared memory (128-byte swizzled rows, the layout the
//        tensor core reads) and, when a row's maximum has grown by more than 2^8, rescale the
//        output accumulator in TMEM (tcgen05.ld / tcgen05.st);
//   warp 4               TMA producer: the K and V rows of a key tile into two stages each: ONE box
//        (cp.async.bulk.tensor.5d over pages x blocks of columns, 128-byte swizzle) when the tile's
//        pages are neighbours in the pool, else one box per page and 64 columns
//        (cp.async.bulk.tensor.2d); a lane owns a page and looks it up one tile ahead; a page that no query of the tile may read, or
//        that the block table does not hold, is fetched from beyond the end of the tensor, which
//        the TMA unit fills with zeros; the rows of V behind the tile's last key (another request's
//        leftovers, possibly NaN) are zeroed in shared memory once the last key tile has landed;
//   warp 5, one thread   issues S_j = Q K_j^T (M 128, N 64, K = head size; both operands K-major)
//        into one of two score buffers, as soon as the rows of the tile two before have been read,
//        so that scores are computed while the rows of the tile before are exponentiated;
//   warp 6, one thread   issues O += P_j V_j (M 128, N = head size, K 64; V is read as stored, i.e.
//        with its N index contiguous) once P_j lies in shared memory.
// Two blocks fit on an SM (112 KB of shared memory and 256 TMEM columns each at head size 128):
// one block's softmax runs beside the other's products.
// A row keeps a stale maximum until the true one exceeds it by more than 8 (in log2 units): the
// probabilities then reach 2^8 at most, and output and sum are scaled alike, so the quotient is the
// same; the decision is taken row by row, so a row's result does not depend on its neighbours.
// Every wait on an mbarrier is bounded; when one expires the block records VL_DEV_WAIT_EXPIRED,
// stops, and still frees its TMEM.
#include "tc5.cuh"

#ifndef FA_HD
#define FA_HD 128
#endif

using namespace tc5;

namespace {
constexpr int HD = FA_HD;
static_assert(HD == 64 || HD == 128, "this kernel is built for head sizes 64 and 128");
constexpr int BM = 128, BN = 64, CB = HD / 64;       // CB: blocks of 64 columns (one swizzled row) per head
constexpr int NTHREADS = 224;
constexpr unsigned ROW_BYTES = 128;
constexpr unsigned Q_BYTES = BM * HD * 2;            // CB blocks of [128 rows][128 bytes]
constexpr unsigned KV_STAGE = BN * HD * 2;           // CB blocks of [64 rows][128 bytes]
constexpr unsigned P_BYTES = BM * BN * 2;            // [128 rows][128 bytes]
constexpr unsigned TILE_BYTES = Q_BYTES + 4 * KV_STAGE + P_BYTES;
constexpr unsigned SMEM_BYTES = TILE_BYTES + 160;    // + barriers; two blocks per SM only without any slack
constexpr unsigned TMEM_COLS = 256;                  // scores 2 x 64, output HD (a power of two >= their sum)
constexpr unsigned O_COL = 2 * BN;
constexpr float RESCALE_ABOVE = 8.0f;

__device__ __forceinline__ float exp2_mufu(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// two float32 operations in one instruction (sm_100): a register pair holds (x, y)
__device__ __forceinline__ unsigned long long pair(float x, float y) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void unpair(unsigned long long v, float& x, float& y) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// tcgen05.mma with the accumulate flag known at compile time; the descriptors' upper words are the
// same for every tile of a layout, so the issuing thread keeps lower words and adds offsets
template <bool ACC>
__device__ __forceinline__ void mma_lo(unsigned tmem_c, unsigned a_lo, unsigned b_lo, unsigned a_hi, unsigned b_hi, unsigned idesc) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %5, 0;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %6, p;\n}"
        ::"r"(tmem_c), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(ACC ? 1u : 0u), "r"(idesc) : "memory");
}
// byte offset of the 16-byte chunk `chunk` (0..7) of row `row` in a tile of 128-byte swizzled rows
__device__ __forceinline__ unsigned swizzled(int row, int chunk) {
    return (unsigned)row * ROW_BYTES + (unsigned)((chunk ^ (row & 7)) << 4);
}
}  // namespace

// tiles[i] = {row of the block table, index of the tile's first token in the step, tokens (<= 128),
// position of the first}
extern "C" __global__ void __launch_bounds__(NTHREADS, 2)
flash_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 const __grid_constant__ CUtensorMap pages_k, const __grid_constant__ CUtensorMap pages_v, int use_pages,
                 const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                 const int* __restrict__ block_table, int max_blocks, const int4* __restrict__ tiles, int num_tiles,
                 int nq, int nkv, int page_size, int num_pages, float scale_log2, int window, unsigned* err) {
    // tiles of the 128-byte swizzle must start on 1024-byte boundaries; there is no static shared
    // memory in this kernel, so the array starts the block's window
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* Qs = smem;
    unsigned char* Ks = Qs + Q_BYTES;                // 2 stages
    unsigned char* Vs = Ks + 2 * KV_STAGE;           // 2 stages
    unsigned char* Ps = Vs + 2 * KV_STAGE;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + TILE_BYTES);
    unsigned long long *k_full = bars, *k_empty = bars + 2, *v_full = bars + 4, *v_empty = bars + 6, *s_full = bars + 8;
    unsigned long long &p_full = bars[10], &pv_done = bars[11], &v_fixed = bars[12];
    unsigned long long* s_free = bars + 13;
    unsigned& tmem_base_slot = *reinterpret_cast<unsigned*>(bars + 15);
    int& failed = *reinterpret_cast<int*>(bars + 16);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (smem_u32(smem) & 1023u) {                    // (uniform) never expected; the tiles would be misread
        if (tid == 0 && err) atomicOr(err, VL_DEV_WAIT_EXPIRED);
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_free[i], BM);
        }
        mbar_init(&p_full, BM);
        mbar_init(&pv_done, 1);
        mbar_init(&v_fixed, 1);
        mbar_fence_init();
        failed = 0;
    }
    // Tensor memory is taken only after the kernels before this one have completed: a block started as a
    // programmatic dependent then holds nothing of the SM that an earlier kernel may still be waiting for.
    pdl_launch_dependents();
    pdl_wait();                                      // q and the cache are written by the kernel before
    if (warp == 5) tc5_alloc(&tmem_base_slot, TMEM_COLS);
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    // The list is in order of position and blocks start in the order of their number (x fastest): the
    // tiles with the longest rows of keys go first, for all heads, so that the longest blocks do not
    // start last.
    const int4 tile = tiles[num_tiles - 1 - (int)blockIdx.y];
    const int req = tile.x, tok0 = tile.y, count = tile.z, pos0 = tile.w;
    const int h = blockIdx.x, kvh = h / (nq / nkv);
    const int hi = pos0 + count - 1;                             // the last key any row reads
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;   // the first key any row reads
    const int jt0 = lo / BN, n_tiles = hi / BN - jt0 + 1;

    // the query tile, rows beyond `count` zero, into the swizzled layout
    for (int idx = tid; idx < BM * (HD / 8); idx += NTHREADS) {
        const int r = idx / (HD / 8), c = idx - r * (HD / 8);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < count) v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + r) * q_stride + (size_t)h * HD + c * 8);
        *reinterpret_cast<uint4*>(Qs + (unsigned)(c >> 3) * (BM * ROW_BYTES) + swizzled(r, c & 7)) = v;
    }
    fence_proxy_async_smem();
    __syncthreads();

    if (warp == 4) {                                             // ---- TMA producer (whole warp) ----
        const int* table = block_table + (size_t)req * max_blocks;
        const int box_rows = page_size < BN ? page_size : BN, nbox = BN / box_rows;
        const int beyond = num_pages * nkv * page_size;          // a row coordinate past the tensor: zeros
        // lane b < nbox owns box b of every key tile: the cache row of the box's first key, looked up
        // one tile ahead of its use
        auto lookup = [&](int it) -> int {
            if (lane >= nbox || it >= n_tiles) return beyond;
            const int first = (jt0 + it) * BN + lane * box_rows;
            if (first > hi || first + box_rows - 1 < lo) return beyond;
            const int blk = first / page_size;
            const int page = blk < max_blocks ? table[blk] : -1;
            if (page < 0 || page >= num_pages) {
                atomicOr(err, VL_DEV_BAD_PAGE);
                return beyond;
            }
            return (page * nkv + kvh) * page_size + (first - blk * page_size);
        };
        // Order of the copies = order in which their stages come free: the scores of tile i + 1 are
        // issued before the second product of tile i, so keys run one tile ahead of values.
        int row_k = lookup(0), row_v = beyond;
        bool ok = true;
        for (int step = 0; step <= n_tiles && ok; ++step) {
            const int row_next = lookup(step + 1);
            for (int kv = 0; kv < 2 && ok; ++kv) {
                const int it = kv ? step - 1 : step;
                if (it < 0 || it >= n_tiles) continue;
                const int s = it & 1;
                unsigned long long* full = kv ? &v_full[s] : &k_full[s];
                if (lane == 0) {
                    if (it >= 2 && !mbar_wait_bounded(kv ? &v_empty[s] : &k_empty[s], (unsigned)((it / 2 - 1) & 1))) ok = false;
                    else mbar_arrive_expect_tx(full, KV_STAGE);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                // The pages of the tile are neighbours in the pool (the usual case: the pool hands pages out in
                // a row) and all of them are read: one box brings them all.  Else a box per page and block of
                // columns.
                const int row = kv ? row_v : row_k;
                const int row0 = __shfl_sync(0xffffffffu, row, 0);
                const bool in_a_row = use_pages && __all_sync(0xffffffffu, lane >= nbox || (row != beyond && row == row0 + lane * nkv * page_size));
                if (ok && in_a_row) {
                    if (lane == 0)
                        tma_load_5d((kv ? Vs : Ks) + (unsigned)s * KV_STAGE, kv ? &pages_v : &pages_k, 0, 0,
                                    row0 / (nkv * page_size), 0, kvh, full);
                } else if (ok && lane < nbox) {
                    unsigned char* st = (kv ? Vs : Ks) + (unsigned)s * KV_STAGE + (unsigned)(lane * box_rows) * ROW_BYTES;
                    for (int cb = 0; cb < CB; ++cb)
                        tma_load_2d(st + (unsigned)cb * (BN * ROW_BYTES), kv ? &map_v : &map_k, cb * 64, row, full);
                }
            }
            row_v = row_k;
            row_k = row_next;
        }
        // Slots behind the request's last key hold whatever the page's earlier owner left there.  Their
        // probabilities are zero, but 0 * NaN is NaN: zero those rows of V of the last key tile.
        const int last = n_tiles - 1, first_bad = hi + 1 - (jt0 + last) * BN;
        if (ok && first_bad < BN) {
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&v_full[last & 1], (unsigned)((last / 2) & 1)));
            if (ok) {
                unsigned char* vs = Vs + (unsigned)(last & 1) * KV_STAGE;
                for (int r = first_bad; r < BN; ++r)
                    if (lane < CB * 8)
                        *reinterpret_cast<uint4*>(vs + (unsigned)(lane >> 3) * (BN * ROW_BYTES) + (unsigned)r * ROW_BYTES + ((lane & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                fence_proxy_async_smem();
                __syncwarp();
            }
        }
        if (lane == 0) {
            if (ok) mbar_arrive(&v_fixed);
            else atomicExch(&failed, 1);
        }
    } else if (warp == 5) {
        if (lane == 0) {                                         // ---- issuer of the scores S = Q K^T ----
            constexpr unsigned idesc_qk = make_idesc(BM, BN);
            // descriptors: upper words once, lower words (the address field, in 16-byte units) by addition
            const unsigned long long dq = make_smem_desc(Qs), dk = make_smem_desc(Ks);
            const unsigned q_lo = (unsigned)dq, k_lo = (unsigned)dk, kmaj_hi = (unsigned)(dq >> 32);
            bool ok = true;
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it & 1;
                // the score buffer is free once every row of the tile two before has been read
                if ((it >= 2 && !mbar_wait_bounded(&s_free[s], (unsigned)((it / 2 - 1) & 1))) ||
                    !mbar_wait_bounded(&k_full[s], (unsigned)((it / 2) & 1))) { ok = false; break; }
                tc5_fence_after();
                const unsigned kb = k_lo + (unsigned)s * (KV_STAGE >> 4), tc = tmem_base + (unsigned)(s * BN);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    // 16 columns further on: 32 bytes inside the swizzled row; 64 columns: the next block of rows
                    const unsigned qo = (unsigned)(ks >> 2) * (BM * ROW_BYTES >> 4) + (unsigned)(ks & 3) * 2;
                    const unsigned ko = (unsigned)(ks >> 2) * (BN * ROW_BYTES >> 4) + (unsigned)(ks & 3) * 2;
                    if (ks == 0) mma_lo<false>(tc, q_lo + qo, kb + ko, kmaj_hi, kmaj_hi, idesc_qk);
                    else mma_lo<true>(tc, q_lo + qo, kb + ko, kmaj_hi, kmaj_hi, idesc_qk);
                }
                tc5_commit(&k_empty[s]);
                tc5_commit(&s_full[s]);
            }
            if (!ok) atomicExch(&failed, 1);
        }
    } else if (warp == 6) {
        if (lane == 0) {                                         // ---- issuer of the output O += P V ----
            constexpr unsigned idesc_pv = make_idesc(BM, HD) | IDESC_B_MN_MAJOR;
            const unsigned long long dp = make_smem_desc(Ps);
            const unsigned long long dv = make_smem_desc_lbo_sbo(Vs, BN * ROW_BYTES, 8 * ROW_BYTES);
            const unsigned p_lo = (unsigned)dp, v_lo = (unsigned)dv;
            const unsigned kmaj_hi = (unsigned)(dp >> 32), v_hi = (unsigned)(dv >> 32);
            bool ok = true;
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it & 1;
                if (!mbar_wait_bounded(&p_full, (unsigned)(it & 1)) ||
                    !mbar_wait_bounded(&v_full[s], (unsigned)((it / 2) & 1)) ||
                    (it == n_tiles - 1 && !mbar_wait_bounded(&v_fixed, 0u))) { ok = false; break; }
                tc5_fence_after();
                const unsigned vb = v_lo + (unsigned)s * (KV_STAGE >> 4);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    // 16 keys further on: 32 bytes inside a row of P, 16 rows of 128 bytes of V
                    if (k == 0 && it == 0) mma_lo<false>(tmem_base + O_COL, p_lo, vb, kmaj_hi, v_hi, idesc_pv);
                    else mma_lo<true>(tmem_base + O_COL, p_lo + (unsigned)k * 2, vb + (unsigned)k * (16 * ROW_BYTES >> 4), kmaj_hi, v_hi, idesc_pv);
                }
                tc5_commit(&v_empty[s]);
                tc5_commit(&pv_done);
            }
            if (!ok) atomicExch(&failed, 1);
        }
    } else {                                                     // ---- softmax: a thread per query row ----
        const int row = warp * 32 + lane;
        const int qpos = pos0 + row;
        const int first_key = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
        const unsigned lane_base = (unsigned)(warp * 32) << 16;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it & 1;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(&s_full[s], (unsigned)((it / 2) & 1)))) { ok = false; break; }
            tc5_fence_after();
            unsigned sv[BN];
            tc5_ld32_nowait(tmem_base + lane_base + (unsigned)(s * BN), sv);
            tc5_ld32_nowait(tmem_base + lane_base + (unsigned)(s * BN + 32), sv + 32);
            tc5_wait_ld();
            tc5_fence_before();
            mbar_arrive(&s_free[s]);                             // the scores are in registers: the buffer may be written again
            const int j0 = (jt0 + it) * BN;
            // (warp-uniform) does any row of this warp see a key of the tile that it must not read?
            const bool edge = (j0 + BN - 1 > pos0 + warp * 32) || (window > 0 && j0 < pos0 + warp * 32 + 31 - window + 1);
            float mx = -INFINITY;
            if (edge) {
#pragma unroll
                for (int c = 0; c < BN; ++c)
                    if (j0 + c > qpos || j0 + c < first_key) sv[c] = 0xff800000u;     // -inf
            }
#pragma unroll
            for (int c = 0; c < BN; c += 2) mx = max3(mx, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
            const float m_new = fmaxf(m, mx * scale_log2);       // the scale is positive
            const bool bump = (m_new - m) > RESCALE_ABOVE;       // false when both are -inf (NaN compares false)
            const float corr = bump ? exp2_mufu(m - m_new) : 1.0f;
            if (bump) m = m_new;
            const float base = (m == -INFINITY) ? 0.f : m;
            const unsigned long long scale2 = pair(scale_log2, scale_log2), nbase2 = pair(-base, -base);
            unsigned pk[BN / 2];
            unsigned long long sum2 = pair(0.f, 0.f);
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                float t0, t1;
                unpair(fma2(pair(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, nbase2), t0, t1);
                const float p0 = exp2_mufu(t0), p1 = exp2_mufu(t1);
                sum2 = add2(sum2, pair(p0, p1));
                pk[c >> 1] = pack_bf16(p0, p1);
            }
            float sum, sum_hi;
            unpair(sum2, sum, sum_hi);
            sum += sum_hi;
            l = l * corr + sum;
            if (it > 0) {                                        // P of the tile before has been read, O is at rest
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(&pv_done, (unsigned)((it - 1) & 1)))) { ok = false; break; }
                tc5_fence_after();
                if (__any_sync(0xffffffffu, bump)) {
#pragma unroll
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        unsigned ov[32];
                        tc5_ld32(tmem_base + lane_base + O_COL + (unsigned)c0, ov);
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                        tc5_st32(tmem_base + lane_base + O_COL + (unsigned)c0, ov);
                    }
                    tc5_wait_st();
                }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(Ps + swizzled(row, c)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            fence_proxy_async_smem();
            tc5_fence_before();
            mbar_arrive(&p_full);
        }
        if (ok && __all_sync(0xffffffffu, mbar_wait_bounded(&pv_done, (unsigned)((n_tiles - 1) & 1)))) {
            tc5_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = out + ((size_t)(tok0 + row) * nq + h) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 32) {
                unsigned ov[32];
                tc5_ld32(tmem_base + lane_base + O_COL + (unsigned)c0, ov);
                if (row < count) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * i) = w;
                    }
                }
            }
        } else {
            atomicExch(&failed, 1);
        }
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    if (warp == 5) tc5_dealloc(tmem_base, TMEM_COLS);
    if (tid == 0 && failed && err) atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_FLASH_TC5);
}

extern "C" int vl_flash_tc5_head_dim() { return HD; }

// Takes page sizes that are a multiple of 8 and divide 64 or are a multiple of it; q rows and `out`
// rows must be 16-byte aligned.  Other sizes: VL_ERR_UNSUPPORTED (csrc/flash_attn.cu takes them).
extern "C" int vl_flash_prefill_tc5(const void* q, int q_stride, void* out, const void* kcache, const void* vcache,
                                    const int* block_table, int max_blocks, const int* tiles, int num_tiles,
                                    int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                                    unsigned* err, void* stream) {
    if (num_tiles <= 0) return VL_OK;
    if (hd != HD) return VL_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0 || num_pages <= 0) return VL_ERR_ARGUMENT;
    if (page_size % 8 || (page_size < BN ? BN % page_size : page_size % BN)) return VL_ERR_UNSUPPORTED;
    if (q_stride % 8 || (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kcache | (uintptr_t)vcache) & 15)) return VL_ERR_UNSUPPORTED;
    if (num_tiles > 65535) return VL_ERR_UNSUPPORTED;
    const long long rows = (long long)num_pages * nkv * page_size;
    if (rows + BN >= (1ll << 31)) return VL_ERR_UNSUPPORTED;
    const int box_rows = page_size < BN ? page_size : BN;
    CUtensorMap map_k, map_v;
    int rc = tc5_make_map(&map_k, kcache, (int)rows, HD, HD, box_rows);
    if (rc) return rc;
    rc = tc5_make_map(&map_v, vcache, (int)rows, HD, HD, box_rows);
    if (rc) return rc;
    // pages smaller than a key tile: a second pair of maps whose box spans the tile's pages when they are neighbours
    CUtensorMap pages_k = map_k, pages_v = map_v;
    const int use_pages = page_size < BN ? 1 : 0;
    if (use_pages) {
        rc = tc5_make_map_pages(&pages_k, kcache, num_pages, nkv, page_size, HD, BN / page_size);
        if (rc) return rc;
        rc = tc5_make_map_pages(&pages_v, vcache, num_pages, nkv, page_size, HD, BN / page_size);
        if (rc) return rc;
    }
    cudaError_t e = cudaFuncSetAttribute(flash_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    return vl_launch(flash_tc5_kernel, dim3(nq, num_tiles), dim3(NTHREADS), SMEM_BYTES, (cudaStream_t)stream,
                     map_k, map_v, pages_k, pages_v, use_pages, (const bf16*)q, q_stride, (bf16*)out, block_table, max_blocks, (const int4*)tiles,
                     num_tiles, nq, nkv, page_size, num_pages, scale * 1.4426950408889634f, window, err);
}
