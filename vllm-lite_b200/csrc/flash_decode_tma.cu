// bfloat16 decode attention over the paged cache as a persistent, warp-specialised stream:
// -DFA_HD=64 or 128.  The function and the partial-result layout are those of vl_flash_decode
// (csrc/flash_attn.cu): a token at position p reads the keys lo..p of its request,
//     s_j = (q . k_j) * scale;  p = softmax_j(s);  o = sum_j p_j v_j,
// split into chunks of `chunk` key positions; each (token, KV head, chunk) yields an unnormalised
// partial output with its maximum and sum, merged by vl_decode_attention_merge.
//
// A decode step is bound by one read of the keys and values, and with a block per (token, KV head,
// chunk) each block's start-up (positions, block table, first copies) and wind-down are paid once
// per 128 KB of stream.  Here one block per SM walks many such work items:
//   warp 4   producer: looks up the pages of a work item and copies its K and V rows, 64 keys a
//        stage, by TMA boxes (cp.async.bulk.tensor.3d, 128-byte swizzle, one box per page: its blocks
//        of 64 columns one after the other) into a ring of stages that runs on across work items; it also brings the item's
//        query rows (bulk copies) and its description into one of two slots.  The producer runs
//        ahead of the arithmetic by the depth of the ring, so the start-up of the next item is
//        hidden behind the stream of this one;
//   warps 0..3   consumers: per stage each warp takes 16 of the 64 keys (mma.sync m16n8k16, the query
//        heads of the KV head as rows), keeps its own running maximum, sum and output; at the end of
//        an item the four are merged through shared memory in warp order and written as the item's
//        partial result.
// Keys outside the item's range are masked by position; pages outside it, or that the block table
// does not hold, are fetched from beyond the end of the tensor (zeros); rows of V behind the
// request's last key are zeroed in shared memory (another request's leftovers may be anything).
// Every wait on an mbarrier is bounded; when one expires the block records VL_DEV_WAIT_EXPIRED and
// stops.
#include "tc5.cuh"

#ifndef FA_HD
#define FA_HD 128
#endif

using namespace tc5;

namespace {
constexpr int HD = FA_HD;
static_assert(HD == 64 || HD == 128, "this kernel is built for head sizes 64 and 128");
constexpr int BN = 64, CB = HD / 64, KSTEPS = HD / 16, DTILES = HD / 8;
constexpr int ROWS = 16;                               // query heads per work item (rows of the tensor-core tile)
constexpr int CONSUMERS = 4, NTHREADS = 32 * (CONSUMERS + 1);
constexpr unsigned ROW_BYTES = 128;
constexpr unsigned KV_BYTES = BN * HD * 2;             // K (or V) of a stage: CB blocks of [64 rows][128 bytes]
constexpr unsigned STAGE_BYTES = 2 * KV_BYTES;
constexpr int NST = HD == 128 ? 5 : 8;                 // stages in the ring
constexpr int QLD = HD + 8;                            // padded query row (elements)
constexpr unsigned Q_BYTES = ROWS * QLD * 2;
constexpr int OLD = HD + 4;                            // padded row of the merge buffer (floats)
constexpr unsigned MERGE_BYTES = CONSUMERS * ROWS * OLD * 4;
constexpr unsigned SMEM_BYTES = NST * STAGE_BYTES + MERGE_BYTES + 2 * Q_BYTES + 256;

struct ItemInfo {                                      // what the producer tells the consumers about a work item
    int tok, out_row, h0, nvalid, pos, c0, c1, split;  // out_row: the token's number within the launch
};

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float exp2_mufu(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
}  // namespace

// Work item i = (token z, KV head and head tile y, split x), x fastest; block b takes the items
// b, b + gridDim.x, ...
extern "C" __global__ void __launch_bounds__(NTHREADS, 1)
flash_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, int q_stride,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ req_index, const int* __restrict__ positions,
                        int T, int nq, int nkv, int page_size, int num_pages, float scale_log2, int window,
                        int chunk, int S, float* __restrict__ part_acc, float* __restrict__ part_ml, unsigned* err,
                        const int* __restrict__ token_index) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* ring = smem;                                            // [NST][K | V]
    float* sO = reinterpret_cast<float*>(smem + NST * STAGE_BYTES);        // [4][16][OLD]
    bf16* Qs = reinterpret_cast<bf16*>(smem + NST * STAGE_BYTES + MERGE_BYTES);   // [2][16][QLD]
    unsigned char* tail = smem + NST * STAGE_BYTES + MERGE_BYTES + 2 * Q_BYTES;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(tail);       // [NST]
    unsigned long long* empty = full + NST;                                       // [NST]
    unsigned long long* q_full = empty + NST;                                     // [2]
    unsigned long long* q_empty = q_full + 2;                                     // [2]
    ItemInfo* info = reinterpret_cast<ItemInfo*>(q_empty + 2);                    // [2]
    __shared__ float s_m[CONSUMERS][ROWS], s_l[CONSUMERS][ROWS];
    __shared__ int failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();
    if (smem_u32(smem) & 1023u) {                        // (uniform) never expected; the tiles would be misread
        if (tid == 0 && err) atomicOr(err, VL_DEV_WAIT_EXPIRED);
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < NST; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], CONSUMERS); }
        for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], CONSUMERS); }
        mbar_fence_init();
        failed = 0;
    }
    for (int i = tid; i < 2 * ROWS * QLD / 2; i += NTHREADS) reinterpret_cast<unsigned*>(Qs)[i] = 0u;   // rows no head uses stay zero
    fence_proxy_async_smem();
    __syncthreads();
    const int grp = nq / nkv;
    const int htiles = (grp + ROWS - 1) / ROWS;
    const int ny = nkv * htiles;
    const int num_items = T * ny * S;
    pdl_wait();                                          // q and the cache are written by the kernel before

    if (warp == CONSUMERS) {                             // ---- producer (whole warp) ----
        const int box_rows = page_size < BN ? page_size : BN, nbox = BN / box_rows;
        const int beyond = num_pages * nkv * page_size;  // a row coordinate past the tensor: zeros
        int stage_it = 0;                                // stages issued so far, over all items
        int n = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++n) {
            const int split = item % S, y = (item / S) % ny, z = item / (S * ny);
            const int tok = token_index ? token_index[z] : z;
            const int kvh = y / htiles, htile = y - kvh * htiles;
            const int h0 = kvh * grp + htile * ROWS, nvalid = min(ROWS, grp - htile * ROWS);
            int pos = positions[tok];
            if ((long long)pos >= (long long)S * chunk) {  // beyond the S chunks the launch was sized for: flagged,
                if (lane == 0 && split == 0 && err) atomicOr(err, VL_DEV_BEYOND_BOUND);   // served like an empty place
                pos = -1;
            }
            const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
            const int c0 = max(split * chunk, lo), c1 = min((split + 1) * chunk, pos + 1);
            const int ib = n & 1;
            if (lane == 0 && n >= 2 && !mbar_wait_bounded(&q_empty[ib], (unsigned)((n / 2 - 1) & 1))) ok = false;
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const bool live = pos >= 0 && c0 < c1;
            if (lane == 0) {
                ItemInfo ii;
                ii.tok = tok; ii.out_row = z; ii.h0 = h0; ii.nvalid = nvalid; ii.pos = pos; ii.split = split;
                ii.c0 = c0; ii.c1 = live ? c1 : c0;
                info[ib] = ii;
                mbar_arrive_expect_tx(&q_full[ib], live ? (unsigned)(nvalid * HD * 2) : 0u);
            }
            __syncwarp();
            if (!live) continue;
            if (lane < nvalid)
                bulk_copy_g2s(Qs + (size_t)(ib * ROWS + lane) * QLD, q + (size_t)tok * q_stride + (size_t)(h0 + lane) * HD,
                              HD * 2, &q_full[ib]);
            const int* table = block_table + (size_t)req_index[tok] * max_blocks;
            const int st0 = c0 / BN, st1 = (c1 - 1) / BN;
            // lane b < nbox owns box b of every key tile: the cache row of the box's first key, looked up
            // one tile ahead of its use
            auto lookup = [&](int st) -> int {
                if (lane >= nbox || st > st1) return beyond;
                const int first = st * BN + lane * box_rows;
                if (first >= c1 || first + box_rows - 1 < c0) return beyond;
                const int blk = first / page_size;
                const int page = blk < max_blocks ? table[blk] : -1;
                if (page < 0 || page >= num_pages) {
                    atomicOr(err, VL_DEV_BAD_PAGE);
                    return beyond;
                }
                return (page * nkv + kvh) * page_size + (first - blk * page_size);
            };
            int row = lookup(st0);
            for (int st = st0; st <= st1 && ok; ++st, ++stage_it) {
                const int row_next = lookup(st + 1);
                const int s = stage_it % NST;
                if (lane == 0) {
                    if (stage_it >= NST && !mbar_wait_bounded(&empty[s], (unsigned)((stage_it / NST - 1) & 1))) ok = false;
                    else mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (ok && lane < nbox) {
                    // the box of page b: its blocks of 64 columns one after the other, box_rows rows of 128 bytes each
                    unsigned char* kt = ring + (unsigned)s * STAGE_BYTES + (unsigned)(lane * CB * box_rows) * ROW_BYTES;
                    tma_load_3d(kt, &map_k, 0, row, 0, &full[s]);
                    tma_load_3d(kt + KV_BYTES, &map_v, 0, row, 0, &full[s]);
                }
                row = row_next;
            }
        }
        if (!ok && lane == 0) atomicExch(&failed, 1);
    } else {                                             // ---- consumers ----
        const int g = lane >> 2, t = lane & 3;
        const unsigned ring_u32 = smem_u32(ring);
        const int kr0 = warp * 16;                       // this warp's 16 keys of every stage
        // byte offsets of this lane's ldmatrix rows inside a [64 rows][128 bytes] block and its swizzle
        // a stage holds, for K and for V, box after box (a page, or 64 rows of one), in a box the blocks of
        // 64 columns one after the other, in a block its rows of 128 bytes
        const int box_rows = page_size < BN ? page_size : BN;
        const unsigned blk_bytes = (unsigned)box_rows * ROW_BYTES;           // from one block of 64 columns to the next
        auto row_offset = [&](int r) { return (unsigned)(r / box_rows) * CB * blk_bytes + (unsigned)(r % box_rows) * ROW_BYTES; };
        const unsigned k_row = row_offset(kr0 + (lane & 7) + 8 * (lane >> 4));
        const unsigned v_row = row_offset(kr0 + (lane & 7) + 8 * ((lane >> 3) & 1));
        const unsigned sw = (unsigned)(lane & 7);
        int stage_it = 0, n = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++n) {
            const int ib = n & 1;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(&q_full[ib], (unsigned)((n / 2) & 1)))) { ok = false; break; }
            const ItemInfo ii = info[ib];
            const bool live = ii.c0 < ii.c1;
            unsigned qf[KSTEPS][4];
            if (live) {
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks)
                    ldmatrix_x4(qf[ks], smem_u32(Qs + (size_t)(ib * ROWS + (lane & 7) + 8 * ((lane >> 3) & 1)) * QLD + ks * 16 + 8 * (lane >> 4)));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_empty[ib]);    // the slot may be written again
            if (!live) continue;
            float o[DTILES][4], m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
            for (int d = 0; d < DTILES; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
            const int st0 = ii.c0 / BN, st1 = (ii.c1 - 1) / BN;
            for (int st = st0; st <= st1; ++st, ++stage_it) {
                const int s = stage_it % NST;
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full[s], (unsigned)((stage_it / NST) & 1)))) { ok = false; break; }
                const unsigned kt = ring_u32 + (unsigned)s * STAGE_BYTES, vt = kt + KV_BYTES;
                if (st == st1 && ii.c1 - st * BN < kr0 + 16) {
                    // Slots behind the request's last key hold whatever the page's earlier owner left
                    // there.  Their probabilities are zero, but 0 * NaN is NaN: zero those rows of V
                    // (this warp's 16 rows of the stage; the other warps see to theirs).
                    unsigned char* vs = ring + (unsigned)s * STAGE_BYTES + KV_BYTES;
                    for (int r = max(ii.c1 - st * BN, kr0); r < kr0 + 16; ++r)
                        if (lane < CB * 8)
                            *reinterpret_cast<uint4*>(vs + (unsigned)(lane >> 3) * blk_bytes + row_offset(r) + ((lane & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    fence_proxy_async_smem();            // the stage is next written by the TMA unit
                    __syncwarp();
                }
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    unsigned kb[4];
                    const unsigned chunk16 = (unsigned)(2 * ks + ((lane >> 3) & 1));      // 16-byte piece of the key row
                    ldmatrix_x4(kb, kt + (chunk16 >> 3) * blk_bytes + k_row + (((chunk16 & 7) ^ sw) << 4));
                    mma16816(sc[0], qf[ks], kb[0], kb[1]);
                    mma16816(sc[1], qf[ks], kb[2], kb[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nn = 0; nn < 2; ++nn)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = st * BN + kr0 + nn * 8 + 2 * t + (e & 1);
                        const float v = (j >= ii.c0 && j < ii.c1) ? sc[nn][e] * scale_log2 : -INFINITY;
                        sc[nn][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                float corr[2], base[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    const float mn = fmaxf(m_run[r], mx[r]);
                    base[r] = (mn == -INFINITY) ? 0.f : mn;
                    corr[r] = exp2_mufu(m_run[r] - base[r]);
                    m_run[r] = mn;
                    l_run[r] *= corr[r];
                }
                unsigned pf[4];
                {
                    const float p00 = exp2_mufu(sc[0][0] - base[0]), p01 = exp2_mufu(sc[0][1] - base[0]);
                    const float p02 = exp2_mufu(sc[0][2] - base[1]), p03 = exp2_mufu(sc[0][3] - base[1]);
                    const float p10 = exp2_mufu(sc[1][0] - base[0]), p11 = exp2_mufu(sc[1][1] - base[0]);
                    const float p12 = exp2_mufu(sc[1][2] - base[1]), p13 = exp2_mufu(sc[1][3] - base[1]);
                    l_run[0] += p00 + p01 + p10 + p11;
                    l_run[1] += p02 + p03 + p12 + p13;
                    pf[0] = pack_bf16(p00, p01); pf[1] = pack_bf16(p02, p03);
                    pf[2] = pack_bf16(p10, p11); pf[3] = pack_bf16(p12, p13);
                }
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    unsigned vb[4];
                    const unsigned chunk16 = (unsigned)(2 * dp + (lane >> 4));            // 16-byte piece of the value row
                    ldmatrix_x4_trans(vb, vt + (chunk16 >> 3) * blk_bytes + v_row + (((chunk16 & 7) ^ sw) << 4));
                    o[2 * dp][0] *= corr[0]; o[2 * dp][1] *= corr[0]; o[2 * dp][2] *= corr[1]; o[2 * dp][3] *= corr[1];
                    o[2 * dp + 1][0] *= corr[0]; o[2 * dp + 1][1] *= corr[0]; o[2 * dp + 1][2] *= corr[1]; o[2 * dp + 1][3] *= corr[1];
                    mma16816(o[2 * dp], pf, vb[0], vb[1]);
                    mma16816(o[2 * dp + 1], pf, vb[2], vb[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);   // this warp has read the stage
            }
            if (!ok) break;
            // the four warps' partial results, merged in warp order
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
            }
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                float* pa = sO + ((size_t)warp * ROWS + g) * OLD + d * 8 + 2 * t;
                pa[0] = o[d][0]; pa[1] = o[d][1];
                pa[8 * OLD] = o[d][2]; pa[8 * OLD + 1] = o[d][3];
            }
            if (t == 0) {
                s_m[warp][g] = m_run[0]; s_l[warp][g] = l_run[0];
                s_m[warp][g + 8] = m_run[1]; s_l[warp][g + 8] = l_run[1];
            }
            consumer_barrier();
            for (int idx = tid; idx < ii.nvalid * HD; idx += 32 * CONSUMERS) {
                const int r = idx / HD, e = idx - r * HD;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < CONSUMERS; ++w) M = fmaxf(M, s_m[w][r]);
                float acc = 0.f, L = 0.f;
#pragma unroll
                for (int w = 0; w < CONSUMERS; ++w) {
                    const float wgt = (s_m[w][r] == -INFINITY) ? 0.f : exp2_mufu(s_m[w][r] - M);
                    acc += sO[((size_t)w * ROWS + r) * OLD + e] * wgt;
                    L += s_l[w][r] * wgt;
                }
                const size_t prow = ((size_t)ii.out_row * nq + (ii.h0 + r)) * S + ii.split;
                part_acc[prow * HD + e] = acc;
                if (e == 0) {
                    part_ml[prow * 2] = M * 0.6931471805599453f;           // the merge kernel works in natural-log units
                    part_ml[prow * 2 + 1] = L;
                }
            }
            consumer_barrier();                          // the merge buffer is free for the next item
        }
        if (!ok && lane == 0) atomicExch(&failed, 1);
    }
    __syncthreads();
    if (tid == 0 && failed && err) atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_FLASH_DECODE_TMA);
}

extern "C" int vl_flash_decode_tma_head_dim() { return HD; }

// Arguments and scratch as for vl_flash_decode; page sizes that are a multiple of 8 and divide 64 or
// are a multiple of it.  Follow with vl_decode_attention_merge.
extern "C" int vl_flash_decode_tma(const void* q, int q_stride, const void* kcache, const void* vcache,
                                   const int* block_table, int max_blocks, const int* req_index, const int* positions,
                                   int T, int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                                   int chunk, int S, float* part_acc, float* part_ml, unsigned* err,
                                   const int* token_index, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd != HD) return VL_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0 || num_pages <= 0 || q_stride % 8) return VL_ERR_ARGUMENT;
    if (chunk <= 0 || chunk % BN || S <= 0) return VL_ERR_ARGUMENT;
    if (page_size % 8 || (page_size < BN ? BN % page_size : page_size % BN)) return VL_ERR_UNSUPPORTED;
    if ((((uintptr_t)q | (uintptr_t)kcache | (uintptr_t)vcache) & 15)) return VL_ERR_UNSUPPORTED;
    const long long rows = (long long)num_pages * nkv * page_size;
    const int grp = nq / nkv, htiles = (grp + ROWS - 1) / ROWS;
    const long long items = (long long)T * nkv * htiles * S;
    if (rows + BN >= (1ll << 31) || items >= (1ll << 31)) return VL_ERR_UNSUPPORTED;
    const int box_rows = page_size < BN ? page_size : BN;
    CUtensorMap map_k, map_v;
    int rc = tc5_make_map_blocks(&map_k, kcache, (int)rows, HD, HD, box_rows);
    if (rc) return rc;
    rc = tc5_make_map_blocks(&map_v, vcache, (int)rows, HD, HD, box_rows);
    if (rc) return rc;
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    cudaError_t e = cudaFuncSetAttribute(flash_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    const int grid = (int)(items < num_sms ? items : num_sms);
    return vl_launch(flash_decode_tma_kernel, dim3(grid), dim3(NTHREADS), SMEM_BYTES, (cudaStream_t)stream,
                     map_k, map_v, (const bf16*)q, q_stride, block_table, max_blocks, req_index, positions, T, nq, nkv,
                     page_size, num_pages, scale * 1.4426950408889634f, window, chunk, S, part_acc, part_ml, err, token_index);
}
