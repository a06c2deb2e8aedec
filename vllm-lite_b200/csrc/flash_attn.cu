// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, float32
// accumulation), compiled for one head size: -DFA_HD=<head_dim>, a multiple of 16 up to 256.
//
// The function is that of csrc/attention.cu: a query at absolute position p of a request reads
// the keys lo..p of that request from its pages (lo = 0 or p - window + 1),
//     s_j = (q . k_j) * scale;  p = softmax_j(s);  o = sum_j p_j v_j,
// query head h reads KV head h / (nq / nkv).  Scores, running maximum, sum and output are
// float32; the probabilities are rounded to bfloat16 for the second product.
//
// vl_flash_prefill: a block owns up to 64 consecutive tokens of one request and one query head
//   (4 warps x 16 rows) and walks that request's keys in tiles of 64, K and V tiles double
//   buffered in shared memory by cp.async.  The host passes the list of token tiles; a tile of
//   more than 64 tokens is shared out among several blocks.
// vl_flash_decode: a block owns one token, one KV head with all its query heads, and one chunk of
//   `chunk` key positions; its 4 warps take 16 keys each of every 64-key tile, each through a copy
//   ring of its own, and their partial results are merged in warp order.  For groups of up to 8
//   query heads the keys are the rows of the tensor-core tiles and the heads their columns.  The
//   chunks of a token are merged by the blocks of a cluster (up to 16), by the block that arrives
//   last, or (scratch layout of vl_decode_attention) by vl_decode_attention_merge.
// vl_flash_decode_fused: the same, doing the step's head norm, rotation and cache write on the way.
// Rows of shared-memory tiles are padded by 16 bytes, which makes every 8-row ldmatrix access
// hit 8 different banks groups for any head size.
#include "rope_head.cuh"

#ifndef FA_HD
#define FA_HD 128
#endif

namespace {
constexpr int HD = FA_HD;
constexpr int LDS = HD + 8;            // padded row length in elements
constexpr int KSTEPS = HD / 16;        // k-steps of Q K^T
constexpr int DTILES = HD / 8;         // n-tiles of the output
constexpr int CPR = HD / 8;            // 16-byte chunks per row
constexpr int BM = 64, BN = 64, NTHREADS = 128;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16 up to 256");

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;      // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x for x <= 0 on the special-function unit: one MUFU.EX2, no range fix-ups (x = -inf gives 0).
__device__ __forceinline__ float exp2_mufu(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Row of the cache ([pages, nkv, page_size, HD] seen as rows of HD) that holds position j of the
// request, or -1 when j lies outside [first, last] (such rows are filled with zeros and never looked
// up: their pages may not exist, or may have been given back once a window passed them).
__device__ __forceinline__ int cache_row(const int* table, int max_blocks, int j, int first, int last, int kvh,
                                         int nkv, int page_size, int num_pages, unsigned* err) {
    if (j < first || j > last) return -1;
    const int blk = j / page_size;
    const int page = blk < max_blocks ? table[blk] : -1;
    if (page < 0 || page >= num_pages) {
        atomicOr(err, VL_DEV_BAD_PAGE);
        return -1;
    }
    return (page * nkv + kvh) * page_size + (j - blk * page_size);
}

// Copies `rows` rows of keys and of values into two padded tiles; rowidx[r] is the cache row of
// tile row r (or -1: zeros).
__device__ __forceinline__ void load_kv_tiles(bf16* ktile, bf16* vtile, const bf16* kcache, const bf16* vcache,
                                              const int* rowidx, int rows) {
    for (int idx = threadIdx.x; idx < rows * CPR; idx += NTHREADS) {
        const int r = idx / CPR, c = idx - r * CPR;
        const int row = rowidx[r];
        const size_t off = row < 0 ? 0 : (size_t)row * HD + c * 8;
        cp_async16(ktile + (size_t)r * LDS + c * 8, kcache + off, row >= 0);
        cp_async16(vtile + (size_t)r * LDS + c * 8, vcache + off, row >= 0);
    }
}
}  // namespace

// tiles[i] = {row of the block table, index of the tile's first token in the step, tokens, position of the first};
// blocks (h, y) serve head h and, of the list walked from its end, the tokens 64 * (y' % parts) ... of tile y' / parts
extern "C" __global__ void __launch_bounds__(NTHREADS)
flash_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                     const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                     const int* __restrict__ block_table, int max_blocks, const int4* __restrict__ tiles, int parts,
                     int nq, int nkv, int page_size, int num_pages, float scale_log2, int window, unsigned* err) {
    extern __shared__ __align__(128) unsigned char fa_smem[];
    bf16* Qs = reinterpret_cast<bf16*>(fa_smem);                 // [BM][LDS]
    bf16* Ks = Qs + BM * LDS;                                    // [2][BN][LDS]
    bf16* Vs = Ks + 2 * BN * LDS;                                // [2][BN][LDS]
    __shared__ int s_rows[2][BN];                                // cache rows of the tile being loaded / the next one
    // blocks start in the order of their number (x fastest); the list is in order of position, so it
    // is walked from its end: the tiles with the longest rows of keys start first, for all heads
    const int which = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int4 tile = tiles[which / parts];
    const int part0 = (which % parts) * BM;
    if (part0 >= tile.z) return;
    const int req = tile.x, tok0 = tile.y + part0, count = min(BM, tile.z - part0), pos0 = tile.w + part0;
    const int h = blockIdx.x, kvh = h / (nq / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int* table = block_table + (size_t)req * max_blocks;
    const int hi = pos0 + count - 1;                             // the last key any row reads
    const int lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kt_lo = lo / BN, kt_hi = hi / BN;

    for (int idx = tid; idx < BM * CPR; idx += NTHREADS) {       // the query tile (rows beyond count: zeros)
        const int r = idx / CPR, c = idx - r * CPR;
        const bool valid = r < count;
        const bf16* src = valid ? q + (size_t)(tok0 + r) * q_stride + (size_t)h * HD + c * 8 : q;
        cp_async16(Qs + (size_t)r * LDS + c * 8, src, valid);
    }
    if (tid < BN) {
        s_rows[0][tid] = cache_row(table, max_blocks, kt_lo * BN + tid, lo, hi, kvh, nkv, page_size, num_pages, err);
        s_rows[1][tid] = cache_row(table, max_blocks, (kt_lo + 1) * BN + tid, lo, hi, kvh, nkv, page_size, num_pages, err);
    }
    __syncthreads();
    load_kv_tiles(Ks, Vs, kcache, vcache, s_rows[0], BN);
    cp_async_commit();

    float o[DTILES][4], m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DTILES; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    unsigned qf[KSTEPS][4];
    const int row0 = warp * 16;                                  // this warp's rows of the tile
    const int pos_a = pos0 + row0 + g, pos_b = pos_a + 8;        // positions of the lane's two rows
    const bool row_a = row0 + g < count, row_b = row0 + g + 8 < count;

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        if (kt + 1 <= kt_hi) {
            load_kv_tiles(Ks + (buf ^ 1) * BN * LDS, Vs + (buf ^ 1) * BN * LDS, kcache, vcache, s_rows[buf ^ 1], BN);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // rows of tile kt + 2 (read after the barrier that ends this round; slot `buf` is no longer in use)
        if (tid < BN && kt + 2 <= kt_hi)
            s_rows[buf][tid] = cache_row(table, max_blocks, (kt + 2) * BN + tid, lo, hi, kvh, nkv, page_size, num_pages, err);
        if (kt == kt_lo) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks)
                ldmatrix_x4(qf[ks], Qs + (size_t)(row0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks * 16 + 8 * (lane >> 4));
        }
        const bf16* Kt = Ks + buf * BN * LDS;
        const bf16* Vt = Vs + buf * BN * LDS;
        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {               // two key n-tiles per ldmatrix.x4
                unsigned kb[4];
                ldmatrix_x4(kb, Kt + (size_t)(np * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
                mma16816(s[2 * np], qf[ks], kb[0], kb[1]);
                mma16816(s[2 * np + 1], qf[ks], kb[2], kb[3]);
            }
        }
        // mask and online softmax.  The running maximum is kept in units of log2 (score * scale * log2 e);
        // the scale is applied inside the exponent: p = 2^(s * scale_log2 - base).
        const int j_base = kt * BN + 2 * t;
        const bool need_mask = (kt * BN + BN - 1 > pos0 + row0) || (window > 0) || !row_a || !row_b;
        float mx[2] = {-INFINITY, -INFINITY};
        if (need_mask) {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j_base + n * 8 + (e & 1);
                    const int p = (e < 2) ? pos_a : pos_b;
                    const bool rv = (e < 2) ? row_a : row_b;
                    if (!rv || j > p || (window > 0 && j <= p - window)) s[n][e] = -INFINITY;
                }
            }
        }
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
        }
        float corr[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(m_run[r], mx[r] * scale_log2);       // scale_log2 > 0 keeps the order
            base[r] = (mn == -INFINITY) ? 0.f : mn;              // a row with no key yet: 2^(-inf - 0) = 0
            corr[r] = exp2_mufu(m_run[r] - base[r]);
            m_run[r] = mn;
            l_run[r] *= corr[r];
        }
        float ls[2] = {0.f, 0.f};
        unsigned pf[BN / 16][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            const float p0 = exp2_mufu(fmaf(s[n][0], scale_log2, -base[0])), p1 = exp2_mufu(fmaf(s[n][1], scale_log2, -base[0]));
            const float p2 = exp2_mufu(fmaf(s[n][2], scale_log2, -base[1])), p3 = exp2_mufu(fmaf(s[n][3], scale_log2, -base[1]));
            ls[0] += p0 + p1;
            ls[1] += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_run[0] += ls[0];
        l_run[1] += ls[1];
        // once the maxima have settled the correction is 1 for every row of the warp: skip the rescale
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1];
            }
        }
#pragma unroll
        for (int kb16 = 0; kb16 < BN / 16; ++kb16) {
#pragma unroll
            for (int dp = 0; dp < DTILES / 2; ++dp) {            // two d n-tiles per ldmatrix.x4.trans
                unsigned vb[4];
                ldmatrix_x4_trans(vb, Vt + (size_t)(kb16 * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                mma16816(o[2 * dp], pf[kb16], vb[0], vb[1]);
                mma16816(o[2 * dp + 1], pf[kb16], vb[2], vb[3]);
            }
        }
        __syncthreads();                                         // the tile may be overwritten next round
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    if (row_a) {
        bf16* op = out + ((size_t)(tok0 + row0 + g) * nq + h) * HD + 2 * t;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) *reinterpret_cast<unsigned*>(op + d * 8) = pack_bf16(o[d][0] * inv_a, o[d][1] * inv_a);
    }
    if (row_b) {
        bf16* op = out + ((size_t)(tok0 + row0 + g + 8) * nq + h) * HD + 2 * t;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) *reinterpret_cast<unsigned*>(op + d * 8) = pack_bf16(o[d][2] * inv_b, o[d][3] * inv_b);
    }
}

extern "C" int vl_flash_head_dim() { return HD; }

extern "C" int vl_flash_prefill(const void* q, int q_stride, void* out, const void* kcache, const void* vcache,
                                const int* block_table, int max_blocks, const int* tiles, int num_tiles, int tile_rows,
                                int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                                unsigned* err, void* stream) {
    if (num_tiles <= 0) return VL_OK;
    if (hd != HD) return VL_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0 || q_stride % 8) return VL_ERR_ARGUMENT;
    if (tile_rows <= 0 || tile_rows > 65536) return VL_ERR_ARGUMENT;
    const int parts = (tile_rows + BM - 1) / BM;                 // blocks per tile of the list
    if ((long long)num_tiles * parts > 65535) return VL_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(BM + 4 * BN) * LDS * sizeof(bf16);
    cudaError_t e = cudaFuncSetAttribute(flash_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    flash_prefill_kernel<<<dim3(nq, num_tiles * parts), NTHREADS, smem, (cudaStream_t)stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, (const bf16*)kcache, (const bf16*)vcache, block_table, max_blocks,
        (const int4*)tiles, parts, nq, nkv, page_size, num_pages, scale * 1.4426950408889634f, window, err);
    return vl_launch_status();
}

// ---------------------------------------------------------------------------------------------
// decode: one token, one KV head (rows = its query heads), one chunk of key positions per block
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int DEC_NST = (HD <= 128) ? 3 : 2;         // stages of 64 keys (K and V) in the ring
constexpr int DEC_ROWS = 16;                         // query heads per block (rows of the tensor-core tile)
constexpr int DEC_MAX_CHUNK = 1024;                  // most key positions per block
}

namespace {
__device__ __forceinline__ unsigned dec_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned dec_map_to_rank(unsigned local_addr, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
// (volatile keeps it behind the cluster's barrier; no memory clobber, so that several can be in flight)
__device__ __forceinline__ float dec_ld_cluster(unsigned cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
    return v;
}
__device__ __forceinline__ void dec_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
constexpr int DEC_MAX_CLUSTER = 16;                  // most chunks of a token that a cluster merges (8 is the portable cluster
                                                     // size; 16 where the device takes it: vl_flash_decode_max_cluster)

// The chunks of a token and its heads are the blocks of one cluster.  Every block has left its partial
// result in its shared memory (bO [rows][HD], bM maxima in units of log2, bL sums); block `rank` of
// the S merges an S-th of the elements, the chunks in their order, through the cluster's shared
// window, and writes them to the output rows.
__device__ __forceinline__ void decode_cluster_merge(const float* bO, const float* bM, const float* bL, bf16* out,
                                                     int tok, int nq, int h0, int nvalid, int S, int rank, int tid) {
    __syncthreads();
    dec_cluster_sync();
    unsigned aO[DEC_MAX_CLUSTER], aM[DEC_MAX_CLUSTER], aL[DEC_MAX_CLUSTER];
#pragma unroll
    for (int s = 0; s < DEC_MAX_CLUSTER; ++s) {
        const unsigned r = (unsigned)min(s, S - 1);
        aO[s] = dec_map_to_rank(dec_smem_u32(bO), r);
        aM[s] = dec_map_to_rank(dec_smem_u32(bM), r);
        aL[s] = dec_map_to_rank(dec_smem_u32(bL), r);
    }
    const int total = nvalid * HD, per = (total + S - 1) / S;
    const int end = min(total, (rank + 1) * per);
    for (int idx = rank * per + tid; idx < end; idx += NTHREADS) {
        const int r = idx / HD;
        float m[DEC_MAX_CLUSTER], l[DEC_MAX_CLUSTER], a[DEC_MAX_CLUSTER];
#pragma unroll
        for (int s = 0; s < DEC_MAX_CLUSTER; ++s) {              // all loads first: they are in flight together
            m[s] = s < S ? dec_ld_cluster(aM[s] + (unsigned)(r * 4)) : -INFINITY;
            l[s] = s < S ? dec_ld_cluster(aL[s] + (unsigned)(r * 4)) : 0.f;
            a[s] = s < S ? dec_ld_cluster(aO[s] + (unsigned)(idx * 4)) : 0.f;
        }
        float M = m[0];
#pragma unroll
        for (int s = 1; s < DEC_MAX_CLUSTER; ++s) M = fmaxf(M, m[s]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int s = 0; s < DEC_MAX_CLUSTER; ++s) {              // the order of the chunks
            const float wgt = (m[s] == -INFINITY) ? 0.f : exp2_mufu(m[s] - M);
            L += l[s] * wgt;
            acc += a[s] * wgt;
        }
        out[((size_t)tok * nq + h0 + r) * HD + (idx - r * HD)] = __float2bfloat16(acc * (L > 0.f ? 1.0f / L : 0.f));
    }
    dec_cluster_sync();                                          // no block leaves while another may still read its result
}
}  // namespace

// What the decode kernel does on the way when the step's head norm, rotation and cache write are folded into it
// (on != 0): q, the new token's k and its v are then still as the projection left them.  A block norms and
// rotates its own query heads while it brings them into shared memory; the block whose chunk holds the token's
// own position does the same for the token's key, copies its value, writes both to their slot of the cache
// (slots == null: a call that reads another call's cache writes nothing) and lays them over the row of the
// tile that its copy of the cache brought, which may not hold them yet.  The arithmetic is HeadRegs
// (csrc/rope_head.cuh), as in the kernel that serves whole steps: the same bits.
struct DecodeFusion {
    const float* qw; const float* kw; float eps;         // head norm weights (null: none)
    const float* inv_freq; int rot;                      // rotary frequencies (null: none), rotated features
    const int* slots; long long num_slots;               // cache slot of every token of the step
    bf16* kcache; bf16* vcache;                          // the cache again, to write
    int on;
};

// TR: the products are taken the other way round, S^T = K Q^T and O^T = V^T P^T: the 16 keys of a warp's tile are
// the 16 rows of the tensor-core tile and the query heads of the KV head its 8 columns (for groups of up
// to 8 heads; with heads as rows, 16 of them, a group of 4 wastes three quarters of every product): half the
// products, half the accumulators and half the exponentials per key.
template <bool TR>
__global__ void __launch_bounds__(NTHREADS)
flash_decode_kernel(const bf16* __restrict__ q, int q_stride,
                    const bf16* kcache, const bf16* vcache,
                    const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ req_index, const int* __restrict__ positions,
                    int nq, int nkv, int page_size, int num_pages, float scale_log2, int window,
                    int chunk, int S, float* __restrict__ part_acc, float* __restrict__ part_ml, unsigned* err,
                    const int* __restrict__ token_index, bf16* __restrict__ out, int* __restrict__ arrivals,
                    int in_cluster, DecodeFusion fz) {
    extern __shared__ __align__(128) unsigned char fa_dec_smem[];
    bf16* Qs = reinterpret_cast<bf16*>(fa_dec_smem);             // [16][LDS]
    bf16* ring = Qs + DEC_ROWS * LDS;                            // [NST][2][BN][LDS]
    constexpr int RMAX = HD <= 128 ? 128 : 256;                  // HeadRegs is built for head sizes up to this
    __shared__ float s_cos[RMAX / 2], s_sin[RMAX / 2];           // (fz.on) the token's rotation
    __shared__ __align__(16) bf16 s_new[2][HD];                  // (fz.on) the token's own key and value, finished
    __shared__ float s_m[4][DEC_ROWS], s_l[4][DEC_ROWS];
    __shared__ float s_bm[DEC_ROWS], s_bl[DEC_ROWS];             // (in_cluster) the block's maxima and sums
    float* bO = reinterpret_cast<float*>(ring) + 4 * DEC_ROWS * (HD + 4);    // ... and its output sums [rows][HD]
    __shared__ int s_rows[DEC_MAX_CHUNK + BN];                   // cache rows of the chunk's positions, tile aligned
    pdl_launch_dependents();
    // What follows reads the step's description only (positions, block tables: uploaded before the
    // step's first kernel); the wait for the kernel before stands where q and the cache are first read.
    // token_index (optional) picks the tokens of the step that this launch serves; partial results
    // are stored by the number of the token within the launch
    const int split = blockIdx.x, tok = token_index ? token_index[blockIdx.z] : (int)blockIdx.z;
    const int grp = nq / nkv;
    const int htiles = (grp + DEC_ROWS - 1) / DEC_ROWS;
    const int kvh = blockIdx.y / htiles, htile = blockIdx.y - kvh * htiles;
    const int h0 = kvh * grp + htile * DEC_ROWS;
    const int nvalid = min(DEC_ROWS, grp - htile * DEC_ROWS);
    int pos = positions[tok];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    if ((long long)pos >= (long long)S * chunk) {                // beyond the S chunks the launch was sized for:
        if (tid == 0 && split == 0 && err) atomicOr(err, VL_DEV_BEYOND_BOUND);   // flagged and served like an empty place
        pos = -1;
    }
    if (pos < 0) {                                               // a place of the batch that holds no request
        if (out && split == 0) {
            pdl_wait();                                          // earlier kernels may still read the rows
            for (int i = tid; i < nvalid * HD; i += NTHREADS)
                out[((size_t)tok * nq + h0 + i / HD) * HD + i % HD] = __float2bfloat16(0.f);
        }
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int c0 = max(split * chunk, lo);
    const int c1 = min((split + 1) * chunk, pos + 1);
    // (in_cluster) the blocks of a cluster serve one token: they all see the same `alone`
    const bool alone = out != nullptr && lo / chunk == pos / chunk;      // one chunk holds all the keys of the token
    if (c0 >= c1) {
        if (!in_cluster || alone) return;
        // no key of this token lies in this chunk: an empty result for the cluster's merge
        pdl_wait();                                              // the merge writes output rows
        for (int i = tid; i < nvalid * HD; i += NTHREADS) bO[i] = 0.f;
        if (tid < DEC_ROWS) { s_bm[tid] = -INFINITY; s_bl[tid] = 0.f; }
        decode_cluster_merge(bO, s_bm, s_bl, out, tok, nq, h0, nvalid, S, split, tid);
        return;
    }
    const int* table = block_table + (size_t)req_index[tok] * max_blocks;
    const int st0 = c0 / BN, st1 = (c1 - 1) / BN;

    for (int i = tid; i < (st1 - st0 + 1) * BN; i += NTHREADS)
        s_rows[i] = cache_row(table, max_blocks, st0 * BN + i, c0, pos, kvh, nkv, page_size, num_pages, err);
    // (c0 <= pos always) this chunk holds the token's own position, and this call owns the cache (a call that
    // reads another call's cache finds the token's key there: the owner ran before it)
    const bool has_new = fz.on && fz.slots && pos < c1;
    if (fz.on && fz.inv_freq)                                    // positions are part of the step's description: no wait needed
        for (int i = tid; i < fz.rot / 2; i += NTHREADS) sincosf((float)pos * fz.inv_freq[i], &s_sin[i], &s_cos[i]);
    pdl_wait();
    if (!fz.on) {
        for (int idx = tid; idx < DEC_ROWS * CPR; idx += NTHREADS) {
            const int r = idx / CPR, c = idx - r * CPR;
            const bool valid = r < nvalid;
            const bf16* src = valid ? q + (size_t)tok * q_stride + (size_t)(h0 + r) * HD + c * 8 : q;
            cp_async16(Qs + (size_t)r * LDS + c * 8, src, valid);
        }
    }
    cp_async_commit();                                           // the query rows: this thread's oldest group
    __syncthreads();                                             // s_rows, the rotation's table
    // the tile and the row in it that the token's own key and value are laid over once its copy has landed
    const int new_st = pos / BN, new_warp = (pos % BN) / 16, new_row = pos % 16;
    // Every warp runs a pipeline of its own: of each 64 keys it takes 16 (warp w the keys 16 w .. 16 w + 15),
    // copies their K and V rows itself into a ring of DEC_NST tiles that belongs to it, and waits for
    // nobody but its own copies.  No barrier of the block stands in the loop, and of a warp's ring all
    // tiles but the one being multiplied are in flight (64 requests of 4,096 keys: 197 -> 190 us; one
    // request: 11.0 -> 10.2 us).  The keys a warp sees, and so every sum, are those of the shared ring before.
    bf16* wring = ring + (size_t)warp * DEC_NST * 2 * 16 * LDS;  // [DEC_NST][K | V][16][LDS]
    auto load_tile = [&](int st, int buf) {
        bf16* kt = wring + (size_t)buf * 2 * 16 * LDS;
        const int* rows16 = s_rows + (st - st0) * BN + warp * 16;
#pragma unroll
        for (int i = 0; i < 16 * CPR / 32; ++i) {
            const int idx = lane + 32 * i;
            const int r = idx / CPR, c = idx - r * CPR;
            const int row = rows16[r];
            const size_t off = row < 0 ? 0 : (size_t)row * HD + c * 8;
            cp_async16(kt + (size_t)r * LDS + c * 8, kcache + off, row >= 0);
            cp_async16(kt + (size_t)(16 + r) * LDS + c * 8, vcache + off, row >= 0);
        }
    };
    auto lay_new_over = [&](int st, int buf) {                   // (after the tile's copies have landed)
        if (has_new && st == new_st && warp == new_warp) {
            bf16* kt = wring + (size_t)buf * 2 * 16 * LDS;
            for (int c = lane; c < 2 * CPR; c += 32) {
                const int which = c / CPR, cc = c - which * CPR;
                *reinterpret_cast<uint4*>(kt + (size_t)(which * 16 + new_row) * LDS + cc * 8) =
                    *reinterpret_cast<const uint4*>(s_new[which] + cc * 8);
            }
            __syncwarp();
        }
    };
#pragma unroll
    for (int i = 0; i < DEC_NST - 1; ++i) {
        if (st0 + i <= st1) load_tile(st0 + i, i);
        cp_async_commit();
    }
    if (fz.on) {                                                 // the head work, while the first tiles are on their way
        for (int idx = tid; idx < (DEC_ROWS - nvalid) * CPR; idx += NTHREADS)     // rows that no head uses are zero
            *reinterpret_cast<uint4*>(Qs + (size_t)(nvalid + idx / CPR) * LDS + (idx % CPR) * 8) = make_uint4(0u, 0u, 0u, 0u);
        const bf16* row = q + (size_t)tok * q_stride;
        // a warp per head; with the token's own key and value (warps 0 and 1 first) one pass more at most
        for (int r = warp - (has_new ? 2 : 0); r < nvalid; r += 4) {
            HeadRegs<bf16, RMAX> hr;
            hr.live = true;
            if (r >= 0) {
                hr.src = row + (size_t)(h0 + r) * HD; hr.out = Qs + (size_t)r * LDS;
                hr.w = fz.qw; hr.rot = fz.inv_freq ? fz.rot : 0;
            } else if (r == -2) {
                hr.src = row + (size_t)(nq + kvh) * HD; hr.out = s_new[0];
                hr.w = fz.kw; hr.rot = fz.inv_freq ? fz.rot : 0;
            } else {
                hr.src = row + (size_t)(nq + nkv + kvh) * HD; hr.out = s_new[1];
                hr.w = nullptr; hr.rot = 0;
            }
            hr.load(lane, HD);
            hr.finish(lane, HD, fz.eps, s_cos, s_sin);
        }
        if (has_new && htile == 0) {                             // (uniform) one block per token and KV head writes the cache
            __syncthreads();
            const int slot = fz.slots[tok];
            if (slot >= 0 && (long long)slot < fz.num_slots) {
                const int page = slot / page_size, off = slot - page * page_size;
                const size_t at = (((size_t)page * nkv + kvh) * page_size + off) * HD;
                for (int c = tid; c < 2 * CPR; c += NTHREADS) {
                    const int which = c / CPR, cc = c - which * CPR;
                    *reinterpret_cast<uint4*>((which ? fz.vcache : fz.kcache) + at + cc * 8) =
                        *reinterpret_cast<const uint4*>(s_new[which] + cc * 8);
                }
            } else if (slot >= 0 && tid == 0 && err) {
                atomicOr(err, VL_DEV_BAD_SLOT);
            }
        }
    }
    float* sO = reinterpret_cast<float*>(ring);                  // [4][16][HD + 4]: the warps' outputs, once the ring is free
    constexpr int OLD = HD + 4;
    if constexpr (TR) {
        // ---- keys as rows: lane (g, t) holds keys g and g + 8 of the tile and heads 2t, 2t + 1 ----
        constexpr int MT = HD / 16;                              // tiles of 16 features of the output
        float oT[MT][4], m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
        for (int d = 0; d < MT; ++d) { oT[d][0] = oT[d][1] = oT[d][2] = oT[d][3] = 0.f; }
        unsigned qb[KSTEPS][2];                                  // Q^T as the 16 x 8 operand: features 2t.., 2t + 8.. of head g
        cp_async_wait<DEC_NST - 1>();                            // this thread's share of the query rows has landed ...
        __syncthreads();                                         // ... and so has everybody's
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            qb[ks][0] = *reinterpret_cast<const unsigned*>(Qs + (size_t)g * LDS + ks * 16 + 2 * t);
            qb[ks][1] = *reinterpret_cast<const unsigned*>(Qs + (size_t)g * LDS + ks * 16 + 2 * t + 8);
        }
        for (int st = st0; st <= st1; ++st) {
            const int it = st - st0;
            cp_async_wait<DEC_NST - 2>();
            __syncwarp();                                        // the tile has landed for every lane; the tile before is read
            lay_new_over(st, it % DEC_NST);
            if (st + DEC_NST - 1 <= st1) load_tile(st + DEC_NST - 1, (it + DEC_NST - 1) % DEC_NST);
            cp_async_commit();
            const bf16* Kt = wring + (size_t)(it % DEC_NST) * 2 * 16 * LDS;
            const bf16* Vt = Kt + 16 * LDS;
            float sT[4] = {0.f, 0.f, 0.f, 0.f};                  // (key g | g + 8) x (head 2t | 2t + 1)
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                unsigned ka[4];
                ldmatrix_x4(ka, Kt + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks * 16 + 8 * (lane >> 4));
                mma16816(sT, ka, qb[ks][0], qb[ks][1]);
            }
            const int j0 = st * BN + warp * 16 + g;              // this lane's keys: j0 and j0 + 8
            const bool in0 = j0 >= c0 && j0 < c1, in1 = j0 + 8 >= c0 && j0 + 8 < c1;
            sT[0] = in0 ? sT[0] * scale_log2 : -INFINITY; sT[1] = in0 ? sT[1] * scale_log2 : -INFINITY;
            sT[2] = in1 ? sT[2] * scale_log2 : -INFINITY; sT[3] = in1 ? sT[3] * scale_log2 : -INFINITY;
            float mx[2] = {fmaxf(sT[0], sT[2]), fmaxf(sT[1], sT[3])}, corr[2], base[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {                        // over the 16 keys: the lanes of equal t
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 4));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 8));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 16));
                const float mn = fmaxf(m_run[r], mx[r]);
                base[r] = (mn == -INFINITY) ? 0.f : mn;
                corr[r] = exp2_mufu(m_run[r] - base[r]);
                m_run[r] = mn;
                l_run[r] *= corr[r];
            }
            const float p0 = exp2_mufu(sT[0] - base[0]), p1 = exp2_mufu(sT[1] - base[1]);
            const float p2 = exp2_mufu(sT[2] - base[0]), p3 = exp2_mufu(sT[3] - base[1]);
            l_run[0] += p0 + p2;
            l_run[1] += p1 + p3;
            // P^T as the 16 x 8 operand of the second product: keys 2t.., 2t + 8.. of head g = the transposes of
            // the two 8 x 8 blocks (keys g | g + 8, heads 2t..) that this lane's probabilities are rows of
            unsigned pb0, pb1;
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(pack_bf16(p0, p1)));
            asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(pack_bf16(p2, p3)));
#pragma unroll
            for (int d = 0; d < MT; ++d) {
                unsigned va[4];                                  // V^T: features 16 d + (g | g + 8) x keys (2t.. | 2t + 8..)
                ldmatrix_x4_trans(va, Vt + (size_t)((lane & 7) + 8 * (lane >> 4)) * LDS + d * 16 + 8 * ((lane >> 3) & 1));
                oT[d][0] *= corr[0]; oT[d][1] *= corr[1]; oT[d][2] *= corr[0]; oT[d][3] *= corr[1];
                mma16816(oT[d], va, pb0, pb1);
            }
        }
        cp_async_wait<0>();
        __syncthreads();                                         // the ring is free: it now carries the warps' outputs
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 4);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 8);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 16);
        }
#pragma unroll
        for (int d = 0; d < MT; ++d) {
            float* pa = sO + ((size_t)warp * DEC_ROWS + 2 * t) * OLD + d * 16 + g;
            pa[0] = oT[d][0]; pa[OLD] = oT[d][1];
            pa[8] = oT[d][2]; pa[OLD + 8] = oT[d][3];
        }
        if (g == 0) {
            s_m[warp][2 * t] = m_run[0]; s_l[warp][2 * t] = l_run[0];
            s_m[warp][2 * t + 1] = m_run[1]; s_l[warp][2 * t + 1] = l_run[1];
        }
    } else {
        float o[DTILES][4], m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
        for (int d = 0; d < DTILES; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
        unsigned qf[KSTEPS][4];
        cp_async_wait<DEC_NST - 1>();                                // this thread's share of the query rows has landed ...
        __syncthreads();                                             // ... and so has everybody's
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
            ldmatrix_x4(qf[ks], Qs + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks * 16 + 8 * (lane >> 4));

        for (int st = st0; st <= st1; ++st) {
            const int it = st - st0;
            cp_async_wait<DEC_NST - 2>();
            __syncwarp();                                            // the tile has landed for every lane; the tile before is read
            lay_new_over(st, it % DEC_NST);
            if (st + DEC_NST - 1 <= st1) load_tile(st + DEC_NST - 1, (it + DEC_NST - 1) % DEC_NST);
            cp_async_commit();
            const bf16* Kt = wring + (size_t)(it % DEC_NST) * 2 * 16 * LDS;
            const bf16* Vt = Kt + 16 * LDS;
            const int kr0 = warp * 16;                               // this warp's 16 keys of every 64
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                unsigned kb[4];
                ldmatrix_x4(kb, Kt + (size_t)((lane & 7) + 8 * (lane >> 4)) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
                mma16816(s[0], qf[ks], kb[0], kb[1]);
                mma16816(s[1], qf[ks], kb[2], kb[3]);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = st * BN + kr0 + n * 8 + 2 * t + (e & 1);
                    const float v = (j >= c0 && j < c1) ? s[n][e] * scale_log2 : -INFINITY;
                    s[n][e] = v;
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
                const float p00 = exp2_mufu(s[0][0] - base[0]), p01 = exp2_mufu(s[0][1] - base[0]);
                const float p02 = exp2_mufu(s[0][2] - base[1]), p03 = exp2_mufu(s[0][3] - base[1]);
                const float p10 = exp2_mufu(s[1][0] - base[0]), p11 = exp2_mufu(s[1][1] - base[0]);
                const float p12 = exp2_mufu(s[1][2] - base[1]), p13 = exp2_mufu(s[1][3] - base[1]);
                l_run[0] += p00 + p01 + p10 + p11;
                l_run[1] += p02 + p03 + p12 + p13;
                pf[0] = pack_bf16(p00, p01); pf[1] = pack_bf16(p02, p03);
                pf[2] = pack_bf16(p10, p11); pf[3] = pack_bf16(p12, p13);
            }
#pragma unroll
            for (int dp = 0; dp < DTILES / 2; ++dp) {
                unsigned vb[4];
                ldmatrix_x4_trans(vb, Vt + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                o[2 * dp][0] *= corr[0]; o[2 * dp][1] *= corr[0]; o[2 * dp][2] *= corr[1]; o[2 * dp][3] *= corr[1];
                o[2 * dp + 1][0] *= corr[0]; o[2 * dp + 1][1] *= corr[0]; o[2 * dp + 1][2] *= corr[1]; o[2 * dp + 1][3] *= corr[1];
                mma16816(o[2 * dp], pf, vb[0], vb[1]);
                mma16816(o[2 * dp + 1], pf, vb[2], vb[3]);
            }
        }
        cp_async_wait<0>();
        __syncthreads();                                             // the ring is free: it now carries the warps' outputs
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        }
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            float* pa = sO + ((size_t)warp * DEC_ROWS + g) * OLD + d * 8 + 2 * t;
            pa[0] = o[d][0]; pa[1] = o[d][1];
            pa[8 * OLD] = o[d][2]; pa[8 * OLD + 1] = o[d][3];
        }
        if (t == 0) {
            s_m[warp][g] = m_run[0]; s_l[warp][g] = l_run[0];
            s_m[warp][g + 8] = m_run[1]; s_l[warp][g + 8] = l_run[1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < nvalid * HD; idx += NTHREADS) {
        const int r = idx / HD, e = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, s_m[w][r]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = (s_m[w][r] == -INFINITY) ? 0.f : exp2_mufu(s_m[w][r] - M);
            acc += sO[((size_t)w * DEC_ROWS + r) * OLD + e] * wgt;
            L += s_l[w][r] * wgt;
        }
        if (alone) {                                             // nothing to merge with: the output row itself
            out[((size_t)tok * nq + h0 + r) * HD + e] = __float2bfloat16(acc * (L > 0.f ? 1.0f / L : 0.f));
            continue;
        }
        if (in_cluster) {
            bO[idx] = acc;
            if (e == 0) { s_bm[r] = M; s_bl[r] = L; }
            continue;
        }
        const size_t row = ((size_t)blockIdx.z * nq + (h0 + r)) * S + split;
        part_acc[row * HD + e] = acc;
        if (e == 0) {
            part_ml[row * 2] = M * 0.6931471805599453f;          // the merge kernel works in natural-log units
            part_ml[row * 2 + 1] = L;
        }
    }
    if (alone) return;
    if (in_cluster) {
        decode_cluster_merge(bO, s_bm, s_bl, out, tok, nq, h0, nvalid, S, split, tid);
        return;
    }
    if (!arrivals) return;                                       // the caller merges with a kernel of its own
    // The block that arrives last among those of this token and these heads merges their partial
    // results (in the order of the chunks, whoever it is: the result does not depend on the order of
    // arrival) and writes the output rows.
    __shared__ int s_last;
    const int sp0 = lo / chunk, sp1 = pos / chunk;               // the chunks that hold keys of this token
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = arrivals + (size_t)blockIdx.z * gridDim.y + blockIdx.y;
        const int last = atomicAdd(counter, 1) == sp1 - sp0;
        if (last) *counter = 0;                                  // zero again for the next launch
        s_last = last;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Weights of the chunks first (8 threads per row share the chunks out, maximum and sum by a fixed
    // butterfly), into the shared memory that held the keys; then every thread adds up its elements
    // over the chunks with the loads of several chunks in flight.
    float* s_w = reinterpret_cast<float*>(ring);                 // [DEC_ROWS][nsp]
    float* s_inv = s_l[0];                                       // [DEC_ROWS]: 1 / sum of a row
    const int nsp = sp1 - sp0 + 1;
    {
        const int r = tid >> 3, part = tid & 7;                  // 128 threads = 16 rows x 8
        const size_t row0 = ((size_t)blockIdx.z * nq + (h0 + min(r, nvalid - 1))) * S + sp0;
        float M = -INFINITY;
        for (int i = part; i < nsp; i += 8) M = fmaxf(M, __ldcg(part_ml + (row0 + i) * 2));
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 1));
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 2));
        M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 4));
        float L = 0.f;
        for (int i = part; i < nsp; i += 8) {
            const float ms = __ldcg(part_ml + (row0 + i) * 2);
            const float wgt = (ms == -INFINITY) ? 0.f : __expf(ms - M);
            L += __ldcg(part_ml + (row0 + i) * 2 + 1) * wgt;
            s_w[r * nsp + i] = wgt;
        }
        L += __shfl_xor_sync(0xffffffffu, L, 1);
        L += __shfl_xor_sync(0xffffffffu, L, 2);
        L += __shfl_xor_sync(0xffffffffu, L, 4);
        if (part == 0) s_inv[r] = L > 0.f ? 1.0f / L : 0.f;
    }
    __syncthreads();
    for (int idx = tid; idx < nvalid * HD; idx += NTHREADS) {
        const int r = idx / HD, e = idx - r * HD;
        const float* pa = part_acc + (((size_t)blockIdx.z * nq + (h0 + r)) * S + sp0) * HD + e;
        const float* w = s_w + r * nsp;
        float acc = 0.f;
#pragma unroll 8
        for (int i = 0; i < nsp; ++i) acc += __ldcg(pa + (size_t)i * HD) * w[i];
        out[((size_t)tok * nq + h0 + r) * HD + e] = __float2bfloat16(acc * s_inv[r]);
    }
}

// The largest cluster the decode kernel may be launched as on this device: 16 where clusters beyond the
// portable size are allowed and one fits, else 8.
static int decode_max_cluster() {
    static int v = 0;
    if (!v) {
        v = 8;
        if (cudaFuncSetAttribute(flash_decode_kernel<false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
            cudaFuncSetAttribute(flash_decode_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            const size_t ring = (size_t)DEC_NST * 2 * BN * LDS * sizeof(bf16);
            const size_t merge = (size_t)(4 * DEC_ROWS * (HD + 4) + DEC_ROWS * HD) * sizeof(float);
            const size_t smem = (size_t)DEC_ROWS * LDS * sizeof(bf16) + (ring > merge ? ring : merge);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(16, 1, 1);
            cfg.blockDim = dim3(NTHREADS);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 16; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaFuncSetAttribute(flash_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
                cudaFuncSetAttribute(flash_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
                cudaOccupancyMaxActiveClusters(&clusters, flash_decode_kernel<false>, &cfg) == cudaSuccess && clusters >= 8 &&
                cudaOccupancyMaxActiveClusters(&clusters, flash_decode_kernel<true>, &cfg) == cudaSuccess && clusters >= 8)
                v = 16;
        }
        cudaGetLastError();                                      // a refusal above is an answer, not an error of the step
    }
    return v;
}
extern "C" int vl_flash_decode_max_cluster() { return decode_max_cluster(); }

// Most chunks per token that vl_flash_decode merges itself when they are too many for a cluster:
// their weights, for 16 rows, have to fit the shared memory that held the keys.
extern "C" int vl_flash_decode_own_merge_cap() {
    const size_t ring = (size_t)DEC_NST * 2 * BN * LDS * sizeof(bf16);
    const size_t merge = (size_t)(4 * DEC_ROWS * (HD + 4) + DEC_ROWS * HD) * sizeof(float);
    return (int)((ring > merge ? ring : merge) / (DEC_ROWS * sizeof(float)));
}

// Scratch as for vl_decode_attention: part_acc [T, nq, S, hd], part_ml [T, nq, S, 2] float32,
// S = ceil(max_context / chunk).  T counts the tokens served: all tokens of the step, or those that
// token_index (T entries) names.  With out (bfloat16 [tokens of the step, nq * hd]) and arrivals (int32,
// T * nkv * ceil(group / 16) counters, zero before the first launch and left zero by every launch) the
// kernel merges the chunks itself: up to 8 chunks as the blocks of a cluster, through their shared
// memory; more through the scratch, by the block that arrives last.  With both null, follow with
// vl_decode_attention_merge.
static int launch_flash_decode(const void* q, int q_stride, const void* kcache, const void* vcache,
                               const int* block_table, int max_blocks, const int* req_index, const int* positions,
                               int T, int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                               int chunk, int S, float* part_acc, float* part_ml, unsigned* err,
                               const int* token_index, void* out, int* arrivals, DecodeFusion fz, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd != HD) return VL_ERR_UNSUPPORTED;
    if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0 || q_stride % 8) return VL_ERR_ARGUMENT;
    if (chunk <= 0 || chunk % BN || chunk > DEC_MAX_CHUNK || S <= 0 || S > 65535 || T > 65535) return VL_ERR_ARGUMENT;
    if ((out == nullptr) != (arrivals == nullptr)) return VL_ERR_ARGUMENT;
    if (arrivals && S > vl_flash_decode_own_merge_cap()) return VL_ERR_UNSUPPORTED;
    const int grp = nq / nkv;
    const int htiles = (grp + DEC_ROWS - 1) / DEC_ROWS;
    const size_t ring = (size_t)DEC_NST * 2 * BN * LDS * sizeof(bf16);
    const size_t merge = (size_t)(4 * DEC_ROWS * (HD + 4) + DEC_ROWS * HD) * sizeof(float);
    const size_t smem = (size_t)DEC_ROWS * LDS * sizeof(bf16) + (ring > merge ? ring : merge);
    cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // A cluster starts when all its blocks find room at once: good while the whole grid is resident at
    // the same time (measured at 8 requests of 4,096 keys: 33.4 -> 29.5 us), a loss when blocks queue for
    // several rounds (64 requests: 200 -> 209 us); there the last block to arrive merges.
    static int resident = 0;
    if (!resident) {
        int dev = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, flash_decode_kernel<true>, NTHREADS, smem) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        resident = sms * per_sm;
    }
    const int in_cluster = out != nullptr && S >= 2 && S <= decode_max_cluster() && (long long)S * nkv * htiles * T <= resident;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, nkv * htiles, T);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (in_cluster) {                                            // the chunks of a token: one cluster
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = S; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (vl_pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    // groups of up to 8 query heads: keys as the rows of the tensor-core tiles, heads as their 8 columns
    return (int)cudaLaunchKernelEx(&cfg, grp <= 8 ? flash_decode_kernel<true> : flash_decode_kernel<false>, (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache,
                                   block_table, max_blocks, req_index, positions, nq, nkv, page_size, num_pages,
                                   scale * 1.4426950408889634f, window, chunk, S, part_acc, part_ml, err, token_index,
                                   (bf16*)out, arrivals, in_cluster, fz);
}

extern "C" int vl_flash_decode(const void* q, int q_stride, const void* kcache, const void* vcache,
                               const int* block_table, int max_blocks, const int* req_index, const int* positions,
                               int T, int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                               int chunk, int S, float* part_acc, float* part_ml, unsigned* err,
                               const int* token_index, void* out, int* arrivals, void* stream) {
    DecodeFusion fz = {};
    return launch_flash_decode(q, q_stride, kcache, vcache, block_table, max_blocks, req_index, positions, T, nq, nkv, hd,
                               page_size, num_pages, scale, window, chunk, S, part_acc, part_ml, err, token_index, out,
                               arrivals, fz, stream);
}

// The same with the step's head norm, rotation and cache write folded in (DecodeFusion): q [T, q_stride] holds
// the rows q | k | v as the projection left them, qw / kw are the norm weights of a q and a k head (both null:
// no norm), inv_freq [rot / 2] the rotary frequencies (null: no rotation), slots [tokens of the step] each
// token's place in the cache, page * page_size + offset (null: this call writes no cache: it reads another
// call's).  Every token of the launch must be the LAST position of its request (pos = the position the slot
// stands for), which is what a decode step is.
extern "C" int vl_flash_decode_fused(const void* q, int q_stride, void* kcache, void* vcache,
                                     const int* block_table, int max_blocks, const int* req_index, const int* positions,
                                     int T, int nq, int nkv, int hd, int page_size, int num_pages, float scale, int window,
                                     int chunk, int S, float* part_acc, float* part_ml, unsigned* err,
                                     const int* token_index, void* out, int* arrivals,
                                     const float* qw, const float* kw, float eps, const float* inv_freq, int rot,
                                     const int* slots, void* stream) {
    if ((qw == nullptr) != (kw == nullptr) || rot < 0 || rot > hd || (rot & 1)) return VL_ERR_ARGUMENT;
    if (q_stride < (nq + 2 * nkv) * hd) return VL_ERR_ARGUMENT;
    DecodeFusion fz = {qw, kw, eps, inv_freq, inv_freq ? rot : 0, slots, (long long)num_pages * page_size,
                       (bf16*)kcache, (bf16*)vcache, 1};
    return launch_flash_decode(q, q_stride, kcache, vcache, block_table, max_blocks, req_index, positions, T, nq, nkv, hd,
                               page_size, num_pages, scale, window, chunk, S, part_acc, part_ml, err, token_index, out,
                               arrivals, fz, stream);
}
