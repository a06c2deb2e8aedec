// tcgen05 / TMA / mbarrier building blocks shared by the kernels that run on the 5th-generation
// tensor cores (accumulators in TMEM, operands in shared memory behind matrix descriptors).
// Every wait on an mbarrier is bounded: the caller records VL_DEV_WAIT_EXPIRED and winds down.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace tc5 {
constexpr int SWIZZLE_COLS = 64;             // one 128-byte swizzle row of bfloat16

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 0; i < VL_WAIT_POLL_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (vl_wait_gave_up(i, t0)) return false;
    }
    return false;
}
// x = element index along K (a multiple of 8: the copy starts on a 16-byte boundary), y = row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// the same with a third coordinate (z: the block of 64 columns of a row that the box takes first)
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
// five coordinates: (x, row in page, page, block of 64 columns, KV head) of tc5_make_map_pages
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc5_alloc(unsigned* smem_result, unsigned ncols) {          // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc5_dealloc(unsigned taddr, unsigned ncols) {              // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc5_mma(unsigned tmem_c, unsigned long long adesc, unsigned long long bdesc,
                                        unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_c), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the mbarrier once every tcgen05 operation this thread issued before has completed
__device__ __forceinline__ void tc5_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc5_ld32(unsigned taddr, unsigned (&r)[32]) {              // 32 lanes x 32 columns
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// the same load without the wait: issue several, then tc5_wait_ld()
__device__ __forceinline__ void tc5_ld32_nowait(unsigned taddr, unsigned* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc5_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 columns from registers into TMEM; tc5_wait_st() before anyone else may read them
__device__ __forceinline__ void tc5_st32(unsigned taddr, const unsigned* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc5_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// makes this thread's ordinary writes to shared memory visible to the units that read it on their
// own (TMA, the tensor cores); follow with a barrier that the consumer waits on
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16) with the
// 128-byte swizzle: 8 rows make one 1024-byte swizzle atom, atoms follow each other along M/N.
//   bits  0-13  start address >> 4          bits 16-29  leading byte offset >> 4 (unused here)
//   bits 32-45  stride byte offset >> 4 = 1024 >> 4 (from one 8-row atom to the next)
//   bits 46-47  descriptor version 1        bits 61-63  swizzle mode, 2 = 128 bytes
__device__ __forceinline__ unsigned long long make_smem_desc(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3ffff) >> 4);
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// The same with both offsets given: for an operand stored with its M/N index contiguous (rows of 64
// M/N elements = 128 bytes, one row per K index, 128-byte swizzle) the 8 K rows x 128 bytes make the
// atom, `stride` leads from one group of 8 K rows to the next and `leading` from one block of 64
// M/N elements to the next.
__device__ __forceinline__ unsigned long long make_smem_desc_lbo_sbo(const void* tile, unsigned leading, unsigned stride) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) & 0x3ffff) >> 4);
    d |= (unsigned long long)((leading >> 4) & 0x3fff) << 16;
    d |= (unsigned long long)((stride >> 4) & 0x3fff) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
constexpr unsigned IDESC_B_MN_MAJOR = 1u << 16;      // B is stored with N contiguous (bit 15: the same for A)
// Instruction descriptor of kind::f16: float32 accumulator (bits 4-5 = 1), bfloat16 A and B
// (bits 7-9 and 10-12 = 1), both K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in 24-28.
__host__ __device__ constexpr unsigned make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
// Stores 32 neighbouring columns (from column `col` of the product) of one row of the accumulator.
// swiglu: the 32 columns are two blocks of 8 gate and 8 up columns and become 16 columns of C at col / 2:
// C[8b + i] = silu(y[16b + i]) * y[16b + 8 + i].  `crow` points at the row of C.
template <typename TO>
__device__ __forceinline__ void store_chunk32(const unsigned (&v)[32], TO* crow, int col, int N, int swiglu) {
    if (swiglu) {
        TO* dst = crow + col / 2;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            if (col + 16 * blk + 16 <= N) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float gt = __uint_as_float(v[16 * blk + i]), up = __uint_as_float(v[16 * blk + 8 + i]);
                    o[i] = gt / (1.0f + __expf(-gt)) * up;
                }
                if constexpr (sizeof(TO) == 2) {
                    uint4 q;
                    unsigned* w = reinterpret_cast<unsigned*>(&q);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __nv_bfloat162 p = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
                        w[i] = *reinterpret_cast<unsigned*>(&p);
                    }
                    if ((((uintptr_t)(dst + 8 * blk)) & 15) == 0) {
                        *reinterpret_cast<uint4*>(dst + 8 * blk) = q;
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) dst[8 * blk + i] = from_f32<TO>(o[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) dst[8 * blk + i] = from_f32<TO>(o[i]);
                }
            }
        }
        return;
    }
    TO* dst = crow + col;
    if (col + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
        if constexpr (sizeof(TO) == 2) {
            uint4 q[4];
            unsigned* w = reinterpret_cast<unsigned*>(q);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                w[i] = *reinterpret_cast<unsigned*>(&p);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst)[i] = q[i];
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
    } else {
        for (int i = 0; i < 32; ++i)
            if (col + i < N) dst[i] = from_f32<TO>(__uint_as_float(v[i]));
    }
}
}  // namespace tc5

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld elements; boxes of box_rows x 64 elements, 128-byte swizzle.
static inline int tc5_make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return VL_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)tc5::SWIZZLE_COLS, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VL_ERR_ARGUMENT;
}

// A [rows, cols] bfloat16 matrix (cols a multiple of 64, row stride ld elements) seen as
// (64 columns, rows, blocks of 64 columns): one box brings box_rows rows of all the blocks and lays
// them down block after block, each block as box_rows rows of 128 bytes with the 128-byte swizzle.
static inline int tc5_make_map_blocks(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return VL_ERR_UNSUPPORTED;
    if (cols % tc5::SWIZZLE_COLS) return VL_ERR_UNSUPPORTED;
    cuuint64_t dims[3] = {(cuuint64_t)tc5::SWIZZLE_COLS, (cuuint64_t)rows, (cuuint64_t)(cols / tc5::SWIZZLE_COLS)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)tc5::SWIZZLE_COLS * 2};
    cuuint32_t box[3] = {(cuuint32_t)tc5::SWIZZLE_COLS, (cuuint32_t)box_rows, (cuuint32_t)(cols / tc5::SWIZZLE_COLS)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VL_ERR_ARGUMENT;
}


// A paged cache [pages, kv heads, page_size, cols] of bfloat16 (cols a multiple of 64) seen as
// (64 columns, rows of a page, pages, blocks of 64 columns, kv heads): one box brings, for one kv head, the
// rows of `box_pages` NEIGHBOURING pages and lays them down block of columns after block of columns, each
// block as box_pages * page_size rows of 128 bytes (page after page, i.e. in the order of the keys when a
// request holds neighbouring pages) with the 128-byte swizzle.  A request's pages are neighbours whenever
// the pool handed them out in a row, so a tile of 64 keys on pages of 16 is then ONE request of 16 KB to
// the TMA unit instead of four (or eight) small ones.
static inline int tc5_make_map_pages(CUtensorMap* map, const void* base, int num_pages, int nkv, int page_size, int cols,
                                     int box_pages) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return VL_ERR_UNSUPPORTED;
    if (cols % tc5::SWIZZLE_COLS || box_pages <= 0 || box_pages * page_size > 256) return VL_ERR_UNSUPPORTED;
    const cuuint64_t row_bytes = (cuuint64_t)cols * 2;
    cuuint64_t dims[5] = {(cuuint64_t)tc5::SWIZZLE_COLS, (cuuint64_t)page_size, (cuuint64_t)num_pages,
                          (cuuint64_t)(cols / tc5::SWIZZLE_COLS), (cuuint64_t)nkv};
    cuuint64_t strides[4] = {row_bytes, (cuuint64_t)nkv * page_size * row_bytes, (cuuint64_t)tc5::SWIZZLE_COLS * 2,
                             (cuuint64_t)page_size * row_bytes};
    cuuint32_t box[5] = {(cuuint32_t)tc5::SWIZZLE_COLS, (cuuint32_t)page_size, (cuuint32_t)box_pages,
                         (cuuint32_t)(cols / tc5::SWIZZLE_COLS), 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VL_ERR_ARGUMENT;
}
