// Shared helpers of the engine's CUDA kernels (sm_100a).
//
// Every exported entry point is `extern "C" int vl_<name>(..., void* stream)`.
// It returns 0, a positive cudaError_t of the launch, or one of the negative
// codes below when it refuses its arguments; the Python side turns any
// non-zero value into an exception.  Kernels never trap: a bad token id or
// cache slot sets a bit in the caller's error word and the access is skipped.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define VL_OK 0
#define VL_ERR_UNSUPPORTED (-2)   // a size the kernel does not take
#define VL_ERR_ARGUMENT (-3)      // inconsistent arguments

// bits of the device-side error word
#define VL_DEV_BAD_TOKEN 1u
#define VL_DEV_BAD_SLOT 2u
#define VL_DEV_BAD_PAGE 4u
#define VL_DEV_WAIT_EXPIRED 8u
#define VL_DEV_BEYOND_BOUND 0x10u   // a position at or past chunk * S, the context the launch was sized for
// with VL_DEV_WAIT_EXPIRED: the kernel whose wait ran out ...
#define VL_DEV_IN_DECODE_ATTENTION 0x100u
#define VL_DEV_IN_GEMM_SMALL_M 0x200u
#define VL_DEV_IN_GEMM_TC5 0x400u
#define VL_DEV_IN_GEMM_TC5_PAIR 0x800u
#define VL_DEV_IN_FLASH_TC5 0x1000u
#define VL_DEV_IN_FLASH_DECODE_TMA 0x2000u
// ... and, in the two tcgen05 products, which waits gave up in the block (shifted left by 16):
// 1 a free stage (copying thread), 2 a free accumulator, 4 a filled stage (both: issuing thread),
// 8 a complete accumulator (epilogue)
#define VL_DEV_ROLE_SHIFT 16

// dtype codes shared with csrc/ops.py
#define VL_F32 0
#define VL_BF16 1

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NT threads (NT a multiple of 32, at most 1024).  The
// order of additions depends on NT alone, so a row's result does not depend on
// what else is in the launch.  `scratch` holds 32 floats.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) t += scratch[w];
    return t;
}

static inline int vl_launch_status() { return (int)cudaGetLastError(); }

// ---- bounded waits ----------------------------------------------------------------------------------
// A wait on an mbarrier ends after this many polls or this many SM cycles (about two seconds),
// whichever comes first: one poll may itself be suspended by the hardware for a time that no
// document bounds, so a count of polls alone does not bound the time.  The block that gave up records
// VL_DEV_WAIT_EXPIRED, waits (again bounded) for its own copies in flight and leaves.
#define VL_WAIT_POLL_LIMIT (1 << 22)
#define VL_WAIT_CYCLE_LIMIT 4000000000ll
__device__ __forceinline__ bool vl_wait_gave_up(int poll, long long t0) {
    return (poll & 31) == 31 && clock64() - t0 > VL_WAIT_CYCLE_LIMIT;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// Kernels of a step are launched with the attribute that lets the next kernel of the stream start
// while this one is still running.  A kernel calls pdl_launch_dependents() at once (the next grid
// may be brought onto the SMs as soon as every block of this one has started) and pdl_wait() before
// it first touches memory that earlier kernels of the stream write, and before its own first write
// to global memory: pdl_wait() returns when all earlier kernels have completed and their writes are
// visible.  What lies before pdl_wait() may only read constants of the step (weights) and set up
// shared memory.  Launched without the attribute, both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
// Dependent launches are off until vl_set_pdl(1) turns them on for the launches that follow (the engine
// does so for steps of few tokens, whose launch gaps they hide, and turns them off again for steps of
// many tokens); the environment's VLLM_LITE_B200_PDL=0 keeps them off for good.  The product that runs as
// clusters of two blocks (gemm_tc5_pair.cu) is launched without the attribute whatever the switch says:
// started as a dependent while earlier kernels still ran it stood still on the device now and then (about
// once in a few hundred of its launches at 1,588 or 4,096 rows; not once in thousands without the
// attribute).  The kernels that allocate tensor memory do so behind their pdl_wait().
static int g_vl_pdl = 0;
static inline bool vl_pdl_forbidden() {
    const char* v = getenv("VLLM_LITE_B200_PDL");
    return v && v[0] == '0';
}
static inline bool vl_pdl_enabled() { return g_vl_pdl == 1; }
extern "C" void vl_set_pdl(int on) { g_vl_pdl = (on && !vl_pdl_forbidden()) ? 1 : 0; }
extern "C" int vl_get_pdl() { return g_vl_pdl; }

template <typename... KArgs, typename... Args>
static inline int vl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vl_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
