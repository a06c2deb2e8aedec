// Declaration of the decode-attention entry point that needs no memory from its caller beyond
// inputs and outputs.  It has no counterpart in pplmx/vllm-lite; it exists for hosts of this
// library that cannot allocate device memory at the time they need attention.
//
// Who that is: a process whose device memory was handed out in full at start-up (a serving stack
// that reserves the whole GPU for its own pool leaves cudaMalloc nothing to give), code that runs
// where an allocation is forbidden or would stall (a latency-critical loop, or a region in which
// the surrounding framework has frozen its allocator), and embedders that link the library from C
// and have no tensor library at hand to size and own a scratch buffer.  vl_decode_attention wants
// two float32 scratch buffers from such a caller; this entry point brings its own.
//
// The scratch is one array of fixed size inside the library's device image.  Consequences:
//   * Every GPU that loads the library holds VL_NO_ALLOC_SCRATCH_BYTES of device memory for it
//     until the process exits, whether or not the entry point is ever called.
//   * Problems whose partial results do not fit are refused with VL_ERR_SCRATCH (-4); nothing is
//     launched.  The need is  T * nq * S * (hd + 2)  floats with  S = ceil(max_context / chunk),
//     and the limit is VL_NO_ALLOC_SCRATCH_FLOATS.
//   * All calls share the array.  Two calls that overlap on the GPU (different streams, or two
//     host threads) overwrite each other's partial results: keep calls on one stream, or order
//     them yourself.  Nothing in the array has to start at zero; a call writes every element it
//     later reads.
//   * The first call on each device looks up the array's device address (with that device current)
//     and remembers it.  Make that first call outside any stream capture.
//   * S says how many chunks of `chunk` key positions the scratch is laid out for.  A token whose
//     position is chunk * S or more does not fit that layout: it is not half-served, its row of
//     `out` becomes zero and bit 0x10 is set in the error word (positions live on the device, so
//     the host cannot refuse them beforehand).  A position of -1 marks an empty place of the batch:
//     nothing is read for it and its row becomes zero too.
// The entry point calls no cudaMalloc, cudaFree, or any routine of an allocating library.
#pragma once

#define VL_ERR_SCRATCH (-4)
#define VL_NO_ALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)                 /* 16 MiB */
#define VL_NO_ALLOC_SCRATCH_BYTES (VL_NO_ALLOC_SCRATCH_FLOATS * 4u)
#define VL_NO_ALLOC_MAX_DEVICES 64

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as vl_decode_attention without part_acc / part_ml.
// Returns 0, VL_ERR_SCRATCH when the problem exceeds the built-in scratch, another negative code
// for arguments the kernel does not take, or a positive cudaError_t.
int vl_decode_attention_no_alloc(const void* q, int q_stride, void* out, int dtype,
                                 const void* kcache, const void* vcache,
                                 const int* block_table, int max_blocks,
                                 const int* req_index, const int* positions,
                                 int T, int nq, int nkv, int hd, int page_size, int num_pages,
                                 float scale, int window, int chunk, int S,
                                 unsigned* err, void* stream);

#ifdef __cplusplus
}
#endif
