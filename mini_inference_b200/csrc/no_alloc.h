// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in davidjoyme/mini-inference; it exists for embedders of
// this library.  Some hosts of a kernel library may not call cudaMalloc at all: code that runs
// inside another framework's memory plan (every byte of the device is already handed out and a
// stray allocation would fail or fragment the plan), real-time or safety-reviewed loops in which
// allocation is forbidden after start-up, and plug-ins that are only given pointers.  The split-KV
// decode attention needs scratch for the per-split partial outputs; the ordinary entry points
// (mi_attn_decode_mma + mi_attn_decode_merge) take that scratch from the caller, which in this
// package means the framework's allocator.  mi_attn_decode_noalloc needs none: its scratch is a
// fixed array inside the library image.
//
// Cost and limits
//   * The array is MI_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on EVERY GPU that loads the
//     library, from load until the process exits, whether or not this entry point is ever called.
//   * A call needs num_decode * H * splits * (D + 1) floats of it; a larger problem is refused
//     with MI_NOALLOC_TOO_LARGE (nothing is launched).  Use fewer splits, or the ordinary entry
//     points with your own scratch.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current).  Make that first call outside any stream capture; later calls only
//     launch kernels.
//   * All calls share the one array and it keeps what the last call left in it.  Nothing in it has
//     to start at zero: every element a call reads was written by that same call's first kernel.
//     Two calls whose kernels overlap on the GPU (different streams, or graphs replayed
//     concurrently) race on it; serialise them on one stream.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define MI_NOALLOC_SCRATCH_BYTES (8u << 20)
#define MI_NOALLOC_OK 0
#define MI_NOALLOC_BAD_SHAPE (-2)      /* head size, group or page size the tensor-core kernel does not take */
#define MI_NOALLOC_TOO_LARGE (-3)      /* scratch need exceeds MI_NOALLOC_SCRATCH_BYTES */
#define MI_NOALLOC_SETUP_FAILED (-4)   /* the array's device address could not be obtained */

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as mi_attn_decode_mma followed by mi_attn_decode_merge (bfloat16 q,
// caches and out; see attention_decode_mma.cu), minus the two scratch pointers.  Returns
// MI_NOALLOC_OK, one of the codes above, or a positive cudaError_t from a launch.
int mi_attn_decode_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                           const int* decode_segs, int num_decode, const int* seg_q_start, const int* seg_kv_len,
                           const int* block_table, int table_stride, int H, int KV, int D, int page_size,
                           int splits, float scale, int window, cudaStream_t stream);

// A sentence for a return code of mi_attn_decode_noalloc (static storage, never null).
const char* mi_attn_decode_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
