// sandy_decode_attention_static: split-KV decode attention for callers that cannot allocate.
//
// This entry point has NO counterpart in the reference (sunho/SandyRT); it is an addition
// of this engine.  (The reference's decode attention allocates its split scratch with
// cudaMallocAsync on every call, src/device/cuda/CudaAttentionKernels.cu:496-503.)
//
// Who it is for.  sandy_decode_attention() wants a float scratch buffer from its caller
// whenever the keys of a (token, head) pair are split over several blocks.  Some callers
// have no way to provide one: code that runs where device allocation is forbidden or
// impossible, for example inside a region that must not touch the allocator (a real-time
// loop, a plugin hosted by a runtime that owns all device memory and hands out none, a
// context in which cudaMalloc would synchronise the device at a bad moment).  For them the
// scratch lives in a file-scope `static __device__ __align__(256)` array inside the library.
// The caller still passes every input and output; only the scratch is the library's.
//
// The price.  The array has a fixed size, SANDY_DECODE_STATIC_SCRATCH_FLOATS floats (4 MiB),
// and every GPU that loads this library holds those 4 MiB until the process exits.  A call
// whose shape needs more, n_tokens * n_heads * num_splits * (head_dim + 2) floats, is refused
// with SANDY_ERR_STATIC_SCRATCH (-3) and nothing is launched; use fewer splits or the
// ordinary entry point then.  sandy_decode_attention_static_strerror() turns the codes of
// this entry point into text.
//
// Rules of use.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress,
//    once per device, with that device current) and remembers it.  Make that first call
//    outside any stream capture; later calls only launch kernels.
//  * It calls no cudaMalloc, cudaFree, or any allocating routine, of CUDA or of any library.
//  * All calls on a device share the one array, and it keeps whatever the last call left in
//    it.  Nothing in it has to start at zero: every slot a call reads was written by that
//    same call's first kernel.  But two calls that overlap on the GPU (different streams, or
//    the same graph launched twice at once) race on it; serialise them.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SANDY_DECODE_STATIC_SCRATCH_FLOATS (1u << 20)
#define SANDY_ERR_STATIC_SCRATCH (-3)   /* the shape needs more scratch than the static array holds */
#define SANDY_ERR_STATIC_SETUP (-4)     /* the array's device address could not be obtained */

/* Arguments as sandy_decode_attention(), without the scratch pointer. */
int sandy_decode_attention_static(const void* q, int ld_q, const void* k_cache, const void* v_cache,
                                  long long page_stride, const int* block_table, int max_blocks,
                                  const int* token_seq, const int* positions, void* out, int ld_out,
                                  int n_tokens, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                  float scale, int window, int num_splits, int num_pages, int dtype,
                                  int* status, cudaStream_t stream);

/* Capacity of the static scratch, in floats. */
long long sandy_decode_attention_static_capacity(void);

/* A sentence for a return code of sandy_decode_attention_static(). */
const char* sandy_decode_attention_static_strerror(int code);

#ifdef __cplusplus
}
#endif
