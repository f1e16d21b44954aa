// Decode attention for callers that may not allocate device memory.
//
// This entry point has no counterpart in samplecatalina/mini-serve; it exists for embedders of
// this library. Some hosts run the kernels from a context in which cudaMalloc (and every
// allocating library call, a tensor library's allocator included) is off limits: a real-time
// loop that must not take the allocator's locks or risk an implicit device synchronisation, a
// plugin that is handed its input and output buffers and forbidden to own memory, or code that
// runs after the process has fixed its memory budget. The split-K decode kernel needs scratch
// memory for its partial results, so for those callers the scratch lives inside the library.
//
// ms_attn_bf16_d<D>_decode_noalloc (one per head size D, in libms_attn_bf16_d<D>.so) computes
// exactly what ms_attn_bf16_d<D>_decode computes, with the same arguments except that the two
// scratch pointers are gone. The partial results go to a file-scope __device__ array of
// MS_ATTN_NOALLOC_SCRATCH_FLOATS floats (4 MiB) that every GPU which loads the library holds until
// the process exits.
//
//  * Limit: rows * query_heads * splits * (D + 2) must not exceed MS_ATTN_NOALLOC_SCRATCH_FLOATS;
//    larger calls are refused with an error (return code 1, text from ..._last_error()) and
//    nothing is launched. A call with splits == 1 needs no scratch at all.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current), sets the kernel's shared-memory attribute for that device and remembers
//    both. Make that first call outside any stream capture, and from one thread: the tables that
//    remember are filled without a lock, so the first call on a device must not run beside another
//    call of this library; later calls may come from any thread.
//  * The call allocates nothing: no cudaMalloc, cudaFree or allocating library routine.
//  * All calls share the one array, and it keeps what the last call left. Nothing in it has to
//    start at zero: every partial result that the merge reads was written by the same call
//    first. But two calls that overlap on the GPU (different streams, or a graph replayed on
//    another stream) race on it; keep calls that use it in one stream order.
#pragma once

#include <cuda_runtime.h>

#define MS_ATTN_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Declared here for head size 128 as an example of the naming; every compiled head size D exports
// the same signature as ms_attn_bf16_d<D>_decode_noalloc.
//
// out:          [rows, query_heads, D] bfloat16, written
// q:            [rows, query_heads, D] bfloat16 (one new token per request)
// k_pool/v_pool:[pages, kv_heads, page_size, D] bfloat16
// kv_len:       [rows] int32, tokens of each request in the cache (the new one included)
// page_indptr:  [rows + 1] int32; page_indices: page ids of every request, back to back
// num_splits:   how many ways each request's keys are cut across CTAs (>= 1)
// Returns 0 on success.
int ms_attn_bf16_d128_decode_noalloc(void* out, const void* q, const void* k_pool, const void* v_pool,
                                     const int* kv_len, const int* page_indptr, const int* page_indices,
                                     int num_rows, int query_heads, int kv_heads, float scale, int window,
                                     int page_size, int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
