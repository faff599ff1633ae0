// pl_attention_decode_static: split-context paged attention for decoding that
// allocates nothing.
//
// This entry point has no counterpart in the reference project (xiyiji/paged-llm);
// it is an addition of this library.
//
// Why it exists.  The regular decode attention writes one partial result per
// context split into scratch memory that the caller (the Python side) allocates
// and passes in.  Some programs that want to embed this kernel are not allowed to
// allocate device memory at the moment they call it: a host whose memory pool is
// fixed at start-up and owned by somebody else (an inference server with a
// pre-sized arena), code running between the capture calls of such a host, or a
// plug-in loaded into a process whose allocator must not be entered from this
// thread.  For them the partials live in an array that is part of this shared
// library itself: a file-scope `static __device__` array of PL_STATIC_SCRATCH_BYTES
// (8 MiB).  Every GPU on which the library is loaded holds that array until the
// process exits; that is the price of never allocating.
//
// Contract.
//  * Inputs and outputs are still the caller's: q, the cache layer, the block
//    table, lengths, the work list and the output buffer are device pointers
//    passed in, exactly as for the regular entry point (bfloat16, head sizes in
//    steps of 16 up to 128).
//  * The call rejects a problem whose partials do not fit the array
//    (scratch rows x heads x max_splits x (head_dim + 2) floats > 8 MiB) with a
//    clear error and launches nothing.
//  * It calls no cudaMalloc, cudaFree or any allocating library routine.
//  * The first call on a device resolves the device address of the array
//    (cudaGetSymbolAddress, with that device current) and raises the kernel's
//    shared-memory limit.  Make that first call outside of any stream capture.
//  * All calls on one GPU share the one array, and it keeps what the last call
//    left.  Nothing needs clearing: every partial that the merge step reads is
//    written earlier in the same call.  But two calls that overlap on the GPU
//    (different streams, or a graph replay racing a direct call) race on it;
//    keep calls on one stream or order them yourself.
#pragma once

#include <cuda_runtime.h>

#define PL_STATIC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// work: n_work items of four int32 (request, first scratch row of the request,
// split, splits), as the host-side planner makes them for decoding requests: a
// request may bring at most 16 query rows (new tokens x query heads per kv head).
// scratch_rows: the number of new tokens of all requests in the work list.
// Returns 0, or non-zero with the message in pl_last_error().
int pl_attention_decode_static(const void* q, int q_stride, const void* kv_layer, void* out, int out_stride,
                               const int* block_table, int bt_stride, const int* cu_q, const int* k_lens,
                               const int* work, int n_work, int max_splits, int scratch_rows, int num_heads,
                               int num_kv_heads, int head_dim, int page_size, int window, float scale,
                               cudaStream_t stream);

// Size of the built-in scratch array in bytes.
long long pl_attention_decode_static_capacity(void);

#ifdef __cplusplus
}
#endif
