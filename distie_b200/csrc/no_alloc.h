// distie_attention_decode_static: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference project; it exists for
// callers of this library that cannot call cudaMalloc at the point where they
// need attention: code that runs inside a memory budget fixed at start-up (every
// byte of the device handed out in advance, for instance to the cache slab),
// plug-ins that are handed tensors but no allocator, and latency-critical loops in
// which an allocation (and the implicit synchronisation it may bring) is not
// acceptable.  The ordinary entry point, distie_attention_decode, wants a scratch
// buffer from its caller whenever the keys are split; this one keeps that scratch
// inside the library instead.
//
// What it does: exactly distie_attention_decode (same arguments without `scratch`,
// same kernels, same results), with the partial results of the splits written to a
// file-scope device array of DISTIE_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every
// GPU that loads the library holds that array until the process exits.
//
// Limits and rules
//  * tokens * heads * splits * (head_dim + 2) must not exceed
//    DISTIE_STATIC_SCRATCH_FLOATS when splits > 1; a larger request is refused with
//    DISTIE_ERR_SCRATCH_TOO_SMALL and nothing is launched.
//    distie_no_alloc_error(code) gives the words for a code.
//  * The first call on each device looks up the array's device address (once, with
//    that device current).  Make that first call outside any stream capture.
//  * The array that is used is the CURRENT device's (cudaGetDevice at the time of the
//    call).  `stream` and every pointer must belong to that device: make the device
//    that owns the stream current before calling.  The entry point does not check it.
//  * `positions` must lie inside the block table (position / page_size < table_width);
//    a position beyond it reads no memory: its keys count as missing pages and the
//    error word is set to 4.
//  * It calls no cudaMalloc, cudaFree or any other allocating routine, of CUDA or of
//    a tensor library; inputs and outputs are the caller's.
//  * All calls share the one array and it keeps what the last call left there.  No
//    part of it needs clearing, because every value the merge reads was written by
//    the same call before.  Two calls that overlap on the GPU (different streams
//    without an ordering between them) race on it: order them.
#pragma once

#include <cuda_runtime.h>

#define DISTIE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define DISTIE_ERR_SCRATCH_TOO_SMALL (-3)

#ifdef __cplusplus
extern "C" {
#endif

// Floats the array holds.
long long distie_attention_decode_static_capacity(void);

// Words for a return code of distie_attention_decode_static.
const char* distie_no_alloc_error(int code);

// Returns 0, a negative DISTIE_ERR_* code, or a cudaError_t of the set-up or the launch.
int distie_attention_decode_static(const void* q, int q_row_stride, void* out, int out_row_stride,
                                   const int* positions, const int* token_seq, const int* seq_seat,
                                   const int* block_table, int table_width, const void* k_cache,
                                   const void* v_cache, int tokens, int num_heads, int num_kv_heads, int head_dim,
                                   int page_size, int num_pages, int window, float scale, int num_splits, int dtype,
                                   int* error, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
