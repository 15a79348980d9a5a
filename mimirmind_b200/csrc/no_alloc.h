// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference; it is an addition of this library.
//
// Who needs it: code that runs the split-key decode attention from a place where no
// allocation call may be made: inside a region that forbids cudaMalloc (a real-time or
// safety-checked host loop, a plugin whose host hands it only the tensors it declared, a
// process that has given all of the device's memory to one arena up front), or from a
// host language binding that can pass pointers but has no allocator of its own.  The
// ordinary entry point, mm_attention_decode_bf16, needs two scratch buffers from its
// caller for the partial results of the key splits; this one brings its own.
//
// How: the scratch lives in a file-scope `static __device__` array inside the library, of
// MM_NO_ALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU that loads the library holds these
// 16 MiB until the process exits, whether the entry point is ever called or not.
//
// Rules for callers:
//   * The inputs and the output are still the caller's.  Only the scratch is internal.
//   * A call needs n_items * H * max_splits * (head_dim + 2) floats of scratch.  If that is
//     more than MM_NO_ALLOC_SCRATCH_FLOATS the call is refused with MM_ERR_BAD_ARG and a
//     message (mm_last_error) that states both numbers; nothing is launched.  With
//     max_splits == 1 no scratch is used at all.
//   * The first call on each device looks up the array's device address (one
//     cudaGetSymbolAddress with that device current).  Make that first call before any
//     stream capture begins on that device.  Later calls do no set-up.
//   * The function calls no cudaMalloc, cudaFree, or any routine that allocates.
//   * All calls share the one array and it keeps whatever the last call left in it.  The
//     kernels write every partial result they later read, so nothing has to be cleared
//     between calls.  Two calls whose kernels may run at the same time on one GPU (two
//     streams, two threads) race on the array: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define MM_NO_ALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// Same arguments and result as mm_attention_decode_bf16 without part_o / part_ml.
int mm_attention_decode_bf16_no_alloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const void* items, int n_items, const void* positions, const void* token_req,
                                      const void* block_table, int table_width, int page_size, int H, int G, int hd,
                                      int window, float scale, int split_len, int max_splits, void* stream);

#ifdef __cplusplus
}
#endif
