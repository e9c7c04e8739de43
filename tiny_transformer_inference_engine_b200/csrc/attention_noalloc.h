// Split-key paged attention for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts of this library that
// cannot call cudaMalloc when they need attention computed: a serving process that gave all of
// the GPU's memory to its own pools at start-up, a plug-in that lives under another runtime's
// allocator, a latency-critical loop in which an allocation (which may synchronise the device or
// fail) is not acceptable.  The regular entry point, ttie_paged_attention_mma, takes the scratch
// memory for split-key partial results from its caller; this one owns it.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Number of float32 values of scratch the library holds per GPU (a file-scope device array:
// every GPU that loads the library keeps these 16 MiB until the process exits).
#define TTIE_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// Same arguments and result as ttie_paged_attention_mma without `scratch`.  The scratch for
// num_splits > 1 is the library's own array; a call needs T * Hq * num_splits * (D + 2) floats of
// it and is refused (return value != 0, message in ttie_last_error) if that exceeds
// TTIE_NOALLOC_SCRATCH_FLOATS.  It allocates nothing and frees nothing.
//
// * The first call on a device looks up the array's device address (cudaGetSymbolAddress with
//   that device current).  Make that first call before any stream capture begins.
// * T must be the number of query tokens the requests bring, qsl[num_seqs] (no padding tokens behind
//   them): the pass that adds the splits up reads T * Hq rows of partial results, and only the rows of
//   the requests' own tokens have been written.
// * All calls on a device share the array.  Nothing in it has to start at zero - every entry a
//   call reads, the same call has written - so the last call's contents do no harm; but two calls
//   that overlap on the GPU (different streams, no ordering) race on it.  Order them.
int ttie_paged_attention_mma_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                     const int* block_table, int table_width, int page_size, const int* qsl,
                                     const int* seq_lens, void* out, int T, int num_seqs, int Hq, int Hkv, int D,
                                     int max_q_len, float scale, int window, int num_splits, int split_len,
                                     void* stream);

#ifdef __cplusplus
}
#endif
