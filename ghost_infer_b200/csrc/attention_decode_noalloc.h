// An entry point of the decode attention that allocates nothing.  (It has no counterpart in the reference,
// whose sessions own every buffer they use: src/cuda.rs:9826-9870.)
//
// Who needs it: code that drives these kernels from a place where device memory cannot be asked for.  A host
// program that holds no allocator of its own, a plug-in loaded into somebody else's process under a fixed
// memory budget, or a caller in the middle of a latency-critical loop where cudaMalloc would synchronise the
// device all have inputs and outputs already, but nowhere to get the scratch that cutting a context into
// slices needs (the per-slice partial outputs, maxima and sums that gi_attn_decode_tc takes as `part_o` and
// `part_ml`).  For them the scratch lives inside the library, in a file-scope device array of
// GI_NOALLOC_SCRATCH_FLOATS floats (8 MiB); every GPU that loads the library holds that much until exit.
//
// Same arguments and results as gi_attn_decode_tc, without the two scratch pointers.  Limits and rules:
//  * n_seqs * n_heads * n_splits * (hd + 2) must not exceed GI_NOALLOC_SCRATCH_FLOATS; a larger request is
//    refused with an error before anything is launched.
//  * The first call on a device looks up the array's device address (once per device, with that device
//    current).  Make that first call outside any stream capture.
//  * All calls share the one array, and it keeps what the last call left.  Nothing in it has to start at zero:
//    every slice a launch reads was written by that launch.  Two calls whose kernels overlap on the GPU
//    (different streams, no ordering between them) race on the array; order them.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
#pragma once

#define GI_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int gi_attn_decode_tc_noalloc(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                              const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                              int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                              void* stream);

#ifdef __cplusplus
}
#endif
