// Attention over the paged cache for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts
// that use this library's kernels directly through the C interface.
//
// Who cannot allocate: a host that planned its device memory up front and gave
// every byte a purpose (weights, cache pages, workspace) has no budget line for
// a kernel's private scratch, and a late cudaMalloc there can fail or eat into
// the reserve it promised to keep free; a decode loop that must not stall cannot
// afford cudaMalloc or cudaFree either, because both may synchronise the whole
// device; and a plain C or C++ host has no tensor library to hand it a buffer.
// `mdma_attention_mma` asks such a caller for a scratch pointer whenever the
// keys are split over several blocks.  `mdma_attention_mma_noalloc` does the
// same computation with the same arguments, minus the scratch: the split
// partials go to a fixed array that is part of the loaded library.
//
// Limit: the array holds MDMA_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  A call
// needs n_tokens * n_heads * splits * (head_dim + 2) floats when splits > 1 and
// none when splits == 1; a call that needs more is refused with an error, never
// truncated.  Every GPU on which the library is loaded holds the array until
// the process exits.
//
// Set-up: the first call on a device looks up the array's device address (the
// array's name is only a host-side handle; it is not an address a kernel can
// use) and keeps it.  Make that first call on each device, with that device
// current, before any stream capture begins.
//
// Sharing: all calls on a device use the same array, and it keeps what the last
// call left in it.  Nothing in it has to start at zero: the attention kernel
// writes every partial (output, maximum, sum) of every (token, head, split)
// before the merge reads it.  Two calls that may run at the same time on one
// GPU (different streams) would overwrite each other's partials; issue them on
// one stream, or order them yourself.
//
// The function calls no cudaMalloc, cudaFree or any other allocating routine.
// Returns 0 on success; otherwise `mdma_last_error()` of this library has the reason.
#pragma once
#include <cuda_runtime.h>

#define MDMA_NOALLOC_SCRATCH_FLOATS (4l * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int mdma_attention_mma_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                               const int* seq_start, const int* seq_pos0, const int* seq_slot,
                               const int* page_table, int max_pages, int page_size, void* out,
                               int n_tokens, int n_seqs, int max_new, int n_heads, int n_kv_heads,
                               int head_dim, int window, float scale, int splits, cudaStream_t stream);

const char* mdma_last_error();

#ifdef __cplusplus
}
#endif
