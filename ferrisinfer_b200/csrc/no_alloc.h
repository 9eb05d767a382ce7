// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference; it exists for embedders of this library.  Some code
// that wants to run split-KV decode attention is not in a position to obtain device memory: a
// plugin that runs inside another framework's stream callback or memory-pool scope, a process
// whose device memory was handed out in full at start-up, or code inside a region where the CUDA
// allocator may not be entered at all.  The regular entry point (ferris_decode_attention) expects
// such a caller to bring a scratch buffer for the per-split partial results; this one brings its
// own.
//
// The scratch is a fixed array in the library's device image: FERRIS_STATIC_SCRATCH_FLOATS floats
// (8 MiB), present on every GPU that loads the library for as long as the process lives.  Requests
// whose partial results would not fit, tokens * heads * splits * (head_dim + 2) floats, are refused
// with FERRIS_BAD_ARGUMENT and a message; nothing runs in that case.
//
// What the caller must know:
//  * The function calls no cudaMalloc, cudaFree or other allocating routine.  The first call on a
//    device looks up the array's device address (cudaGetSymbolAddress) and remembers it; make that
//    first call outside of any stream capture.  Later calls only launch kernels on `stream`.
//  * All calls on a device share the one array.  Two calls whose kernels may run at the same time
//    (different streams, no ordering between them) overwrite each other's partial results and give
//    wrong output; order them.  Calls on one stream are safe.
//  * The array keeps whatever the last call left in it.  That is harmless: every slot that the
//    merge step reads is written first by the same call, so nothing has to start at zero.
//  * Inputs, outputs and their meaning are exactly those of ferris_decode_attention.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define FERRIS_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

// q: bf16 rows of ldq elements, the first nh*d of each are the query heads of one token.
// out: bf16 [tokens, nh*d] rows of ldo elements.  k_cache / v_cache: bf16 [cache_pages, nkv,
// page_size, d].  block_tables: int32 [requests, max_blocks].  token_seq / positions: int32 [tokens].
// splits >= 1: into how many key ranges each token's keys are cut.  Returns 0, a cudaError_t (> 0),
// or FERRIS_BAD_ARGUMENT (< 0; ferris_last_error() has the text).
__attribute__((visibility("default"))) int ferris_decode_attention_static_scratch(
    const void* q, int ldq, void* out, int ldo, const void* k_cache, const void* v_cache, long long cache_pages,
    const int* block_tables, int max_blocks, const int* token_seq, const int* positions, int tokens, int nh, int nkv,
    int d, int page_size, int window, float scale, int splits, void* stream);

#ifdef __cplusplus
}
#endif
