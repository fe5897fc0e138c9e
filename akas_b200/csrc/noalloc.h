/* akas_decode_attention_bf16_noalloc: split-key decode attention that allocates nothing.
 *
 * This entry point has no counterpart in kreasof-ai/akas; it exists for callers of this library.
 *
 * akas_decode_attention_bf16 (attention_decode.cu) cuts the keys of every request across several blocks and
 * needs float32 scratch for the blocks' partial results, which its caller allocates. Some callers cannot
 * allocate when they need to call it: a serving process that handed all free device memory to its page pool
 * at start-up has nothing left for cudaMalloc to give; a step loop that must not stall cannot afford
 * cudaMalloc and cudaFree, which may synchronise the whole device; and a host program that calls this
 * library through its C symbols may have no allocator (torch's or its own) to lend. For them the scratch
 * lives inside the library: a file-scope device array of AKAS_DECODE_NOALLOC_FLOATS float32 (4 MiB) that every
 * GPU which loads attention_decode's library holds from load until the process exits.
 *
 * The caller passes inputs and output only (same layouts as akas_decode_attention_bf16). A call needs
 * tokens * heads * splits * (head_dim + 2) floats of scratch; if that exceeds AKAS_DECODE_NOALLOC_FLOATS the
 * call launches nothing and returns AKAS_NOALLOC_TOO_LARGE. Use fewer splits or fewer tokens per call then,
 * or the allocating entry point.
 *
 * The first call on a device looks up the device address of the array (with that device current) and keeps
 * it; make that first call before any stream capture begins. The entry point calls no cudaMalloc, no
 * cudaFree and no allocating library routine.
 *
 * All calls on a device share the one array, and it keeps what the last call left. Nothing in it has to be
 * zero: every slot that a call's merge reads, that call's blocks have written first (blocks whose share of
 * the keys is empty write an empty partial). Two calls that overlap on the GPU (different streams, or the
 * same call issued from two threads) race on the array and give wrong results; calls on one stream, one
 * after the other, are safe.
 *
 * Returns 0, a CUDA error code (> 0), or one of the negative codes below; akas_noalloc_error_string gives
 * a sentence for any of them.
 */
#pragma once

#include <cuda_runtime.h>

#define AKAS_DECODE_NOALLOC_FLOATS (1 << 20)
#define AKAS_NOALLOC_TOO_LARGE (-2)  /* the call needs more scratch than the library holds */
#define AKAS_NOALLOC_NO_SYMBOL (-3)  /* the device address of the scratch array could not be found */
#define AKAS_NOALLOC_BAD_ARGUMENT (-4)

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int akas_decode_attention_bf16_noalloc(
    const void* q, const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
    const int* seq_of_token, const int* positions, void* out, float scale, int window, int page_size, int tokens,
    int heads, int kv_heads, int head_dim, int splits, cudaStream_t stream);

/* How many float32 of scratch a call would need; compare with AKAS_DECODE_NOALLOC_FLOATS. Sizes whose product
 * is beyond the array (or beyond 64 bits) all give AKAS_DECODE_NOALLOC_FLOATS + 1. */
__attribute__((visibility("default"))) long long akas_decode_attention_bf16_noalloc_needs(int tokens, int heads,
                                                                                          int splits, int head_dim);

__attribute__((visibility("default"))) const char* akas_noalloc_error_string(int code);

#ifdef __cplusplus
}
#endif
