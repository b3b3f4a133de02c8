/* An entry point for callers that must not allocate device memory.
 *
 * This has no counterpart in Memorithm/NNIS; it exists for users of this library
 * who cannot call cudaMalloc (or anything that calls it for them) at the moment
 * they need decode attention:
 *   - a process that handed all device memory to its own arena at start-up and
 *     has none left for the driver to give out;
 *   - code running where an allocation would stall or break the surrounding
 *     work: inside a latency-critical loop, or on a stream whose neighbours must
 *     not be serialised by the implicit synchronisation of cudaMalloc/cudaFree;
 *   - a host binding without an allocator of its own (plain C, another language's
 *     FFI) that can pass pointers to inputs and outputs but has nothing to make
 *     scratch buffers with.
 *
 * nnis_attention_decode_noalloc computes exactly what nnis_attention_decode_mma
 * computes (decode attention over the paged bfloat16 cache, head sizes 64 and
 * 128, split over the key range), but takes its scratch - the per-split partial
 * records and the per-group tickets - from a fixed array compiled into the
 * library instead of from the caller.
 *
 * Limits and rules:
 *   - The scratch is NNIS_NOALLOC_SCRATCH_BYTES (4 MiB + 16 KiB) per GPU that
 *     loads the library, held until the process exits.
 *   - A call needs n_tokens * heads * n_splits * (head_dim + 2) floats of partial
 *     records (at most NNIS_NOALLOC_PARTIAL_FLOATS) and
 *     n_tokens * kv_heads * ceil(heads / kv_heads / 16) tickets (at most
 *     NNIS_NOALLOC_TICKETS); larger requests return NNIS_ERR_NOALLOC_TOO_LARGE (-5)
 *     and launch nothing.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress; no allocation).  Make that first call outside any
 *     stream capture.
 *   - All calls on a device share the one array.  Each call clears the tickets it
 *     uses on its stream before the kernel; the partial records need no clearing
 *     (every record is written before it is read).  Two calls that can run at the
 *     same time on one GPU (different streams, no dependency) race on the array:
 *     order them.
 *   - No cudaMalloc, cudaFree or allocating library routine is called.
 */
#pragma once

#include <cuda_runtime.h>

#define NNIS_NOALLOC_PARTIAL_FLOATS (1u << 20)
#define NNIS_NOALLOC_TICKETS 4096u
#define NNIS_NOALLOC_SCRATCH_BYTES (NNIS_NOALLOC_PARTIAL_FLOATS * 4u + NNIS_NOALLOC_TICKETS * 4u)
#define NNIS_ERR_NOALLOC_TOO_LARGE (-5)

#ifdef __cplusplus
extern "C" {
#endif

/* Arguments as nnis_attention_decode_mma without `partial`, `tickets` and `pdl`:
 * q [n_tokens, q_stride] bfloat16 (rotated), k_cache/v_cache [pages, kv_heads, 64,
 * head_dim] bfloat16, token_pos/token_seq int32 [n_tokens] (position -1: padding
 * row), page_table int32 [sequences, table_cols], out [n_tokens, heads * head_dim]
 * bfloat16.  Returns 0, a negative argument error, or a positive cudaError_t. */
int nnis_attention_decode_noalloc(const void* q, int q_stride, const void* k_cache,
                                  const void* v_cache, const int* token_pos, const int* token_seq,
                                  const int* page_table, int table_cols, void* out, int n_tokens,
                                  int heads, int kv_heads, int head_dim, int page_size, int window,
                                  float scale, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
