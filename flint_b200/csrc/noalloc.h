/* flint_paged_attention_noalloc: paged attention with a split key range whose scratch memory
 * lives inside the library instead of being passed in.
 *
 * This entry point has no counterpart in the reference project (formetaohy/Flint); it exists
 * for callers that cannot allocate device memory at the moment of the call.  Examples: a host
 * program that has handed all of the GPU's memory to its own pool at start-up, so that a
 * cudaMalloc made on its behalf would fail; a latency-critical loop in which cudaMalloc's
 * implicit device-wide synchronisation would stall the other streams; a plug-in that is only
 * given input and output buffers and no allocator.  Such a caller still passes inputs and
 * outputs, and nothing else.
 *
 * The scratch is one file-scope device array of FLINT_NOALLOC_SCRATCH_BYTES (32 MiB).  Every
 * GPU on which this library is loaded holds that array until the process exits.  A call whose
 * splits need more than that is refused with an error (see flint_noalloc_last_error); callers
 * can ask flint_paged_attention_noalloc_floats for the need of a shape beforehand.
 *
 * Set-up: the first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first call
 * outside any stream capture.  Neither that set-up nor any later call calls cudaMalloc,
 * cudaFree or an allocating library routine.
 *
 * Sharing: all calls on a device use the same array and it keeps the previous call's contents.
 * Nothing in it has to start at zero: the attention kernel writes every (row, head, split)
 * record, empty splits included, before the merge kernel reads it.  Two calls that overlap on
 * the GPU (different streams, no dependency between them) race on the array; put them on one
 * stream or order them with events.
 *
 * Arguments are those of flint_paged_attention without the scratch pointer:
 *   q, out      [T, nq*hd] float32 (q_dtype = 0) or bfloat16 (1); out_dtype must equal q_dtype
 *   k_cache, v_cache   pages [page, nkv, page_size, hd], float32 or bfloat16 (cache_dtype)
 *   block_table [slots, max_pages] int32; pos, slot [T] int32
 *   window 0 = every earlier key; scale multiplies q.k; the key range of each row is cut into
 *   n_splits pieces of split_keys keys (n_splits * split_keys must cover the longest range).
 * Returns 0, or a negative value with the reason in flint_noalloc_last_error().
 */
#pragma once
#include <cuda_runtime.h>

#define FLINT_NOALLOC_SCRATCH_BYTES (32u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int flint_paged_attention_noalloc(const void* q, int q_dtype, const void* k_cache, const void* v_cache,
                                  int cache_dtype, const int* block_table, int max_pages, int page_size,
                                  const int* pos, const int* slot, void* out, int out_dtype, int T, int nq,
                                  int nkv, int hd, int window, float scale, int split_keys, int n_splits,
                                  cudaStream_t stream);

/* Floats of scratch a call of this shape needs (0 for n_splits == 1); the limit is
 * FLINT_NOALLOC_SCRATCH_BYTES / 4. */
long long flint_paged_attention_noalloc_floats(int T, int nq, int hd, int n_splits);

const char* flint_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
