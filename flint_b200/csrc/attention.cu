// Attention over the paged cache, for prefill portions and decoded tokens alike.
//
// Every query row t has a position pos[t] and a request slot slot[t] (with a row list, T counts
// the listed rows and t = row_list[i]); it sees the keys
// of its request at positions lo..pos[t], lo = max(0, pos[t]+1-window) (window 0: all).
// Key j of a request lives in page block_table[slot, j / P] at row j % P; pages are
// [page, kv_head, P, head_dim].  Scores, the running maximum, the sum and the output
// are float32 (online softmax over blocks of 32 keys).
//
// Work is split as (row, kv head, chunk of up to 4 query heads of that kv head, split of
// the key range): one warp each.  In the score phase a lane owns a key and computes
// the dot products of up to 4 query heads with it; in the value phase a lane owns
// head_dim/32 output dims and the probabilities are broadcast by shuffle.  With more
// than one split each warp writes (max, sum, unnormalised output) to scratch and a
// second kernel merges the splits in a fixed order, so results do not depend on timing.
//
// Reference counterpart: crates/thuban_kernel/wgsl/attn.wgsl (8 query rows x 128 keys,
// one dispatch per sequence chunk; window and causal mask at :78-90).
#include "attention_kernels.cuh"

using namespace flint;

// Number of floats of scratch that flint_paged_attention needs for n_splits > 1.
extern "C" long long flint_paged_attention_scratch_floats(int T, int nq, int hd, int n_splits) {
  return n_splits > 1 ? (long long)T * nq * n_splits * (hd + 2) : 0;
}

extern "C" int flint_paged_attention(const void* q, int q_dtype, const void* k_cache,
                                     const void* v_cache, int cache_dtype, const int* block_table,
                                     int max_pages, int page_size, const int* pos, const int* slot,
                                     void* out, int out_dtype, int T, int nq, int nkv, int hd,
                                     int window, float scale, int split_keys, int n_splits,
                                     float* scratch, const int* row_list, cudaStream_t stream) {
  return flint_attn::paged_attention_launch(q, q_dtype, k_cache, v_cache, cache_dtype, block_table, max_pages,
                                            page_size, pos, slot, out, out_dtype, T, nq, nkv, hd, window, scale,
                                            split_keys, n_splits, scratch, stream, row_list);
}

// The same contract with the block kernel (one block per row, kv head and split): for decode.
extern "C" int flint_paged_attention_block(const void* q, int q_dtype, const void* k_cache,
                                           const void* v_cache, int cache_dtype, const int* block_table,
                                           int max_pages, int page_size, const int* pos, const int* slot,
                                           void* out, int out_dtype, int T, int nq, int nkv, int hd,
                                           int window, float scale, int split_keys, int n_splits,
                                           float* scratch, const int* row_list, cudaStream_t stream) {
  return flint_attn::paged_attention_block_launch(q, q_dtype, k_cache, v_cache, cache_dtype, block_table, max_pages,
                                                  page_size, pos, slot, out, out_dtype, T, nq, nkv, hd, window,
                                                  scale, split_keys, n_splits, scratch, stream, row_list);
}

extern "C" const char* flint_attention_last_error() { return g_error; }
