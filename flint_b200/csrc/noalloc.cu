// The allocation-free variant of the paged attention: same kernels as attention.cu, with the
// partial results of a split key range kept in a static device array of this library.
// What it is for, its limit and its rules of use are written in noalloc.h.
#include "noalloc.h"

#include "attention_kernels.cuh"

using namespace flint;

namespace {

// The scratch itself.  In host code this name is only a stand-in for the symbol, never a device
// address: the address is looked up once per device below and passed to the kernels.
static __device__ __align__(256) float g_scratch[FLINT_NOALLOC_SCRATCH_BYTES / sizeof(float)];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {};

// Device address of the array on the current device, looked up on the first call there.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail("noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= MAX_DEVICES) return fail("noalloc: device %d is out of range", dev);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_scratch);
    if (e != cudaSuccess || !p)
      return fail("noalloc: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" long long flint_paged_attention_noalloc_floats(int T, int nq, int hd, int n_splits) {
  return n_splits > 1 ? (long long)T * nq * n_splits * (hd + 2) : 0;
}

extern "C" int flint_paged_attention_noalloc(const void* q, int q_dtype, const void* k_cache,
                                             const void* v_cache, int cache_dtype, const int* block_table,
                                             int max_pages, int page_size, const int* pos, const int* slot,
                                             void* out, int out_dtype, int T, int nq, int nkv, int hd, int window,
                                             float scale, int split_keys, int n_splits, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (nq <= 0 || hd <= 0 || n_splits < 1) return fail("noalloc: bad sizes (heads %d, head size %d, splits %d)", nq, hd, n_splits);
  const long long need = flint_paged_attention_noalloc_floats(T, nq, hd, n_splits);
  const long long have = FLINT_NOALLOC_SCRATCH_BYTES / sizeof(float);
  if (need > have)
    return fail("noalloc: %d rows x %d heads x %d splits of head size %d need %lld bytes of scratch, the built-in "
                "array has %lld; use fewer splits or rows, or the entry point that takes a scratch pointer",
                T, nq, n_splits, hd, need * 4, have * 4);
  float* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  return flint_attn::paged_attention_launch(q, q_dtype, k_cache, v_cache, cache_dtype, block_table, max_pages,
                                            page_size, pos, slot, out, out_dtype, T, nq, nkv, hd, window, scale,
                                            split_keys, n_splits, scratch, stream);
}

extern "C" const char* flint_noalloc_last_error() { return g_error; }
