// Choosing the next token on the device: arg-max, and temperature sampling with the
// reference's filters in the reference's order (repeat penalty, softmax((s-max)/T), top-k,
// top-p, min-p, renormalise, inverse-CDF draw: crates/thuban_generate/src/sampler.rs:56-109).
// The uniform number of each draw comes from the host, which owns the request's
// generator (splitmix64, sampler.rs:135-142), so host and device samplers can be compared.
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {
constexpr int THREADS = 1024;

// A row of scores / probabilities, in global memory or in shared memory.  In shared memory one float of padding
// follows every 32, so that threads that each walk a run of consecutive entries do not meet in one bank.
struct Row {
  float* p;
  int padded;
  __device__ __forceinline__ float& operator[](int i) const { return p[padded ? i + (i >> 5) : i]; }
};

// ---- block-wide helpers (THREADS threads) ---------------------------------------------
__device__ __forceinline__ float block_sum_f(float v, float* red) { return block_sum(v, red); }

__device__ __forceinline__ float block_max_f(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < (int)(blockDim.x >> 5)) ? red[lane] : -INFINITY;
  return warp_max(r);
}

// exclusive prefix sum over threads (in thread order); returns this thread's prefix, total in *total
__device__ __forceinline__ float block_scan_f(float v, float* red, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) red[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    float w = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
    float winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    red[lane] = winc - w;            // exclusive prefix of warp sums
    if (lane == 31) red[32] = winc;  // total
  }
  __syncthreads();
  *total = red[32];
  return red[warp] + inc - v;
}


// The largest bit pattern b in [lo, hi] for which the weight of {i : bits(p[i]) >= b} reaches `target`
// (the caller makes sure that lo qualifies).  MASS: an entry weighs p[i] / s_k, else 1.  Seven thresholds are
// tried per pass over the row, so 31 bits take 11 passes; each threshold's weight is summed in the order of
// block_sum (per thread in index order, a shuffle tree per warp, a shuffle tree over the warps), so the answer
// is the one a bisection with block_sum would give.
constexpr int NT = 7;
constexpr int FEW = 2048;
template <bool MASS>
__device__ unsigned search_largest(const Row p, int V, unsigned lo, unsigned hi, float target, float s_k,
                                   float (*red_nt)[NT], float* tot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  while (lo < hi) {
    const unsigned step = (hi - lo) / (NT + 1) + 1;
    unsigned t[NT];
    float acc[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      t[j] = lo + step * (unsigned)(j + 1);        // valid while <= hi; t[0] always is
      acc[j] = 0.f;
    }
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = p[i];
      const unsigned b = __float_as_uint(v);
      const float w = MASS ? v / s_k : 1.f;
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j] += (b >= t[j]) ? w : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j] = warp_sum(acc[j]);
    __syncthreads();                                // red_nt and tot may still be read from the pass before
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < NT; ++j) red_nt[warp][j] = acc[j];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        float r = lane < n_warps ? red_nt[lane][j] : 0.f;
        r = warp_sum(r);
        if (lane == 0) tot[j] = r;
      }
    }
    __syncthreads();
    // the sets are nested, so the thresholds that qualify are a prefix: the last of them is the new lower end,
    // the one after it (if it is in range) bounds the upper end
    unsigned new_lo = lo, new_hi = t[0] - 1;
#pragma unroll
    for (int j = 0; j < NT; ++j)
      if (t[j] <= hi && tot[j] >= target) {
        new_lo = t[j];
        new_hi = (j + 1 < NT && t[j + 1 < NT ? j + 1 : j] <= hi) ? t[j + 1 < NT ? j + 1 : j] - 1 : hi;
      }
    lo = new_lo;
    hi = new_hi;
  }
  return lo;
}

// first-max-wins arg-max of one row
template <typename R>
__device__ __forceinline__ int block_argmax(const R s, int V, float* red, int* redi) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = s[i];
    if (v > best) { best = v; bi = i; }
  }
  // reduce (value desc, index asc)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { red[warp] = best; redi[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < (int)(blockDim.x >> 5) ? red[lane] : -INFINITY;
    bi = lane < (int)(blockDim.x >> 5) ? redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) redi[0] = bi == 0x7fffffff ? 0 : bi;
  }
  __syncthreads();
  return redi[0];
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  __shared__ float red[33];
  __shared__ int redi[32];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int tok = block_argmax(logits + (size_t)r * V, V, red, redi);
  if (threadIdx.x == 0) out[r] = tok;
}

// Per-row parameters, 8 floats: temperature, top_k, top_p, min_p, repeat_penalty, u, n_context, unused
// work [R, V]: the penalised scores, then the filtered probabilities of every row (left there at the end).  The
// row is worked on in shared memory if it fits (row_in_smem), else in `work`.
__global__ void __launch_bounds__(THREADS, 1)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ params,
              const int* __restrict__ context, int max_context, float* __restrict__ work,
              int* __restrict__ out, int V, int row_in_smem) {
  extern __shared__ float row_s[];
  __shared__ float red[33];
  __shared__ float red_nt[32][NT];
  __shared__ float tot[NT];
  __shared__ int redi[32];
  __shared__ unsigned sh_u[2];
  __shared__ float few[FEW];           // a short list of entries that a search can be confined to
  __shared__ float tmax_s[THREADS];
  __shared__ int n_few;
  const int r = blockIdx.x;
  const float* prm = params + (size_t)r * 8;
  const float temperature = prm[0];
  const int top_k = (int)prm[1];
  const float top_p = prm[2], min_p = prm[3], penalty = prm[4], u = prm[5];
  const int n_ctx = min((int)prm[6], max_context);
  const float* src = logits + (size_t)r * V;
  float* const kept = work + (size_t)r * V;
  const Row p = {row_in_smem ? row_s : kept, row_in_smem};

  for (int i = threadIdx.x; i < V; i += blockDim.x) p[i] = src[i];
  __syncthreads();
  if (penalty != 1.0f && threadIdx.x == 0) {
    // one thread, in order: a token that appears twice is penalised twice, as in the reference
    for (int c = 0; c < n_ctx; ++c) {
      const int tok = context[(size_t)r * max_context + c];
      if (tok >= 0 && tok < V) p[tok] = p[tok] > 0.f ? p[tok] / penalty : p[tok] * penalty;
    }
  }
  __syncthreads();
  if (temperature <= 0.f) {
    const int tok = block_argmax(p, V, red, redi);
    if (threadIdx.x == 0) out[r] = tok;
    if (row_in_smem)
      for (int i = threadIdx.x; i < V; i += blockDim.x) kept[i] = p[i];
    return;
  }
  // softmax((s - max) / T)
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, p[i]);
  mx = block_max_f(mx, red);
  const float inv_t = 1.0f / temperature;
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float e = expf((p[i] - mx) * inv_t);
    p[i] = e;
    sum += e;
  }
  sum = block_sum_f(sum, red);
  for (int i = threadIdx.x; i < V; i += blockDim.x) p[i] = p[i] / sum;
  __syncthreads();

  // contiguous ownership for ordered scans
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int c0 = min(V, (int)threadIdx.x * chunk), c1 = min(V, c0 + chunk);

  // ---- top-k: value of the k-th largest probability by bisection on the float bits
  unsigned thr_k = 0u;       // keep p > thr, plus the first `ties_k` entries equal to thr
  int ties_k = 0x7fffffff;
  if (top_k > 0 && top_k < V) {
    // largest bit pattern b with count(p >= b) >= k (probabilities are finite and >= 0; b = 0 counts them all).
    // The k largest of the threads' own maxima are k different entries, so the k-th largest entry is at least
    // the k-th largest of those maxima: the search runs over the (few) entries that reach that bound.
    unsigned lo = 0u;
    bool found = false;
    if (top_k <= (int)blockDim.x) {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
      float tm = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) tm = fmaxf(tm, p[i]);
      tmax_s[threadIdx.x] = tm;
      const float wm = warp_max(tm);
      if (threadIdx.x == 0) { n_few = 0; sh_u[0] = 0u; }
      __syncthreads();
      if (lane == 0) red[warp] = wm;
      __syncthreads();
      unsigned bound;
      if (top_k <= n_warps) {
        // the k-th largest of the warps' maxima, by counting in one warp how many are ahead of each
        if (warp == 0) {
          const float mine = lane < n_warps ? red[lane] : -1.f;
          int ahead = 0;
          for (int o = 0; o < 32; ++o) {
            const float other = __shfl_sync(0xffffffffu, mine, o);
            ahead += (other > mine || (other == mine && o < lane)) ? 1 : 0;
          }
          if (lane < n_warps && ahead == top_k - 1) sh_u[0] = __float_as_uint(mine);
        }
        __syncthreads();
        bound = sh_u[0];
      } else {
        const Row maxima = {tmax_s, 0};
        bound = search_largest<false>(maxima, blockDim.x, 0u, 0x7f800000u, (float)top_k, 1.f, red_nt, tot);
      }
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = p[i];
        if (__float_as_uint(v) >= bound) {
          const int at = atomicAdd(&n_few, 1);       // the order does not matter to a count
          if (at < FEW) few[at] = v;
        }
      }
      __syncthreads();
      const int n = n_few;
      if (n <= (int)blockDim.x) {
        // few candidates: the k-th largest is the one with k - 1 candidates ahead of it
        if ((int)threadIdx.x < n) {
          const float mine = few[threadIdx.x];
          int ahead = 0;
          for (int j = 0; j < n; ++j) {
            const float other = few[j];
            ahead += (other > mine || (other == mine && j < (int)threadIdx.x)) ? 1 : 0;
          }
          if (ahead == top_k - 1) sh_u[1] = __float_as_uint(mine);
        }
        __syncthreads();
        lo = sh_u[1];
        found = true;
      } else if (n <= FEW) {
        const Row list = {few, 0};
        lo = search_largest<false>(list, n, bound, 0x7f800000u, (float)top_k, 1.f, red_nt, tot);
        found = true;
      }
      __syncthreads();
    }
    if (!found) lo = search_largest<false>(p, V, 0u, 0x7f800000u, (float)top_k, 1.f, red_nt, tot);
    thr_k = lo;
    float gt = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) gt += (__float_as_uint(p[i]) > thr_k) ? 1.f : 0.f;
    gt = block_sum_f(gt, red);
    ties_k = top_k - (int)gt;
  }
  // drop what top-k drops (in place), ties in index order
  {
    float my_ties = 0.f;
    for (int i = c0; i < c1; ++i) my_ties += (__float_as_uint(p[i]) == thr_k) ? 1.f : 0.f;
    float total;
    float before = block_scan_f(my_ties, red, &total);
    int rank = (int)before;
    for (int i = c0; i < c1; ++i) {
      const unsigned b = __float_as_uint(p[i]);
      if (b < thr_k) p[i] = 0.f;
      else if (b == thr_k) { if (rank >= ties_k) p[i] = 0.f; ++rank; }
    }
  }
  __syncthreads();
  float pmax = 0.f, s_k = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) { pmax = fmaxf(pmax, p[i]); s_k += p[i]; }
  pmax = block_max_f(pmax, red);
  s_k = block_sum_f(s_k, red);

  // ---- top-p: smallest prefix (descending) whose mass / s_k reaches top_p
  if (top_p < 1.0f) {
    // largest bit pattern b with mass(p >= b) / s_k >= top_p ; none -> keep all
    unsigned lo = 1u, hi = 0x7f800000u;
    // after top-k few entries are left: they are listed (in index order, so that sums have one order) and the
    // search runs over the list; else over the whole row
    float my_kept = 0.f;
    for (int i = c0; i < c1; ++i) my_kept += p[i] > 0.f ? 1.f : 0.f;
    float n_kept;
    const float kept_before = block_scan_f(my_kept, red, &n_kept);
    const bool listed = n_kept <= (float)FEW;
    if (listed) {
      int at = (int)kept_before;
      for (int i = c0; i < c1; ++i)
        if (p[i] > 0.f) few[at++] = p[i];
    }
    __syncthreads();
    const Row over = listed ? Row{few, 0} : p;
    const int n_over = listed ? (int)n_kept : V;
    const bool direct = listed && n_over <= 256;
    float mass_all = 0.f;
    unsigned thr_direct = 0u;
    float gt_direct = 0.f;
    if (direct) {
      // The threshold is one of the listed values: the largest one at which the mass of the entries that reach it
      // is enough.  Every thread adds in list order, thread i for the i-th value.
      const float mine = (int)threadIdx.x < n_over ? few[threadIdx.x] : INFINITY;
      float reach = 0.f;
      for (int j = 0; j < n_over; ++j) {
        const float w = few[j] / s_k;
        mass_all += w;
        reach += few[j] >= mine ? w : 0.f;
      }
      if (threadIdx.x == 0) sh_u[0] = 0u;
      __syncthreads();
      if ((int)threadIdx.x < n_over && reach >= top_p) atomicMax(&sh_u[0], __float_as_uint(mine));
      __syncthreads();
      thr_direct = sh_u[0];
      for (int j = 0; j < n_over; ++j) gt_direct += (__float_as_uint(few[j]) > thr_direct) ? few[j] / s_k : 0.f;
    } else {
      for (int i = threadIdx.x; i < n_over; i += blockDim.x) mass_all += over[i] / s_k;
      mass_all = block_sum_f(mass_all, red);
    }
    if (mass_all >= top_p) {
      unsigned thr_p;
      float mass_gt;
      if (direct) {
        thr_p = thr_direct;
        mass_gt = gt_direct;
      } else {
        thr_p = search_largest<true>(over, n_over, lo, hi, top_p, s_k, red_nt, tot);
        mass_gt = 0.f;
        for (int i = threadIdx.x; i < n_over; i += blockDim.x)
          mass_gt += (__float_as_uint(over[i]) > thr_p) ? over[i] / s_k : 0.f;
        mass_gt = block_sum_f(mass_gt, red);
      }
      const float w = __uint_as_float(thr_p) / s_k;
      int need = 1;   // ties at the threshold that the prefix still takes
      {
        float acc = mass_gt + w;
        while (acc < top_p && need < V) { acc += w; ++need; }
      }
      float my_ties = 0.f;
      for (int i = c0; i < c1; ++i) my_ties += (__float_as_uint(p[i]) == thr_p) ? 1.f : 0.f;
      float total;
      float before = block_scan_f(my_ties, red, &total);
      int rank = (int)before;
      for (int i = c0; i < c1; ++i) {
        const unsigned b = __float_as_uint(p[i]);
        if (b < thr_p) p[i] = 0.f;
        else if (b == thr_p) { if (rank >= need) p[i] = 0.f; ++rank; }
      }
      __syncthreads();
    }
  }
  // ---- min-p: keep probabilities >= min_p * max
  if (min_p > 0.f) {
    const float thr = min_p * pmax;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (p[i] < thr && p[i] != pmax) p[i] = 0.f;
    __syncthreads();
  }
  // ---- renormalise and draw: first index whose running sum reaches u
  float s_f = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s_f += p[i];
  s_f = block_sum_f(s_f, red);
  float mine = 0.f;
  for (int i = c0; i < c1; ++i) mine += p[i] / s_f;
  float total;
  const float before = block_scan_f(mine, red, &total);
  if (threadIdx.x == 0) { sh_u[0] = 0xffffffffu; sh_u[1] = 0u; }
  __syncthreads();
  {
    float acc = before;
    int last_kept = -1;
    for (int i = c0; i < c1; ++i) {
      if (p[i] > 0.f) last_kept = i;
      acc += p[i] / s_f;
      if (acc >= u && p[i] > 0.f) { atomicMin(&sh_u[0], (unsigned)i); break; }
    }
    if (last_kept >= 0) atomicMax(&sh_u[1], (unsigned)last_kept);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = sh_u[0] != 0xffffffffu ? (int)sh_u[0] : (int)sh_u[1];
  if (row_in_smem)
    for (int i = threadIdx.x; i < V; i += blockDim.x) kept[i] = p[i];
}
}  // namespace

extern "C" int flint_argmax(const float* logits, int* out, int rows, int V, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return fail("argmax: bad vocabulary %d", V);
  launch_pdl(argmax_kernel, dim3(rows), dim3(THREADS), 0, stream, logits, out, V);
  return check_launch("argmax");
}

extern "C" int flint_sample(const float* logits, const float* params, const int* context,
                            int max_context, float* work, int* out, int rows, int V,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return fail("sample: bad vocabulary %d", V);
  if (!work) return fail("sample: needs a work buffer of rows x V floats");
  // a row of up to 200 KB is worked on in shared memory
  const size_t row_bytes = ((size_t)V + V / 32 + 1) * sizeof(float);      // with the padding
  const int row_in_smem = row_bytes <= 200 * 1024;
  static bool configured = false;
  if (row_in_smem && row_bytes > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail("sample: cannot raise shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  sample_kernel<<<rows, THREADS, row_in_smem ? row_bytes : 0, stream>>>(logits, params, context, max_context, work, out, V,
                                                                     row_in_smem);
  return check_launch("sample");
}

extern "C" const char* flint_sampling_last_error() { return g_error; }
