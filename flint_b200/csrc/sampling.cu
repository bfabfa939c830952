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

// first-max-wins arg-max of one row
__device__ __forceinline__ int block_argmax(const float* s, int V, float* red, int* redi) {
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
// work [R, V]: scratch for the penalised scores / probabilities.
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ params,
              const int* __restrict__ context, int max_context, float* __restrict__ work,
              int* __restrict__ out, int V) {
  __shared__ float red[33];
  __shared__ int redi[32];
  __shared__ unsigned sh_u[2];
  const int r = blockIdx.x;
  const float* prm = params + (size_t)r * 8;
  const float temperature = prm[0];
  const int top_k = (int)prm[1];
  const float top_p = prm[2], min_p = prm[3], penalty = prm[4], u = prm[5];
  const int n_ctx = min((int)prm[6], max_context);
  const float* src = logits + (size_t)r * V;
  float* p = work + (size_t)r * V;

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
    unsigned lo = 0u, hi = 0x7f800000u;   // probabilities are finite and >= 0
    // largest bit pattern b with count(p >= b) >= k
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1) / 2;
      float cnt = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += (__float_as_uint(p[i]) >= mid) ? 1.f : 0.f;
      cnt = block_sum_f(cnt, red);
      if ((int)cnt >= top_k) lo = mid; else hi = mid - 1;
    }
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
    float mass_all = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mass_all += p[i] / s_k;
    mass_all = block_sum_f(mass_all, red);
    if (mass_all >= top_p) {
      while (lo < hi) {
        const unsigned mid = lo + (hi - lo + 1) / 2;
        float mass = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x)
          mass += (__float_as_uint(p[i]) >= mid) ? p[i] / s_k : 0.f;
        mass = block_sum_f(mass, red);
        if (mass >= top_p) lo = mid; else hi = mid - 1;
      }
      const unsigned thr_p = lo;
      float mass_gt = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x)
        mass_gt += (__float_as_uint(p[i]) > thr_p) ? p[i] / s_k : 0.f;
      mass_gt = block_sum_f(mass_gt, red);
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
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, params, context, max_context, work, out, V);
  return check_launch("sample");
}

extern "C" const char* flint_sampling_last_error() { return g_error; }
