// Kernels and launcher of the paged attention, shared by attention.cu (scratch passed by the
// caller) and noalloc.cu (scratch in a static device array).  See attention.cu for the method.
#pragma once
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

namespace flint_attn {
using namespace flint;

constexpr int GC = 4;          // query heads handled by one warp
constexpr int WARPS = 4;       // warps per block
constexpr int MAX_DPL = 8;     // output dims per lane: head_dim <= 256

template <typename TC>
__device__ __forceinline__ void load8(const TC* p, float* f);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache,
                       const TC* __restrict__ v_cache, const int* __restrict__ block_table,
                       int max_pages, int page_size, const int* __restrict__ pos,
                       const int* __restrict__ slot, TO* __restrict__ out,
                       float* __restrict__ scratch, int T, int nq, int nkv, int hd, int window,
                       float scale, int split_keys, int n_splits, int g_chunks,
                       const int* __restrict__ row_list) {
  extern __shared__ float smem[];  // per warp: GC * hd floats of q
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  const long long n_items = (long long)T * nkv * g_chunks * n_splits;
  if (item >= n_items) return;
  const int split = (int)(item % n_splits);
  long long rest = item / n_splits;
  const int gchunk = (int)(rest % g_chunks);
  rest /= g_chunks;
  const int kvh = (int)(rest % nkv);
  const int ti = (int)(rest / nkv);                 // index into the rows this launch covers
  const int t = row_list ? row_list[ti] : ti;       // row of the batch

  const int G = nq / nkv;
  const int g0 = gchunk * GC;
  const int ng = min(GC, G - g0);          // query heads of this warp
  const int h0 = kvh * G + g0;             // first query head
  const int p = pos[t];
  const int lo_row = window > 0 ? max(0, p + 1 - window) : 0;
  const int lo = lo_row + split * split_keys;
  const int hi = min(p + 1, lo + split_keys);   // keys [lo, hi)
  const int* bt = block_table + (size_t)slot[t] * max_pages;

  float* qs = smem + warp * GC * hd;
  for (int i = lane; i < ng * hd; i += 32)
    qs[i] = to_f32(q[((size_t)t * nq + h0) * hd + i]) * scale;
  __syncwarp();

  const int dpl = (hd + 31) / 32;
  float m[GC], l[GC], acc[GC][MAX_DPL];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) acc[g][i] = 0.f;
  }

  for (int j0 = lo; j0 < hi; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j < hi;
    long long row = -1;   // index of the key's row in [page, kv_head, P] units
    if (valid) {
      const int page = bt[j / page_size];
      if (page >= 0) row = ((long long)page * nkv + kvh) * page_size + (j % page_size);
    }
    float s[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) s[g] = 0.f;
    if (row >= 0) {
      const TC* kr = k_cache + row * hd;
      for (int d = 0; d < hd; d += 8) {   // head_dim is a multiple of 16
        float kf[8];
        load8<TC>(kr + d, kf);
#pragma unroll
        for (int g = 0; g < GC; ++g)
          if (g < ng) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s[g] = fmaf(qs[g * hd + d + e], kf[e], s[g]);
          }
      }
    }
    float pr[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      const float sg = row >= 0 ? s[g] : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sg));
      const bool any = m_new > -INFINITY;               // false only if no key was readable yet
      const float alpha = any ? expf(m[g] - m_new) : 1.f;   // 0 on the first block (m = -inf)
      pr[g] = (any && row >= 0) ? expf(sg - m_new) : 0.f;
      l[g] = l[g] * alpha + warp_sum(pr[g]);
      m[g] = m_new;
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) acc[g][i] *= alpha;
    }
    const int nk = min(32, hi - j0);
    for (int jj = 0; jj < nk; ++jj) {
      const long long vrow = __shfl_sync(0xffffffffu, row, jj);
      float pj[GC];
#pragma unroll
      for (int g = 0; g < GC; ++g) pj[g] = __shfl_sync(0xffffffffu, pr[g], jj);
      if (vrow < 0) continue;
      const TC* vr = v_cache + vrow * hd;
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) {
        const int d = lane + 32 * i;
        if (i < dpl && d < hd) {
          const float vv = to_f32(vr[d]);
#pragma unroll
          for (int g = 0; g < GC; ++g) acc[g][i] = fmaf(pj[g], vv, acc[g][i]);
        }
      }
    }
  }

  if (n_splits == 1) {
#pragma unroll
    for (int g = 0; g < GC; ++g)
      if (g < ng) {
        const float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) {
          const int d = lane + 32 * i;
          if (i < dpl && d < hd) out[((size_t)t * nq + h0 + g) * hd + d] = from_f32<TO>(acc[g][i] * inv);
        }
      }
  } else {
    // scratch [T, nq, n_splits, hd + 2]: unnormalised output, then max, then sum
#pragma unroll
    for (int g = 0; g < GC; ++g)
      if (g < ng) {
        float* dst = scratch + (((size_t)ti * nq + h0 + g) * n_splits + split) * (hd + 2);
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) {
          const int d = lane + 32 * i;
          if (i < dpl && d < hd) dst[d] = acc[g][i];
        }
        if (lane == 0) {
          dst[hd] = m[g];
          dst[hd + 1] = l[g];
        }
      }
  }
}

// Merge the splits of one (row, head): out = sum_s e^{m_s-M} o_s / sum_s e^{m_s-M} l_s.
template <typename TO>
__global__ void attention_combine_kernel(const float* __restrict__ scratch, TO* __restrict__ out,
                                         int hd, int n_splits, int nq, const int* __restrict__ row_list) {
  pdl_launch();
  pdl_wait();
  const size_t rh = blockIdx.x;   // (index of the row in this launch) * nq + head
  const float* base = scratch + rh * n_splits * (hd + 2);
  const size_t out_rh = row_list ? (size_t)row_list[rh / nq] * nq + rh % nq : rh;
  // up to 256 splits: the (max, sum) records are fetched side by side, and the weights
  // e^{m_s-M} are then shared by every output dim
  __shared__ float w_s[256];
  __shared__ float l_s[256];
  if (n_splits <= 256) {
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
      w_s[s] = base[(size_t)s * (hd + 2) + hd];
      l_s[s] = base[(size_t)s * (hd + 2) + hd + 1];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int i = 0; i < n_splits; ++i) M = fmaxf(M, w_s[i]);
    __syncthreads();
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) w_s[s] = w_s[s] > -INFINITY ? expf(w_s[s] - M) : 0.f;
    __syncthreads();
    float L = 0.f;
    for (int i = 0; i < n_splits; ++i) L += w_s[i] * l_s[i];     // fixed order, the same in every thread
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      float o = 0.f;
      for (int s0 = 0; s0 < n_splits; s0 += 8) {          // eight loads in flight, added in order
        float t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) t[u] = s0 + u < n_splits ? base[(size_t)(s0 + u) * (hd + 2) + d] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)      // an empty slot (weight 0) may hold anything, even NaN: it is left out
          if (s0 + u < n_splits && w_s[s0 + u] != 0.f) o += w_s[s0 + u] * t[u];
      }
      out[out_rh * hd + d] = from_f32<TO>(o * inv);
    }
    return;
  }
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[(size_t)s * (hd + 2) + hd]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = base[(size_t)s * (hd + 2) + hd];
    if (ms > -INFINITY) L += expf(ms - M) * base[(size_t)s * (hd + 2) + hd + 1];
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = base[(size_t)s * (hd + 2) + hd];
      if (ms > -INFINITY) o += expf(ms - M) * base[(size_t)s * (hd + 2) + d];
    }
    out[out_rh * hd + d] = from_f32<TO>(o * inv);
  }
}

// Validates the sizes, launches the attention kernel and, with more than one split, the
// kernel that merges the splits.  `scratch` must hold T*nq*n_splits*(hd+2) floats then.
// With a row list, T is the number of listed rows and row_list[i] the batch row of the i-th.
inline int paged_attention_launch(const void* q, int q_dtype, const void* k_cache,
                                     const void* v_cache, int cache_dtype, const int* block_table,
                                     int max_pages, int page_size, const int* pos, const int* slot,
                                     void* out, int out_dtype, int T, int nq, int nkv, int hd,
                                     int window, float scale, int split_keys, int n_splits,
                                     float* scratch, cudaStream_t stream, const int* row_list = nullptr) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd % 16 || hd > 32 * MAX_DPL)
    return fail("paged_attention: head size %d is not a multiple of 16 up to %d", hd, 32 * MAX_DPL);
  if (nkv <= 0 || nq % nkv) return fail("paged_attention: %d query heads do not divide into %d kv heads", nq, nkv);
  if (n_splits < 1 || split_keys < 1) return fail("paged_attention: bad split (%d keys, %d splits)", split_keys, n_splits);
  if (n_splits > 1 && !scratch) return fail("paged_attention: splits need scratch memory");
  if (q_dtype != out_dtype) return fail("paged_attention: output type must equal the query type");
  const int G = nq / nkv;
  const int g_chunks = (G + GC - 1) / GC;
  const long long items = (long long)T * nkv * g_chunks * n_splits;
  const long long blocks = (items + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return fail("paged_attention: too many work items");
  const size_t smem = (size_t)WARPS * GC * hd * sizeof(float);
#define LAUNCH(TQ, TC)                                                                         \
  paged_attention_kernel<TQ, TC, TQ><<<(unsigned)blocks, WARPS * 32, smem, stream>>>(          \
      (const TQ*)q, (const TC*)k_cache, (const TC*)v_cache, block_table, max_pages, page_size, \
      pos, slot, (TQ*)out, scratch, T, nq, nkv, hd, window, scale, split_keys, n_splits, g_chunks, row_list)
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC, LAUNCH(TQ, TC)));
#undef LAUNCH
  int rc = check_launch("paged_attention");
  if (rc || n_splits == 1) return rc;
  const int threads = hd >= 128 ? 128 : 64;
  FLINT_DISPATCH_DTYPE(out_dtype, TO,
      (attention_combine_kernel<TO><<<(unsigned)((long long)T * nq), threads, 0, stream>>>(
          scratch, (TO*)out, hd, n_splits, nq, row_list)));
  return check_launch("attention_combine");
}



// ---------------------------------------------------------------------------------------------
// Block kernel for few rows over long contexts (decode).  One block of 128 threads per
// (split, kv head x chunk of 4 query heads, row).  Per chunk of 128 keys: thread t owns key t
// in the score phase (its K row is read with 16-byte loads, the 4 query heads share it), the
// block agrees on the new maximum and sum per head through shared memory, the probabilities
// are left in shared memory, and in the value phase thread t owns output dim t (and t+128):
// V rows are read coalesced across the block, unrolled for memory-level parallelism.
constexpr int BT = 128;        // threads per block = keys per chunk

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(BT)
paged_attention_block_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache,
                             const TC* __restrict__ v_cache, const int* __restrict__ block_table,
                             int max_pages, int page_size, const int* __restrict__ pos,
                             const int* __restrict__ slot, TO* __restrict__ out,
                             float* __restrict__ scratch, int nq, int nkv, int hd, int window,
                             float scale, int split_keys, int n_splits, int g_chunks,
                             const int* __restrict__ row_list) {
  extern __shared__ float smem[];
  float* qs = smem;                       // [GC][hd]
  float* ps = qs + GC * hd;               // [GC][BT] probabilities of the chunk
  float* red = ps + GC * BT;              // [GC][4] per-warp partials
  long long* rows = (long long*)(red + GC * 4 + 4);   // [BT] row index of each key (or -1)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / g_chunks, gchunk = blockIdx.y % g_chunks;
  const int ti = blockIdx.z;                        // index into the rows this launch covers
  const int t = row_list ? row_list[ti] : ti;       // row of the batch
  const int G = nq / nkv;
  const int g0 = gchunk * GC;
  const int ng = min(GC, G - g0);
  const int h0 = kvh * G + g0;
  const int p = pos[t];
  const int lo_row = window > 0 ? max(0, p + 1 - window) : 0;
  const int lo = lo_row + split * split_keys;
  const int hi = min(p + 1, lo + split_keys);
  const int* bt = block_table + (size_t)slot[t] * max_pages;

  for (int i = tid; i < ng * hd; i += BT) qs[i] = to_f32(q[((size_t)t * nq + h0) * hd + i]) * scale;
  __syncthreads();

  const int groups = hd / 8;             // 8-dim groups of a value row
  const int lanes = BT / groups;         // key lanes working side by side in the value phase
  const int dg = tid % groups, kl = tid / groups;
  float m[GC], l[GC], acc[GC][8];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }

  // score phase: 16 lanes share one key row; each lane keeps its 8 query dims of every head in registers
  float* ss = ps;                        // raw scores of the chunk share the probabilities' place
  const int khalf = lane >> 4, kq = lane & 15;
  float qreg[GC][8];
#pragma unroll
  for (int g = 0; g < GC; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) qreg[g][e] = (g < ng && kq * 8 < hd) ? qs[g * hd + kq * 8 + e] : 0.f;

  for (int j0 = lo; j0 < hi; j0 += BT) {
    const int j = j0 + tid;
    long long row = -1;
    if (j < hi) {
      const int page = bt[j / page_size];
      if (page >= 0) row = ((long long)page * nkv + kvh) * page_size + (j % page_size);
    }
    rows[tid] = row;
    __syncthreads();
    // a warp reads two whole key rows per instruction (16 lanes x 16 bytes each), four such loads in
    // flight; every lane gets partial dot products over its 8 dims and a butterfly over the 16 lanes
    // leaves the sum of head 2*bit3+bit2 in each lane.  Rows wider than 128 dims take more passes.
    constexpr int UK = 4;
#pragma unroll 1
    for (int k0 = warp * 2 + khalf; k0 < BT; k0 += 8 * UK) {
      float kf[UK][8];
      long long rr[UK];
#pragma unroll
      for (int u = 0; u < UK; ++u) {
        rr[u] = rows[k0 + 8 * u];
        if (rr[u] >= 0 && kq * 8 < hd) {
          load8<TC>(k_cache + rr[u] * hd + kq * 8, kf[u]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) kf[u][e] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < UK; ++u) {
        float s[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
          s[g] = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) s[g] = fmaf(qreg[g][e], kf[u][e], s[g]);
        }
        if (hd > 128 && rr[u] >= 0) {
          for (int d = kq * 8 + 128; d < hd; d += 128) {
            float k2[8];
            load8<TC>(k_cache + rr[u] * hd + d, k2);
#pragma unroll
            for (int g = 0; g < GC; ++g)
              if (g < ng) {
#pragma unroll
                for (int e = 0; e < 8; ++e) s[g] = fmaf(qs[g * hd + d + e], k2[e], s[g]);
              }
          }
        }
        const bool b3 = lane & 8, b2 = lane & 4;
        float a0 = b3 ? s[2] : s[0], a1 = b3 ? s[3] : s[1];
        const float x0 = b3 ? s[0] : s[2], x1 = b3 ? s[1] : s[3];
        a0 += __shfl_xor_sync(0xffffffffu, x0, 8);
        a1 += __shfl_xor_sync(0xffffffffu, x1, 8);
        float c = b2 ? a1 : a0;
        const float x2 = b2 ? a0 : a1;
        c += __shfl_xor_sync(0xffffffffu, x2, 4);
        c += __shfl_xor_sync(0xffffffffu, c, 2);
        c += __shfl_xor_sync(0xffffffffu, c, 1);
        if ((lane & 3) == 0) ss[((b3 ? 2 : 0) + (b2 ? 1 : 0)) * BT + k0 + 8 * u] = c;
      }
    }
    __syncthreads();
    float s[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) s[g] = ss[g * BT + tid];
    __syncthreads();      // ss is overwritten by the probabilities below
    // block maximum per head
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      const float v = warp_max(row >= 0 ? s[g] : -INFINITY);
      if (lane == 0) red[g * 4 + warp] = v;
    }
    __syncthreads();
    float alpha[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      const float mc = fmaxf(fmaxf(red[g * 4], red[g * 4 + 1]), fmaxf(red[g * 4 + 2], red[g * 4 + 3]));
      const float m_new = fmaxf(m[g], mc);
      const bool any = m_new > -INFINITY;
      alpha[g] = any ? expf(m[g] - m_new) : 1.f;
      const float pr = (any && row >= 0) ? expf(s[g] - m_new) : 0.f;
      ps[g * BT + tid] = pr;
      m[g] = m_new;
      s[g] = pr;
    }
    __syncthreads();      // red is read by all, ps written by all
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      const float v = warp_sum(s[g]);
      if (lane == 0) red[g * 4 + warp] = v;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      l[g] = l[g] * alpha[g] + (red[g * 4] + red[g * 4 + 1]) + (red[g * 4 + 2] + red[g * 4 + 3]);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= alpha[g];
    }
    // values: thread (dg, kl) owns 8 output dims (group dg) and the keys kl, kl + lanes, ...;
    // one 16-byte load per key, partial sums over key lanes are added up at the end
    const int nk = min(BT, hi - j0);
    if (kl < lanes) {
      constexpr int U = 4;      // rows in flight per thread
#pragma unroll 1
      for (int j1 = kl; j1 < nk; j1 += lanes * U) {
        float vv[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int jj = j1 + u * lanes;
          const long long r = jj < nk ? rows[jj] : -1;
          if (r >= 0) {
            load8<TC>(v_cache + r * hd + dg * 8, vv[u]);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) vv[u][e] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int jj = min(j1 + u * lanes, BT - 1);     // beyond nk the values are zero
#pragma unroll
          for (int g = 0; g < GC; ++g) {
            const float pj = ps[g * BT + jj];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj, vv[u][e], acc[g][e]);
          }
        }
      }
    }
    __syncthreads();      // ps, rows and red are rewritten by the next chunk
  }

  // add the key lanes' partial sums into osum [GC][hd], which reuses the query staging area
  float* osum = qs;
  __syncthreads();
  for (int i = tid; i < GC * hd; i += BT) osum[i] = 0.f;
  __syncthreads();
  for (int lane_k = 0; lane_k < lanes; ++lane_k) {      // fixed order: results do not depend on timing
    if (kl == lane_k) {
#pragma unroll
      for (int g = 0; g < GC; ++g)
        if (g < ng) {
#pragma unroll
          for (int e = 0; e < 8; ++e) osum[g * hd + dg * 8 + e] += acc[g][e];
        }
    }
    __syncthreads();
  }
  for (int g = 0; g < ng; ++g) {
    if (n_splits == 1) {
      const float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
      for (int d = tid; d < hd; d += BT) out[((size_t)t * nq + h0 + g) * hd + d] = from_f32<TO>(osum[g * hd + d] * inv);
    } else {
      float* dst = scratch + (((size_t)ti * nq + h0 + g) * n_splits + split) * (hd + 2);
      for (int d = tid; d < hd; d += BT) dst[d] = osum[g * hd + d];
      if (tid == 0) { dst[hd] = m[g]; dst[hd + 1] = l[g]; }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Warp-level tensor-core helpers (mma.sync m16n8k16, bf16 in, float32 out) for the decode
// kernel in attention_tc.cu.  A decoded token brings only nq/nkv (typically 4) query rows per
// key/value head, far below the 128 rows of a tcgen05 tile, and the float32-pipe kernels here
// are bound by instruction issue; the warp-level MMA with 16 rows (the group's heads, zero
// padded) cuts the instruction count per byte of cache about tenfold:
//   S = Q K^T    ldmatrix (K rows are already the "col" operand), 2 x hd/16 MMAs per 16 keys
//   softmax      on the accumulator fragment: 4 lanes share a row; float32 max, sum, exp
//   O += P V     P re-packed from the S fragment as the A operand, V through ldmatrix.trans
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same contract as paged_attention_launch, with the block kernel: for few rows and long key ranges.
inline int paged_attention_block_launch(const void* q, int q_dtype, const void* k_cache,
                                        const void* v_cache, int cache_dtype, const int* block_table,
                                        int max_pages, int page_size, const int* pos, const int* slot,
                                        void* out, int out_dtype, int T, int nq, int nkv, int hd,
                                        int window, float scale, int split_keys, int n_splits,
                                        float* scratch, cudaStream_t stream, const int* row_list = nullptr) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd % 16 || hd > 2 * BT)
    return fail("paged_attention: head size %d is not a multiple of 16 up to %d", hd, 2 * BT);
  if (nkv <= 0 || nq % nkv) return fail("paged_attention: %d query heads do not divide into %d kv heads", nq, nkv);
  if (n_splits < 1 || split_keys < 1) return fail("paged_attention: bad split (%d keys, %d splits)", split_keys, n_splits);
  if (n_splits > 1 && !scratch) return fail("paged_attention: splits need scratch memory");
  if (q_dtype != out_dtype) return fail("paged_attention: output type must equal the query type");
  const int G = nq / nkv;
  const int g_chunks = (G + GC - 1) / GC;
  if (T > 65535 || nkv * g_chunks > 65535) return fail("paged_attention: too many rows or heads for the block kernel");
  dim3 grid(n_splits, nkv * g_chunks, T);
  const size_t smem = (size_t)(GC * hd + GC * BT + GC * 4 + 4) * sizeof(float) + BT * sizeof(long long);
#define LAUNCH(TQ, TC)                                                                          \
  paged_attention_block_kernel<TQ, TC, TQ><<<grid, BT, smem, stream>>>(                         \
      (const TQ*)q, (const TC*)k_cache, (const TC*)v_cache, block_table, max_pages, page_size,  \
      pos, slot, (TQ*)out, scratch, nq, nkv, hd, window, scale, split_keys, n_splits, g_chunks, row_list)
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC, LAUNCH(TQ, TC)));
#undef LAUNCH
  int rc = check_launch("paged_attention (block kernel)");
  if (rc || n_splits == 1) return rc;
  const int threads = hd >= 128 ? 128 : 64;
  FLINT_DISPATCH_DTYPE(out_dtype, TO,
      (attention_combine_kernel<TO><<<(unsigned)((long long)T * nq), threads, 0, stream>>>(
          scratch, (TO*)out, hd, n_splits, nq, row_list)));
  return check_launch("attention_combine");
}

}  // namespace flint_attn
