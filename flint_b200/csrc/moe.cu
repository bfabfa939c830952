// Routing for a top-2 mixture of experts: router logits and sparsemixer selection, and
// the plan that sorts token rows by expert for the grouped products.
//
// The reference has no mixture of experts (its feed-forward is dense:
// crates/thuban_model/src/ops/mlp.rs:24-79); these kernels have no counterpart there.
// Router logits, the mask threshold and both softmaxes are float32 in every mode.
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {
constexpr int MAX_E = 256;

// One block per TT tokens.  The tokens' rows are staged in shared memory; each warp takes
// experts warp, warp+16, ... and computes their logits for all TT tokens while reading the
// router row once with 16-byte loads; then one thread per token does the selection:
//   i1 = argmax s (lowest index on ties), m1 = s[i1]
//   keep_j = !((m1 - s_j) / max(|s_j|, m1) > 2 eps);  g1 = e^{s_i1 - m1} / sum_{keep} e^{s_j - m1}
//   the same again over s without i1 for (i2, g2); the gates are not renormalised.
constexpr int TT = 4;
constexpr int ROUTER_WARPS = 16;

template <typename TW> struct Vec;                       // 16 bytes of a weight row
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ void load_vec(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float* f) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename TW>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_sparsemixer_kernel(const float* __restrict__ x, const TW* __restrict__ wr, float eps,
                          int* __restrict__ expert_ids, float* __restrict__ gates,
                          float* __restrict__ logits_out, int T, int H, int E, int vec_ok) {
  extern __shared__ float smem[];   // TT rows of x, then TT x E logits
  float* xs = smem;
  float* s_all = smem + (size_t)TT * H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TT;
  const int nt = min(TT, T - t0);
  if (vec_ok) {        // rows are staged with 16-byte loads, several in flight per thread
    const int n4 = TT * H / 4, live4 = nt * H / 4;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)t0 * H);
    float4* dst = reinterpret_cast<float4*>(xs);
#pragma unroll 8
    for (int i = threadIdx.x; i < n4; i += blockDim.x)
      dst[i] = i < live4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    for (int i = threadIdx.x; i < TT * H; i += blockDim.x) xs[i] = i < nt * H ? x[(size_t)t0 * H + i] : 0.f;
  }
  __syncthreads();
  constexpr int VN = Vec<TW>::N;
  for (int e = warp; e < E; e += ROUTER_WARPS) {
    const TW* w = wr + (size_t)e * H;
    float a[TT];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) a[tt] = 0.f;
    if (vec_ok) {
#pragma unroll 4
      for (int d = lane * VN; d < H; d += 32 * VN) {
        float wv[VN];
        load_vec(w + d, wv);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          float xv[VN];                       // 16-byte reads of the staged row: no bank conflicts
#pragma unroll
          for (int i = 0; i < VN; i += 4) load_vec(xs + tt * H + d + i, xv + i);
#pragma unroll
          for (int i = 0; i < VN; ++i) a[tt] = fmaf(xv[i], wv[i], a[tt]);
        }
      }
    } else {
      for (int d = lane; d < H; d += 32) {
        const float wv = to_f32(w[d]);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) a[tt] = fmaf(xs[tt * H + d], wv, a[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const float v = warp_sum(a[tt]);
      if (lane == 0) s_all[tt * E + e] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x >= nt) return;
  const int t = t0 + threadIdx.x;
  const float* s = s_all + threadIdx.x * E;
  if (logits_out)
    for (int e = 0; e < E; ++e) logits_out[(size_t)t * E + e] = s[e];
  int sel[2];
  float gate[2];
  int excluded = -1;
  for (int r = 0; r < 2; ++r) {
    float m = -INFINITY;
    int im = 0;
    for (int e = 0; e < E; ++e)
      if (e != excluded && s[e] > m) { m = s[e]; im = e; }
    float denom = 0.f;
    for (int e = 0; e < E; ++e) {
      if (e == excluded) continue;
      const float factor = fmaxf(fabsf(s[e]), m);
      const bool masked = ((m - s[e]) / factor) > 2.0f * eps;
      if (!masked) denom += expf(s[e] - m);
    }
    sel[r] = im;
    gate[r] = 1.0f / denom;   // e^{m - m} / denom
    excluded = im;
  }
  expert_ids[2 * t] = sel[0];
  expert_ids[2 * t + 1] = sel[1];
  gates[2 * t] = gate[0];
  gates[2 * t + 1] = gate[1];
}

// One block.  expert_ids [T*2] -> per-expert counts, offsets (exclusive scan), the sorted row
// of every (token, choice) and the tile map for the grouped products.
__global__ void moe_plan_kernel(const int* __restrict__ expert_ids, int n_assign, int E,
                                int tile_rows, int* __restrict__ counts, int* __restrict__ offsets,
                                int* __restrict__ row_of, int* __restrict__ token_of,
                                int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                int* __restrict__ n_tiles, int max_tiles) {
  __shared__ int cnt[MAX_E];
  __shared__ int off[MAX_E + 1];
  pdl_launch();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  // rank of each assignment inside its expert (the order inside an expert has no effect on
  // any result: rows are independent in the products and are added back per token)
  for (int a = threadIdx.x; a < n_assign; a += blockDim.x) row_of[a] = atomicAdd(&cnt[expert_ids[a]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      counts[e] = cnt[e];
      offsets[e] = run;
      for (int r = 0; r < cnt[e]; r += tile_rows) {
        if (tiles < max_tiles) {
          tile_expert[tiles] = e;
          tile_row0[tiles] = run + r;
        }
        ++tiles;
      }
      run += cnt[e];
    }
    off[E] = run;
    offsets[E] = run;
    *n_tiles = tiles < max_tiles ? tiles : max_tiles;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < n_assign; a += blockDim.x) {
    const int row = off[expert_ids[a]] + row_of[a];
    row_of[a] = row;
    token_of[row] = a >> 1;
  }
}

// Few assignments (decode): the plan and the gather of the rows in one launch.  Every block works the
// (tiny) plan out again in shared memory, with ranks by position so that all blocks agree; block r then
// copies the row of its token to sorted row r, and block 0 also writes the plan out.
constexpr int DISPATCH_MAX = 256;      // assignments
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const int* __restrict__ expert_ids, int n_assign, int E, int tile_rows,
                    int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_of,
                    int* __restrict__ token_of, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                    int* __restrict__ n_tiles, int max_tiles, const uint4* __restrict__ x,
                    uint4* __restrict__ xs, int row_vecs) {
  __shared__ int ids[DISPATCH_MAX];
  __shared__ int cnt[MAX_E];
  __shared__ int off[MAX_E + 1];
  __shared__ int my_token;
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x;
  if (tid < n_assign) ids[tid] = expert_ids[tid];
  __syncthreads();
  if (tid < E) {
    int c = 0;
    for (int a = 0; a < n_assign; ++a) c += ids[a] == tid;
    cnt[tid] = c;
  }
  int rank = 0;                       // assignments before this one that chose the same expert
  if (tid < n_assign)
    for (int a = 0; a < tid; ++a) rank += ids[a] == ids[tid];
  __syncthreads();
  if (tid == 0) {
    const bool out = blockIdx.x == 0;
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      if (out) {
        counts[e] = cnt[e];
        offsets[e] = run;
        for (int r = 0; r < cnt[e]; r += tile_rows) {
          if (tiles < max_tiles) {
            tile_expert[tiles] = e;
            tile_row0[tiles] = run + r;
          }
          ++tiles;
        }
      }
      run += cnt[e];
    }
    off[E] = run;
    if (out) {
      offsets[E] = run;
      *n_tiles = tiles < max_tiles ? tiles : max_tiles;
    }
  }
  __syncthreads();
  if (tid < n_assign) {
    const int row = off[ids[tid]] + rank;
    if (blockIdx.x == 0) {
      row_of[tid] = row;
      token_of[row] = tid >> 1;
    }
    if (row == (int)blockIdx.x) my_token = tid >> 1;
  }
  __syncthreads();
  const uint4* src = x + (size_t)my_token * row_vecs;
  uint4* dst = xs + (size_t)blockIdx.x * row_vecs;
  for (int i = tid; i < row_vecs; i += blockDim.x) dst[i] = src[i];
}
}  // namespace

extern "C" int flint_router_sparsemixer(const float* x, const void* wr, int w_dtype, float eps,
                                        int* expert_ids, float* gates, float* logits_out, int T,
                                        int H, int E, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E < 2 || E > MAX_E) return fail("router: %d experts (supported: 2..%d)", E, MAX_E);
  const size_t smem = ((size_t)TT * H + (size_t)TT * E) * sizeof(float);
  if (smem > 200 * 1024) return fail("router: width %d is too large for the staging buffer", H);
  const int blocks = (T + TT - 1) / TT;
  // 16-byte loads of the router rows need rows that start on 16 bytes
  const int vec_ok = (H % 8 == 0) && (((uintptr_t)wr & 15) == 0);
  static bool configured[2] = {false, false};
  if (smem > 48 * 1024 && !configured[w_dtype ? 1 : 0]) {
    cudaError_t e = w_dtype == FLINT_F32
        ? cudaFuncSetAttribute(router_sparsemixer_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
        : cudaFuncSetAttribute(router_sparsemixer_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail("router: cannot raise shared memory: %s", cudaGetErrorString(e));
    configured[w_dtype ? 1 : 0] = true;
  }
  FLINT_DISPATCH_DTYPE(w_dtype, TW,
      (router_sparsemixer_kernel<TW><<<blocks, ROUTER_WARPS * 32, smem, stream>>>(
          x, (const TW*)wr, eps, expert_ids, gates, logits_out, T, H, E, vec_ok)));
  return check_launch("router_sparsemixer");
}

// Upper bound of row tiles for n_assign rows over E experts.
extern "C" int flint_moe_max_tiles(int n_assign, int E, int tile_rows) {
  return n_assign / tile_rows + (E < n_assign ? E : n_assign);
}

extern "C" int flint_moe_plan(const int* expert_ids, int n_assign, int E, int tile_rows, int* counts,
                              int* offsets, int* row_of, int* token_of, int* tile_expert,
                              int* tile_row0, int* n_tiles, int max_tiles, cudaStream_t stream) {
  if (n_assign <= 0) return 0;
  if (E < 1 || E > MAX_E) return fail("moe_plan: %d experts (supported: 1..%d)", E, MAX_E);
  if (tile_rows <= 0) return fail("moe_plan: bad tile size %d", tile_rows);
  if (max_tiles < flint_moe_max_tiles(n_assign, E, tile_rows))
    return fail("moe_plan: tile map of %d entries is too small", max_tiles);
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, expert_ids, n_assign, E, tile_rows, counts, offsets, row_of,
                                          token_of, tile_expert, tile_row0, n_tiles, max_tiles);
  return check_launch("moe_plan");
}

// The plan of flint_moe_plan and xs[r, :] = x[token_of[r], :] in one launch, for up to 256 assignments and rows
// of a multiple of 16 bytes (x and xs 16-byte aligned).
extern "C" int flint_moe_dispatch(const int* expert_ids, int n_assign, int E, int tile_rows, int* counts,
                                  int* offsets, int* row_of, int* token_of, int* tile_expert, int* tile_row0,
                                  int* n_tiles, int max_tiles, const void* x, void* xs, int row_bytes,
                                  cudaStream_t stream) {
  if (n_assign <= 0) return 0;
  if (n_assign > DISPATCH_MAX) return fail("moe_dispatch: %d assignments (up to %d)", n_assign, DISPATCH_MAX);
  if (E < 1 || E > MAX_E) return fail("moe_dispatch: %d experts (supported: 1..%d)", E, MAX_E);
  if (tile_rows <= 0) return fail("moe_dispatch: bad tile size %d", tile_rows);
  if (max_tiles < flint_moe_max_tiles(n_assign, E, tile_rows))
    return fail("moe_dispatch: tile map of %d entries is too small", max_tiles);
  if (row_bytes <= 0 || (row_bytes & 15) || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15))
    return fail("moe_dispatch: rows must be a multiple of 16 bytes and 16-byte aligned");
  launch_pdl(moe_dispatch_kernel, dim3(n_assign), dim3(256), 0, stream, expert_ids, n_assign, E, tile_rows, counts,
             offsets, row_of, token_of, tile_expert, tile_row0, n_tiles, max_tiles, (const uint4*)x, (uint4*)xs,
             row_bytes / 16);
  return check_launch("moe_dispatch");
}

extern "C" const char* flint_moe_last_error() { return g_error; }
