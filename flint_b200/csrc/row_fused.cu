// The row kernel of the residual stream: apply what earlier kernels left pending, normalise,
// and (optionally) route -- one block per row, or for a handful of rows a cluster of blocks per row, the row
// held in registers.
//
//   x[row] += sum_z partials[z][row] + bias          (a product whose K range was split)
//   x[row] += g0 * y[r0] + g1 * y[r1]                 (the two selected experts' outputs)
//   y = LayerNorm(x[row]) or RMSNorm(x[row])          float32 statistics, two passes over registers
//   out_f32 / out_bf16 <- y
//   logits_e = <y, Wr[e]>, sparsemixer top-2          (float32; same selection as moe.cu)
//
// Fusing these saves, per layer of a decode step, the kernels that would only add to the
// residual stream and one pass over it.  Widths that are not a multiple of 4 or exceed 16384
// are refused; the caller then uses the separate kernels.
// Reference counterparts: crates/thuban_kernel/wgsl/norm.wgsl (mode 3), add.wgsl, merge_gemm.wgsl.
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {
constexpr int MAX_VPT = 4;
constexpr int MAX_E = 256;

struct RowArgs {
  float* x;
  const int* row_index;
  const float* partials; int n_partials; long long partial_stride; const float* add_bias;
  const float* comb_y; const int* comb_row_of; const float* comb_gates;
  const float* gamma; const float* beta; float eps; int mode;
  float* out_f32; __nv_bfloat16* out_bf16;
  const void* wr; int E; float jitter_eps; int* expert_ids; float* gates;
  float* router_logits;        // optional [rows, E]: the logits the selection was made from (for tests)
  int H;
};

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void add4(float4& a, const float4 b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
__device__ __forceinline__ void fma4(float4& a, float g, const float4 b) {
  a.x = fmaf(g, b.x, a.x); a.y = fmaf(g, b.y, a.y); a.z = fmaf(g, b.z, a.z); a.w = fmaf(g, b.w, a.w);
}

__device__ __forceinline__ void load_w8(const float* p, float* f) {
  const float4 a = ld4(p), b = ld4(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load_w8(const __nv_bfloat16* p, float* f) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// sparsemixer top-2 of one row (float32; same selection as moe.cu).  Up to 32 experts sit one per lane of a
// warp (arg-max and the masked sums by shuffle).
__device__ __forceinline__ void select_two_by_lanes(float sv, int lane, int E, float jitter_eps, int* ids, float* gates) {
  int excluded = -1;
  for (int round = 0; round < 2; ++round) {
    // arg-max over lanes, lowest index on ties
    float m = (lane < E && lane != excluded) ? sv : -INFINITY;
    int im = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, im, o);
      if (om > m || (om == m && oi < im)) { m = om; im = oi; }
    }
    float term = 0.f;
    if (lane < E && lane != excluded) {
      const float factor = fmaxf(fabsf(sv), m);
      if (!(((m - sv) / factor) > 2.0f * jitter_eps)) term = expf(sv - m);
    }
    // the sum in lane order, so that it does not depend on the shuffle tree
    float denom = 0.f;
    for (int e = 0; e < E; ++e) denom += __shfl_sync(0xffffffffu, term, e);
    if (lane == 0) {
      ids[round] = im;
      gates[round] = 1.0f / denom;
    }
    excluded = im;
  }
}
// any number of experts, by one thread
__device__ __forceinline__ void select_two_serial(const float* s, int E, float jitter_eps, int* ids, float* gates) {
  int excluded = -1;
  for (int round = 0; round < 2; ++round) {
    float m = -INFINITY;
    int im = 0;
    for (int e = 0; e < E; ++e)
      if (e != excluded && s[e] > m) { m = s[e]; im = e; }
    float denom = 0.f;
    for (int e = 0; e < E; ++e) {
      if (e == excluded) continue;
      const float factor = fmaxf(fabsf(s[e]), m);
      if (!(((m - s[e]) / factor) > 2.0f * jitter_eps)) denom += expf(s[e] - m);
    }
    ids[round] = im;
    gates[round] = 1.0f / denom;
    excluded = im;
  }
}

// One block per row; a thread holds VPT vectors of four values of its row.
template <int VPT, typename TW>
__global__ void __launch_bounds__(1024)
row_norm_kernel(const __grid_constant__ RowArgs a) {
  extern __shared__ float smem[];          // router only: H floats of the normalised row, then partial logits
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int H = a.H, n4 = H >> 2;
  {
    const int r = blockIdx.x;
    const int src = a.row_index ? a.row_index[r] : r;
    float* xr = a.x + (size_t)src * H;
    float4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      v[i] = c < n4 ? ld4(xr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const bool pending = a.partials || a.comb_y;
    if (a.partials) {
      const float* pr = a.partials + (size_t)src * H;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) {
          for (int z0 = 0; z0 < a.n_partials; z0 += 4) {      // four loads in flight, added in a fixed order
            float4 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
              t[u] = z0 + u < a.n_partials ? ld4(pr + (size_t)(z0 + u) * a.partial_stride + 4 * c)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 4; ++u) add4(v[i], t[u]);
          }
        }
      }
      if (a.add_bias) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int c = threadIdx.x + i * blockDim.x;
          if (c < n4) add4(v[i], ld4(a.add_bias + 4 * c));
        }
      }
    }
    if (a.comb_y) {
      const int r0 = a.comb_row_of[2 * src], r1 = a.comb_row_of[2 * src + 1];
      const float g0 = a.comb_gates[2 * src], g1 = a.comb_gates[2 * src + 1];
      const float* y0 = a.comb_y + (size_t)r0 * H;
      const float* y1 = a.comb_y + (size_t)r1 * H;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) {
          float4 t = make_float4(0.f, 0.f, 0.f, 0.f);   // g0*y0 + g1*y1 first, then added: the order of moe_combine
          fma4(t, g0, ld4(y0 + 4 * c));
          fma4(t, g1, ld4(y1 + 4 * c));
          add4(v[i], t);
        }
      }
    }
    if (pending) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) *reinterpret_cast<float4*>(xr + 4 * c) = v[i];
      }
    }
    if (!a.gamma) return;                     // only the additions were wanted
    // statistics
    float mean = 0.f;
    if (a.mode == 0) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);   // zeros beyond the row
      mean = block_sum(s, red) / (float)H;
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < n4) {
        const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
        ss += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)H + a.eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < n4) {
        const float4 g = ld4(a.gamma + 4 * c);
        float4 y = make_float4((v[i].x - mean) * inv * g.x, (v[i].y - mean) * inv * g.y,
                               (v[i].z - mean) * inv * g.z, (v[i].w - mean) * inv * g.w);
        if (a.beta) add4(y, ld4(a.beta + 4 * c));
        if (a.out_f32) *reinterpret_cast<float4*>(a.out_f32 + (size_t)r * H + 4 * c) = y;
        if (a.out_bf16) {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
          uint2 pk;
          pk.x = *reinterpret_cast<const uint32_t*>(&lo);
          pk.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(a.out_bf16 + (size_t)r * H + 4 * c) = pk;
        }
        if (a.wr) *reinterpret_cast<float4*>(smem + 4 * c) = y;
      }
    }
  }
  if (!a.wr) return;
  // ---- router: a job is (group of 4 experts, strided share of the row); a warp keeps 4 sums, so that
  // every value read from shared memory feeds 4 multiply-adds; partial sums meet in shared memory
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int E = a.E;
  constexpr int EG = 4;
  const int groups = (E + EG - 1) / EG;
  const int k = n_warps >= groups ? n_warps / groups : 1;   // warps per expert group
  float* part = smem + H;                                    // [E][k]
  const TW* wr = (const TW*)a.wr;
  const bool vec = (H & 7) == 0;
  for (int job = warp; job < groups * k; job += n_warps) {
    const int e0 = (job / k) * EG, sl = job % k;
    float acc[EG];
#pragma unroll
    for (int j = 0; j < EG; ++j) acc[j] = 0.f;
    if (vec) {
#pragma unroll 2
      for (int d = (sl * 32 + lane) * 8; d < H; d += k * 256) {
        float wv[EG][8];
#pragma unroll
        for (int j = 0; j < EG; ++j) {
          if (e0 + j < E) {
            load_w8(wr + (size_t)(e0 + j) * H + d, wv[j]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) wv[j][i] = 0.f;
          }
        }
        const float4 x0 = ld4(smem + d), x1 = ld4(smem + d + 4);
        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int j = 0; j < EG; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j] = fmaf(xv[i], wv[j][i], acc[j]);
      }
    } else {
      for (int d = sl * 32 + lane; d < H; d += k * 32) {
        const float xv = smem[d];
#pragma unroll
        for (int j = 0; j < EG; ++j)
          acc[j] = fmaf(xv, e0 + j < E ? to_f32(wr[(size_t)(e0 + j) * H + d]) : 0.f, acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < EG; ++j) {
      const float t = warp_sum(acc[j]);
      if (lane == 0 && e0 + j < E) part[(e0 + j) * k + sl] = t;
    }
  }
  __syncthreads();
  // selection by the first warp.  Up to 32 experts sit one per lane (argmax and the masked sums by
  // shuffle); more experts are handled by lane 0 alone.
  if (warp != 0) return;
  const int r = blockIdx.x;
  if (E <= 32) {
    float sv = -INFINITY;
    if (lane < E) {
      sv = 0.f;
      for (int i = 0; i < k; ++i) sv += part[lane * k + i];    // fixed order
      if (a.router_logits) a.router_logits[(size_t)r * E + lane] = sv;
    }
    select_two_by_lanes(sv, lane, E, a.jitter_eps, a.expert_ids + 2 * r, a.gates + 2 * r);
    return;
  }
  if (lane != 0) return;
  float* s = smem;                                         // the row is no longer needed
  for (int e = 0; e < E; ++e) {
    float t = 0.f;
    for (int i = 0; i < k; ++i) t += part[e * k + i];    // fixed order
    s[e] = t;
    if (a.router_logits) a.router_logits[(size_t)r * E + e] = t;
  }
  select_two_serial(s, E, a.jitter_eps, a.expert_ids + 2 * r, a.gates + 2 * r);
}

// ---- few rows: a cluster of blocks per row
// With a handful of rows (a decode step) one block per row leaves the device empty and pulls the whole row,
// its pending partial sums and the router's weights through one SM.  Here the blocks of a cluster share a
// row: each takes a run of columns, the statistics and the router's partial sums meet through distributed
// shared memory (every block writes its share into the others' memory, one cluster barrier, then every block
// adds the shares in rank order, so all of them hold the same bits), and block 0 selects the experts.
constexpr int MAX_CL = 8;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_blocks() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// every thread of every block of the cluster; what was stored before it is visible after it
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// store into the same shared-memory place of another block of the cluster
__device__ __forceinline__ void store_to_block(float* local, uint32_t rank, float v) {
  const uint32_t la = (uint32_t)__cvta_generic_to_shared(local);
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}
// the sum of one value per block; slots: MAX_CL floats of this block that nothing else uses
__device__ __forceinline__ float cluster_sum(float block_value, float* slots, uint32_t rank, uint32_t n) {
  if (threadIdx.x < n) store_to_block(slots + rank, threadIdx.x, block_value);
  __syncwarp();
  cluster_barrier();
  float t = 0.f;
  for (uint32_t i = 0; i < n; ++i) t += slots[i];
  return t;
}

template <int VPT, typename TW>
__global__ void __launch_bounds__(256)
row_norm_cluster_kernel(const __grid_constant__ RowArgs a, const int vec_per_block) {
  extern __shared__ float smem[];          // router only: this block's columns of the normalised row, partial logits
  __shared__ float red[32];
  __shared__ float sum_slots[MAX_CL], sq_slots[MAX_CL];
  const uint32_t rank = cluster_rank(), CL = cluster_blocks();
  const int H = a.H, n4 = H >> 2;
  const int r = blockIdx.x / CL;
  const int c0 = rank * vec_per_block;     // first vector of four columns of this block
  int col[VPT];
  bool ok[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int l = threadIdx.x + i * blockDim.x;
    col[i] = c0 + l;
    ok[i] = l < vec_per_block && col[i] < n4;
  }
  // scale and shift are weights, which no kernel writes: they are fetched while the kernel before still runs
  float4 g[VPT], b[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    g[i] = (a.gamma && ok[i]) ? ld4(a.gamma + 4 * col[i]) : make_float4(0.f, 0.f, 0.f, 0.f);
    b[i] = (a.gamma && a.beta && ok[i]) ? ld4(a.beta + 4 * col[i]) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_launch();
  cluster_barrier();        // every block of the cluster runs before any of them writes into another's memory
  pdl_wait();
  const int src = a.row_index ? a.row_index[r] : r;
  float* xr = a.x + (size_t)src * H;
  float4 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) v[i] = ok[i] ? ld4(xr + 4 * col[i]) : make_float4(0.f, 0.f, 0.f, 0.f);
  const bool pending = a.partials || a.comb_y;
  if (a.partials) {
    const float* pr = a.partials + (size_t)src * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (ok[i]) {
        for (int z0 = 0; z0 < a.n_partials; z0 += 8) {      // eight loads in flight, added in a fixed order
          float4 t[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            t[u] = z0 + u < a.n_partials ? ld4(pr + (size_t)(z0 + u) * a.partial_stride + 4 * col[i])
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < 8; ++u) add4(v[i], t[u]);
        }
        if (a.add_bias) add4(v[i], ld4(a.add_bias + 4 * col[i]));
      }
    }
  }
  if (a.comb_y) {
    const int r0 = a.comb_row_of[2 * src], r1 = a.comb_row_of[2 * src + 1];
    const float g0 = a.comb_gates[2 * src], g1 = a.comb_gates[2 * src + 1];
    const float* y0 = a.comb_y + (size_t)r0 * H;
    const float* y1 = a.comb_y + (size_t)r1 * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (ok[i]) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);   // g0*y0 + g1*y1 first, then added: the order of moe_combine
        fma4(t, g0, ld4(y0 + 4 * col[i]));
        fma4(t, g1, ld4(y1 + 4 * col[i]));
        add4(v[i], t);
      }
    }
  }
  if (pending) {
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (ok[i]) *reinterpret_cast<float4*>(xr + 4 * col[i]) = v[i];
  }
  if (!a.gamma) return;                     // only the additions were wanted (the same for every block)
  float mean = 0.f;
  if (a.mode == 0) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);   // zeros outside the block's columns
    mean = cluster_sum(block_sum(s, red), sum_slots, rank, CL) / (float)H;
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (ok[i]) {
      const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
      ss += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  const float inv = 1.0f / sqrtf(cluster_sum(block_sum(ss, red), sq_slots, rank, CL) / (float)H + a.eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (ok[i]) {
      const int c = col[i];
      float4 y = make_float4((v[i].x - mean) * inv * g[i].x, (v[i].y - mean) * inv * g[i].y,
                             (v[i].z - mean) * inv * g[i].z, (v[i].w - mean) * inv * g[i].w);
      if (a.beta) add4(y, b[i]);
      if (a.out_f32) *reinterpret_cast<float4*>(a.out_f32 + (size_t)r * H + 4 * c) = y;
      if (a.out_bf16) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(a.out_bf16 + (size_t)r * H + 4 * c) = pk;
      }
      if (a.wr) *reinterpret_cast<float4*>(smem + 4 * (c - c0)) = y;
    }
  }
  if (!a.wr) return;
  // ---- router over this block's columns: a job is (group of 4 experts, strided share of the columns)
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int E = a.E;
  constexpr int EG = 4;
  const int groups = (E + EG - 1) / EG;
  const int k = n_warps >= groups ? n_warps / groups : 1;   // warps per expert group
  const int cols = 4 * vec_per_block;
  const int first = 4 * c0;
  const int n_valid = max(0, min(cols, H - first));          // columns of the row that this block holds
  float* part = smem + cols;                                  // [E][k]
  float* logit_slots = part + E * k;                          // [CL][E], filled in block 0 by every block
  float* s = logit_slots + MAX_CL * E;                        // [E], for more than 32 experts
  const TW* wr = (const TW*)a.wr + first;
  const bool vec = (H & 7) == 0 && (first & 7) == 0;
  for (int job = warp; job < groups * k; job += n_warps) {
    const int e0 = (job / k) * EG, sl = job % k;
    float acc[EG];
#pragma unroll
    for (int j = 0; j < EG; ++j) acc[j] = 0.f;
    if (vec) {
#pragma unroll 2
      for (int d = (sl * 32 + lane) * 8; d < n_valid; d += k * 256) {
        float wv[EG][8];
#pragma unroll
        for (int j = 0; j < EG; ++j) {
          if (e0 + j < E) {
            load_w8(wr + (size_t)(e0 + j) * H + d, wv[j]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) wv[j][i] = 0.f;
          }
        }
        const float4 x0 = ld4(smem + d), x1 = ld4(smem + d + 4);
        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int j = 0; j < EG; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j] = fmaf(xv[i], wv[j][i], acc[j]);
      }
    } else {
      for (int d = sl * 32 + lane; d < n_valid; d += k * 32) {
        const float xv = smem[d];
#pragma unroll
        for (int j = 0; j < EG; ++j)
          acc[j] = fmaf(xv, e0 + j < E ? to_f32(wr[(size_t)(e0 + j) * H + d]) : 0.f, acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < EG; ++j) {
      const float t = warp_sum(acc[j]);
      if (lane == 0 && e0 + j < E) part[(e0 + j) * k + sl] = t;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float t = 0.f;
    for (int i = 0; i < k; ++i) t += part[e * k + i];      // fixed order
    store_to_block(logit_slots + rank * E + e, 0, t);
  }
  __syncwarp();
  cluster_barrier();
  if (rank != 0 || warp != 0) return;
  if (E <= 32) {
    float sv = -INFINITY;
    if (lane < E) {
      sv = 0.f;
      for (uint32_t q = 0; q < CL; ++q) sv += logit_slots[q * E + lane];    // fixed order
      if (a.router_logits) a.router_logits[(size_t)r * E + lane] = sv;
    }
    select_two_by_lanes(sv, lane, E, a.jitter_eps, a.expert_ids + 2 * r, a.gates + 2 * r);
    return;
  }
  if (lane != 0) return;
  for (int e = 0; e < E; ++e) {
    float t = 0.f;
    for (uint32_t q = 0; q < CL; ++q) t += logit_slots[q * E + e];
    s[e] = t;
    if (a.router_logits) a.router_logits[(size_t)r * E + e] = t;
  }
  select_two_serial(s, E, a.jitter_eps, a.expert_ids + 2 * r, a.gates + 2 * r);
}

template <int VPT, typename TW>
int launch_row(const RowArgs& a, int rows, int threads, size_t smem, cudaStream_t stream) {
  if (smem > 48 * 1024) {
    static bool configured = false;   // per instantiation
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(row_norm_kernel<VPT, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024);
      if (e != cudaSuccess) return fail("row_norm: cannot raise shared memory: %s", cudaGetErrorString(e));
      configured = true;
    }
  }
  launch_pdl(row_norm_kernel<VPT, TW>, dim3(rows), dim3(threads), smem, stream, a);
  return check_launch("row_norm");
}

template <int VPT, typename TW>
int launch_row_cluster(const RowArgs& a, int rows, int cl, int vec_per_block, int threads, size_t smem, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows * cl);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cl;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaLaunchKernelEx(&cfg, row_norm_cluster_kernel<VPT, TW>, a, vec_per_block);
  return check_launch("row_norm (cluster)");
}

int g_cluster_rows = 16;      // up to this many rows a cluster of blocks shares each row; 0: never
}  // namespace

// For measurements and tests: the largest number of rows that run with a cluster of blocks per row (0: none).
extern "C" int flint_row_norm_set_cluster_rows(int rows) {
  g_cluster_rows = rows < 0 ? 0 : rows;
  return 0;
}

// x [T, H] float32 residual stream, updated in place if anything is pending.
// rows: number of output rows (T, or the length of row_index if given; then x rows are gathered).
// pending: partials [n_partials][T][H] (stride partial_stride floats) + add_bias [H]; and/or
//          comb_y [2T, H] with comb_row_of [T, 2] and comb_gates [T, 2].
// gamma NULL: only apply the pending additions.  wr != NULL (router weights [E, H], bf16 or f32):
// also fill expert_ids [rows, 2] and gates [rows, 2] (and router_logits [rows, E] if given); then row_index
// must be NULL.
extern "C" int flint_row_norm(float* x, const int* row_index, int rows, int H, const float* partials,
                              int n_partials, long long partial_stride, const float* add_bias,
                              const float* comb_y, const int* comb_row_of, const float* comb_gates,
                              const float* gamma, const float* beta, float eps, int mode, float* out_f32,
                              void* out_bf16, const void* wr, int w_dtype, int E, float jitter_eps,
                              int* expert_ids, float* gates, float* router_logits, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || (H & 3) || H > 4 * 1024 * MAX_VPT) return fail("row_norm: width %d (multiples of 4 up to %d)", H, 4096 * MAX_VPT);
  if (gamma && !out_f32 && !out_bf16 && !wr) return fail("row_norm: no output given");
  if (mode != 0 && mode != 1) return fail("row_norm: unknown mode %d", mode);
  if (wr && (E < 2 || E > MAX_E)) return fail("row_norm: %d experts (2..%d)", E, MAX_E);
  if (wr && (row_index || !gamma || !expert_ids || !gates)) return fail("row_norm: the router needs a norm and all rows");
  if (wr && (((uintptr_t)wr & 15) != 0)) return fail("row_norm: router weights must be 16-byte aligned");
  RowArgs a;
  a.x = x; a.row_index = row_index;
  a.partials = partials; a.n_partials = n_partials; a.partial_stride = partial_stride; a.add_bias = add_bias;
  a.comb_y = comb_y; a.comb_row_of = comb_row_of; a.comb_gates = comb_gates;
  a.gamma = gamma; a.beta = beta; a.eps = eps; a.mode = mode;
  a.out_f32 = out_f32; a.out_bf16 = (__nv_bfloat16*)out_bf16;
  a.wr = wr; a.E = E; a.jitter_eps = jitter_eps; a.expert_ids = expert_ids; a.gates = gates;
  a.router_logits = wr ? router_logits : nullptr;
  a.H = H;
  const int n4 = H / 4;
  // a handful of rows: a cluster of blocks per row
  // (measured on a decode step of rows of 4,096: 1, 8 and 16 rows gain 3.7, 1.8 and 1.0 % of the step; 32 rows
  // lose 1.2 %, also with clusters of four: with that many blocks the barriers cost more than the blocks gain)
  const int cl = n4 >= 512 ? 8 : (n4 >= 256 ? 4 : (n4 >= 128 ? 2 : 1));
  if (cl > 1 && rows <= g_cluster_rows) {
    const int vec_per_block = (((n4 + cl - 1) / cl) + 1) & ~1;       // even: a block's columns start on 32 bytes
    int threads = ((vec_per_block + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    const int vpt = (vec_per_block + threads - 1) / threads;
    const int n_warps = threads / 32;
    const int groups = (E + 3) / 4;
    const int k = wr ? (n_warps >= groups ? n_warps / groups : 1) : 0;
    const size_t smem = wr ? (size_t)(4 * vec_per_block + E * k + MAX_CL * E + E) * sizeof(float) : 0;
    if (smem <= 48 * 1024 && vpt <= MAX_VPT) {
#define GOC(V) (wr && w_dtype == FLINT_BF16 ? launch_row_cluster<V, __nv_bfloat16>(a, rows, cl, vec_per_block, threads, smem, stream) \
                                            : launch_row_cluster<V, float>(a, rows, cl, vec_per_block, threads, smem, stream))
      switch (vpt) {
        case 1: return GOC(1);
        case 2: return GOC(2);
        default: return GOC(4);
      }
#undef GOC
    }
  }
  // few rows: a wide block per row (more warps share the router's rows); many rows: narrow blocks
  // with four vectors per thread, so that several blocks fit an SM and hide each other's latency
  int threads = rows < 148 ? ((n4 + 31) / 32) * 32 : ((n4 / 4 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  if (wr && threads < 128) threads = 128;               // a few warps for the router's dot products
  const int vpt = (n4 + threads - 1) / threads;
  const int n_warps = threads / 32;
  const int groups = (E + 3) / 4;
  const int k = wr ? (n_warps >= groups ? n_warps / groups : 1) : 0;
  const size_t smem = wr ? (size_t)(H + E * k) * sizeof(float) : 0;
#define GO(V) (wr && w_dtype == FLINT_BF16 ? launch_row<V, __nv_bfloat16>(a, rows, threads, smem, stream) \
                                           : launch_row<V, float>(a, rows, threads, smem, stream))
  if (smem > 200 * 1024) return fail("row_norm: width %d is too large for the fused router", H);
  switch (vpt) {
    case 1: return GO(1);
    case 2: return GO(2);
    case 3: case 4: return GO(4);
    default: return fail("row_norm: width %d is too large", H);
  }
#undef GO
}

extern "C" const char* flint_row_fused_last_error() { return g_error; }
