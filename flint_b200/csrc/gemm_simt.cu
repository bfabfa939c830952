// General matrix products on the ordinary float32 pipes: y[m,n] = sum_k x[m,k] * W[n,k].
//
// This is the true 32-bit path (plain FFMA, no tensor cores, no reduced-precision mode)
// and the path for shapes that the tensor-core kernel refuses.  Inputs may be float32
// or bfloat16 (widened on load), the accumulator is float32.  It takes any M, N, K.
// One kernel serves four uses:
//   dense            out = x W^T (+ bias) (+ out if accumulate)
//   dense, gated     out = act(x W^T) * (x W_up^T)
//   grouped          rows are sorted by expert; a tile map names each row tile's expert
//   grouped, gated   both
// Reference counterparts: crates/thuban_kernel/wgsl/gemm.wgsl (64x128x32 tiles, ACC=1 for
// the residual add), bias.wgsl, swiglu.wgsl.
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {
constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

__device__ __forceinline__ float act_fn(float g, int act) {
  if (act == 0) return g / (1.0f + expf(-g));                       // silu
  return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

template <typename TX, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TX* __restrict__ x, int ldx, const TW* __restrict__ w, const float* __restrict__ bias,
                 TO* __restrict__ out, int ldo, int accumulate, int act,
                 const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                 const int* __restrict__ n_tiles, const int* __restrict__ offsets, int tile_rows,
                 long long expert_stride, int M, int N, int K) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  __shared__ float us[GATED ? BK : 1][BN + 4];

  int expert = 0, row0 = blockIdx.y * BM, row_end = M;
  if (tile_expert) {
    if ((int)blockIdx.y >= *n_tiles) return;
    expert = tile_expert[blockIdx.y];
    row0 = tile_row0[blockIdx.y];
    row_end = min(offsets[expert + 1], row0 + tile_rows);
  }
  const int col0 = blockIdx.x * BN;
  const TW* we = w + (size_t)expert * expert_stride;

  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4] = {}, acc_u[GATED ? 4 : 1][4] = {};

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread; k runs fastest in memory
    for (int i = threadIdx.x; i < BM * BK; i += THREADS) {
      const int r = i / BK, k = i % BK;
      const int gr = row0 + r, gk = k0 + k;
      xs[k][r] = (gr < row_end && gk < K) ? to_f32(x[(size_t)gr * ldx + gk]) : 0.f;
      const int gc = col0 + r;
      const bool ok = gc < N && gk < K;
      const size_t wr = GATED ? paired_gate_row(gc) : gc;      // gated: the up row lies GATE_BLOCK rows further
      ws[k][r] = ok ? to_f32(we[wr * K + gk]) : 0.f;
      if (GATED) us[k][r] = ok ? to_f32(we[(wr + GATE_BLOCK) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
      if (GATED) {
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = us[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acc_u[i][j] = fmaf(a[i], u[j], acc_u[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tx * 4 + j;
      if (gc >= N) continue;
      float v = acc[i][j];
      if (GATED) v = act_fn(v, act) * acc_u[i][j];
      if (bias) v += bias[gc];
      const size_t o = (size_t)gr * ldo + gc;
      if (accumulate) v += to_f32(out[o]);
      out[o] = from_f32<TO>(v);
    }
  }
}
}  // namespace

// x [rows, K] (row stride ldx), w [E, N, K] (gated: [E, paired_rows(N), K], gate and up rows paired in blocks),
// out [rows, N].
// Dense: tile_expert == NULL, rows = M, one "expert".  Grouped: rows of expert e are
// offsets[e] .. offsets[e+1]-1, and tile i covers up to tile_rows (<= 64) rows from tile_row0[i] of
// expert tile_expert[i]; only the first *n_tiles tiles exist (max_tiles bounds the grid).
extern "C" int flint_gemm_simt(const void* x, int x_dtype, int ldx, const void* w, int gated,
                               int w_dtype, const float* bias, void* out, int out_dtype, int ldo,
                               int accumulate, int act, const int* tile_expert,
                               const int* tile_row0, const int* n_tiles, const int* offsets,
                               int max_tiles, int tile_rows, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return fail("gemm_simt: K=%d", K);
  const long long expert_stride = (long long)(gated ? paired_rows(N) : N) * K;
  if (gated && accumulate) return fail("gemm_simt: a gated product cannot accumulate");
  if (tile_expert && (tile_rows < 1 || tile_rows > BM)) return fail("gemm_simt: row tiles of %d rows (1..%d)", tile_rows, BM);
  const int tiles_m = tile_expert ? max_tiles : (M + BM - 1) / BM;
  if (tiles_m <= 0) return 0;
  if (tiles_m > 65535) return fail("gemm_simt: %d row tiles exceed the grid limit", tiles_m);
  dim3 grid((N + BN - 1) / BN, tiles_m);
#define LAUNCH(TX, TW, TO)                                                                        \
  do {                                                                                            \
    if (gated)                                                                                    \
      gemm_simt_kernel<TX, TW, TO, true><<<grid, THREADS, 0, stream>>>(                           \
          (const TX*)x, ldx, (const TW*)w, bias, (TO*)out, ldo, accumulate, act,                  \
          tile_expert, tile_row0, n_tiles, offsets, tile_rows, expert_stride, M, N, K);                                     \
    else                                                                                          \
      gemm_simt_kernel<TX, TW, TO, false><<<grid, THREADS, 0, stream>>>(                          \
          (const TX*)x, ldx, (const TW*)w, bias, (TO*)out, ldo, accumulate, act,                  \
          tile_expert, tile_row0, n_tiles, offsets, tile_rows, expert_stride, M, N, K);                                     \
  } while (0)
  FLINT_DISPATCH_DTYPE(x_dtype, TX, FLINT_DISPATCH_DTYPE(w_dtype, TW,
      FLINT_DISPATCH_DTYPE(out_dtype, TO, LAUNCH(TX, TW, TO))));
#undef LAUNCH
  return check_launch("gemm_simt");
}

extern "C" const char* flint_gemm_simt_last_error() { return g_error; }
