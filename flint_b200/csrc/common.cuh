// Shared helpers of the sm_100a kernels: element types, loads that widen to float,
// stores that narrow from float, warp reductions and the error convention.
//
// Every exported function is extern "C", takes raw device pointers and a stream, does
// no allocation, and returns 0 or a negative code; the text of the last error is
// kept per thread and read with <module>_last_error().
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define FLINT_F32 0
#define FLINT_BF16 1

namespace flint {

// Gate and up weights of a gated feed-forward are kept paired: blocks of GATE_BLOCK gate rows alternate with
// the GATE_BLOCK up rows of the same features, and the feature count is padded to a multiple of GATE_BLOCK with
// zero rows.  Feature f has its gate row at paired_gate_row(f) and its up row GATE_BLOCK rows further.
constexpr int GATE_BLOCK = 16;
__host__ __device__ inline int paired_rows(int features) { return 2 * ((features + GATE_BLOCK - 1) / GATE_BLOCK) * GATE_BLOCK; }
__host__ __device__ inline int paired_gate_row(int f) { return (f / GATE_BLOCK) * 2 * GATE_BLOCK + f % GATE_BLOCK; }

static thread_local char g_error[512];

inline int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
inline int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return -1;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
  return 0;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl may begin (its blocks are
// scheduled, run their prologue, even fetch data that no earlier kernel writes) while the kernel
// before it in the stream is still finishing.  Every such kernel must call pdl_wait() before it
// reads anything an earlier kernel wrote and before it writes anything at all; pdl_launch() at its
// top lets the kernel after it start early in turn.  With FLINT_PDL=0 launches are ordinary and
// both calls do nothing.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FLINT_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);  // round to nearest even
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // smem32 may still be read from an earlier call
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float r = (lane < nwarps) ? smem32[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

}  // namespace flint

// Dispatch on a run-time element type code to a lambda templated on the C++ type.
#define FLINT_DISPATCH_DTYPE(code, T, ...)                        \
  do {                                                            \
    if ((code) == FLINT_F32) { using T = float; __VA_ARGS__; }    \
    else { using T = __nv_bfloat16; __VA_ARGS__; }                \
  } while (0)
