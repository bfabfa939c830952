// Prefill attention on the tcgen05 tensor cores, over the paged bfloat16 cache.
//
// One block per (tile of up to 128 consecutive query rows of one request, query head).  The keys
// of the request are walked in tiles of 64, always read from the cache pages (so a portion of a
// prompt sees the keys of earlier portions as well as its own):
//   S = Q K^T        tcgen05.mma, Q [128, hd] and K [64, hd] both K-major in shared memory, S in
//                    tensor memory (128 lanes = query rows, 64 columns = keys)
//   softmax          one thread per query row reads its row of S with tcgen05.ld, applies scale,
//                    the causal and window mask, keeps the running maximum and sum in float32,
//                    and writes P = exp2(..) as bfloat16 into shared memory (K-major, swizzled)
//   O_tile = P V     tcgen05.mma with V [64 keys, hd] as an MN-major B operand, fresh accumulator;
//                    the row's thread then folds it into its float32 output registers:
//                    o = o * alpha + O_tile
// Q, K and V tiles come by TMA (128-byte swizzle, no multicast); K/V tiles are double-buffered.
// Roles (192 threads): warp 0 lane 0 loads, warp 1 owns tensor memory and its lane 0 issues MMAs,
// warps 2..5 are the 128 softmax rows.  Every mbarrier wait is bounded; on a timeout the block
// sets the error flag, frees its tensor memory and returns.
//
// Sizes: head sizes in steps of 16 up to 128, any head counts, page sizes that divide 64 or are
// multiples of 64.  Other shapes are refused and run on the float32-pipe kernel.
//
// Reference counterpart: crates/thuban_kernel/wgsl/attn.wgsl (8 query rows x 128 keys per
// workgroup, subgroup reductions, no tensor cores).
#include <math.h>
#include <stdarg.h>

#include "common.cuh"
#include "tc_common.cuh"

using namespace flint;
using namespace flint_tc;

namespace {

constexpr int BQ = 128;      // query rows per block
constexpr int BKV = 64;      // keys per tile
constexpr int THREADS = 192;
constexpr int STAGES = 2;

struct Params {
  const int* tiles;          // [n_tiles, 4]: first row, rows, slot, position of the first row
  const int* block_table;
  __nv_bfloat16* out;
  int* error_flag;
  int max_pages, page_size, nq, nkv, hd, window;
  float scale_log2;          // scale * log2(e)
};

__device__ __forceinline__ uint32_t idesc_f16(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(BQ >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int HDM>   // HDM: 64 or 128, the largest head size this instantiation holds in registers
__global__ void __launch_bounds__(THREADS)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[8];   // q, kv_full[2], kv_empty[2], s_full, p_full, o_full
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  if (*(volatile int*)p.error_flag) return;
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int row0 = tile[0], n_rows = tile[1], slot = tile[2], pos0 = tile[3];
  const int head = blockIdx.y;
  const int hd = p.hd;
  const int kvh = head / (p.nq / p.nkv);
  const int chunks = (hd + 63) / 64;
  const int P = p.page_size;
  const int piece = P < BKV ? P : BKV;        // rows of one TMA load of keys
  const int pieces = BKV / piece;

  // keys this tile of queries can see: [k_lo, k_hi)
  const int k_hi = pos0 + n_rows;
  const int k_lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;
  const int tile_lo = k_lo / BKV;
  const int n_kv_tiles = (k_hi + BKV - 1) / BKV - tile_lo;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;                                       // chunks x [128 rows][128 B]
  const uint32_t kv_smem = q_smem + chunks * BQ * 128;                // per stage: K chunks, then V chunks
  const uint32_t kv_stage_bytes = 2u * chunks * BKV * 128;
  const uint32_t p_smem = kv_smem + STAGES * kv_stage_bytes;          // [128 rows][128 B]
  const uint32_t bar_q = smem_u32(&bars[0]), bar_full0 = smem_u32(&bars[1]), bar_empty0 = smem_u32(&bars[3]);
  const uint32_t bar_s = smem_u32(&bars[5]), bar_p = smem_u32(&bars[6]), bar_o = smem_u32(&bars[7]);
  const uint32_t tmem_cols = HDM <= 64 ? 128 : 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full0 + 8 * s, 1);
      mbar_init(bar_empty0 + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, BQ);       // every softmax row arrives itself
    mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  const uint32_t tmem_s = tmem, tmem_o = tmem + BKV;
  volatile int* ab = &abort_flag;

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- loads
    mbar_expect_tx(bar_q, chunks * BQ * 128);
    for (int c = 0; c < chunks; ++c) tma_load_2d(q_smem + c * BQ * 128, &map_q, head * hd + c * 64, row0, bar_q);
    const int* bt = p.block_table + (size_t)slot * p.max_pages;
    for (int i = 0; i < n_kv_tiles; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(bar_empty0 + 8 * s, ((i / STAGES) & 1) ^ 1, ab)) break;
      const uint32_t bar = bar_full0 + 8 * s;
      mbar_expect_tx(bar, kv_stage_bytes);
      const uint32_t k_dst = kv_smem + s * kv_stage_bytes, v_dst = k_dst + chunks * BKV * 128;
      const int kv0 = (tile_lo + i) * BKV;
      for (int pc = 0; pc < pieces; ++pc) {
        const int key = kv0 + pc * piece;
        const int lp = key / P;
        int page = lp < p.max_pages ? bt[lp] : -1;
        if (page < 0) page = 0;   // never visible to these queries (masked): any finite page will do
        const int row = (page * p.nkv + kvh) * P + key % P;
        for (int c = 0; c < chunks; ++c) {
          tma_load_2d(k_dst + c * BKV * 128 + pc * piece * 128, &map_k, c * 64, row, bar);
          tma_load_2d(v_dst + c * BKV * 128 + pc * piece * 128, &map_v, c * 64, row, bar);
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issue
    const uint32_t idesc_s = idesc_f16(BKV, 0), idesc_o = idesc_f16(hd, 1);
    bool ok = mbar_wait(bar_q, 0, ab);
    for (int i = 0; i < n_kv_tiles && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(bar_full0 + 8 * s, (i / STAGES) & 1, ab);
      if (!ok) break;
      tc_fence_after();
      const uint32_t k_src = kv_smem + s * kv_stage_bytes, v_src = k_src + chunks * BKV * 128;
      for (int k = 0; k < hd / 16; ++k) {      // S = Q K^T over the head dimension
        const uint32_t off = (k >> 2) * 128 * 128 + (k & 3) * 32;          // Q: 128 rows per chunk
        const uint32_t koff = (k >> 2) * BKV * 128 + (k & 3) * 32;         // K: 64 rows per chunk
        umma_bf16(tmem_s, smem_desc(q_smem + off), smem_desc(k_src + koff), idesc_s, k > 0 ? 1u : 0u);
      }
      umma_commit(bar_s);
      ok = mbar_wait(bar_p, i & 1, ab);         // P is in shared memory, S has been read
      if (!ok) break;
      tc_fence_after();
      for (int k = 0; k < BKV / 16; ++k) {      // O_tile = P V over the 64 keys
        // V [keys, hd] is MN-major for B: 16 keys down = 2048 bytes; 64-wide chunks of hd are BKV*128 apart
        const uint64_t vd = smem_desc_mn(v_src + k * 16 * 128, BKV * 128, 1024);
        umma_bf16(tmem_o, smem_desc(p_smem + k * 32), vd, idesc_o, k > 0 ? 1u : 0u);
      }
      umma_commit(bar_o);
      umma_commit(bar_empty0 + 8 * s);
    }
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- softmax rows
    const int q = warp & 3;
    const int r = q * 32 + lane;                    // row of the tile = TMEM lane
    const bool row_ok = r < n_rows;
    const int q_pos = pos0 + (row_ok ? r : n_rows - 1);
    const int first = p.window > 0 ? max(0, q_pos + 1 - p.window) : 0;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float o[HDM];
#pragma unroll
    for (int d = 0; d < HDM; ++d) o[d] = 0.f;
    float m = -1e30f, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_kv_tiles && ok; ++i) {
      ok = mbar_wait(bar_s, i & 1, ab);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = (tile_lo + i) * BKV;
      // pass 1: the row's maximum over this tile
      float mx = m;
#pragma unroll
      for (int c0 = 0; c0 < BKV; c0 += 16) {
        float v[16];
        tmem_ld16(tmem_s + lane_addr + c0, v);
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const int kj = kv0 + c0 + c;
          if (kj <= q_pos && kj >= first) mx = fmaxf(mx, v[c] * p.scale_log2);
        }
      }
      const float alpha = exp2f(m - mx);
      m = mx;
      // pass 2: probabilities, as bf16 into shared memory (row r, 16-byte unit u at (u ^ (r & 7)))
      float sum = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < BKV; c0 += 16) {
        float v[16];
        tmem_ld16(tmem_s + lane_addr + c0, v);
        uint32_t packed[8];
#pragma unroll
        for (int c = 0; c < 16; c += 2) {
          float pr[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kj = kv0 + c0 + c + e;
            pr[e] = (kj <= q_pos && kj >= first) ? exp2f(v[c + e] * p.scale_log2 - m) : 0.f;
          }
          const __nv_bfloat162 b = __floats2bfloat162_rn(pr[0], pr[1]);
          // the sum uses the rounded values that the MMA will see
          sum += __bfloat162float(b.x) + __bfloat162float(b.y);
          packed[c >> 1] = *reinterpret_cast<const uint32_t*>(&b);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int unit = (c0 >> 3) + u;
          const uint32_t addr = p_smem + r * 128 + ((unit ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[4 * u]), "r"(packed[4 * u + 1]),
                       "r"(packed[4 * u + 2]), "r"(packed[4 * u + 3]) : "memory");
        }
      }
      l = l * alpha + sum;
      // hand P to the tensor core: make this row's writes visible to the async proxy, then arrive
      // (the barrier counts all 128 rows; no thread waits on another here)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(bar_p);
      ok = mbar_wait(bar_o, i & 1, ab);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int d0 = 0; d0 < HDM; d0 += 16) {
        if (d0 < hd) {
          float v[16];
          tmem_ld16(tmem_o + lane_addr + d0, v);
#pragma unroll
          for (int d = 0; d < 16; ++d) o[d0 + d] = fmaf(o[d0 + d], alpha, v[d]);
        }
      }
      tc_fence_before();
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(row0 + r) * p.nq + head) * hd;
#pragma unroll
      for (int d0 = 0; d0 < HDM; d0 += 8) {
        if (d0 < hd) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(o[d0 + 2 * e] * inv, o[d0 + 2 * e + 1] * inv);
            w[e] = *reinterpret_cast<const uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(dst + d0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) {
      atomicExch(p.error_flag, 1);
      const long long t0 = clock64();
      while (clock64() - t0 < 200000) {}
    }
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, tmem_cols);
  }
}

}  // namespace

// q, out [T, nq*hd] bf16; k_cache, v_cache pages [n_pages, nkv, page_size, hd] bf16;
// tiles [n_tiles, 4] int32 on the device: first row, rows (1..128), request slot, position of the
// first row.  Rows of a tile are consecutive positions of one request.
extern "C" int flint_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, int n_pages,
                                          const int* block_table, int max_pages, int page_size, const int* tiles,
                                          int n_tiles, void* out, int T, int nq, int nkv, int hd, int window,
                                          float scale, int* error_flag, cudaStream_t stream) {
  if (n_tiles <= 0 || T <= 0) return 0;
  if (hd <= 0 || hd % 16 || hd > 128) return fail("attention_tc: head size %d (multiples of 16 up to 128)", hd);
  if (nkv <= 0 || nq % nkv) return fail("attention_tc: %d query heads do not divide into %d kv heads", nq, nkv);
  if (!(page_size > 0 && (BKV % page_size == 0 || page_size % BKV == 0)) || page_size % 8)
    return fail("attention_tc: page size %d must divide 64 or be a multiple of 64", page_size);
  if (n_tiles > 0x7fffffff / 4 || nq > 65535) return fail("attention_tc: too many tiles or heads");
  if (!error_flag) return fail("attention_tc: needs an error flag");
  if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15))
    return fail("attention_tc: operands must be 16-byte aligned");
  CUtensorMap mq, mk, mv;
  const long long kv_rows = (long long)n_pages * nkv * page_size;
  const int piece = page_size < BKV ? page_size : BKV;
  int rc = make_map_bf16(&mq, q, T, (long long)nq * hd, (long long)nq * hd, BQ);
  if (!rc) rc = make_map_bf16(&mk, k_cache, kv_rows, hd, hd, piece);
  if (!rc) rc = make_map_bf16(&mv, v_cache, kv_rows, hd, hd, piece);
  if (rc) return fail("attention_tc: cuTensorMapEncodeTiled failed (%d)", rc);
  Params p;
  p.tiles = tiles; p.block_table = block_table; p.out = (__nv_bfloat16*)out; p.error_flag = error_flag;
  p.max_pages = max_pages; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int chunks = (hd + 63) / 64;
  const size_t smem = (size_t)chunks * BQ * 128 + (size_t)STAGES * 2 * chunks * BKV * 128 + BQ * 128 + 1024;
  dim3 grid(n_tiles, nq);
  static bool configured[2] = {false, false};
  if (hd <= 64) {
    if (!configured[0]) {
      cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      configured[0] = true;
    }
    attention_prefill_tc_kernel<64><<<grid, THREADS, smem, stream>>>(mq, mk, mv, p);
  } else {
    if (!configured[1]) {
      cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      configured[1] = true;
    }
    attention_prefill_tc_kernel<128><<<grid, THREADS, smem, stream>>>(mq, mk, mv, p);
  }
  return check_launch("attention_prefill_tc");
}

extern "C" const char* flint_attention_tc_last_error() { return g_error; }
